// Python bindings of the all-to-all-v + grouped GEMM ops (argument validation, tensor maps, launch).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <stdexcept>
#include <string>
#include <vector>

#include "kernels/gmm_api.h"
#include "runtime/session.h"

namespace py = pybind11;
using namespace dep;

namespace {
template <class T> T* gptr(const py::dict& d, const char* key) {
  if (!d.contains(key) || d[key].is_none()) return nullptr;
  return reinterpret_cast<T*>(d[key].cast<uintptr_t>());
}
int gint(const py::dict& d, const char* key) { return d[key].cast<int>(); }

// `gather` = true: a2av_gmm (A operand is the gathered buffer); false: gmm_a2av (A operand is x).
void fill(GmmArgs& a, const WsLayout& lay, const py::dict& d, py::object session, bool gather) {
  Session& s = session.cast<Session&>();
  a.ctx = s.ctx();
  const long long max_rows = d["max_rows"].cast<long long>(), max_k = d["max_k"].cast<long long>(), max_n = d["max_n"].cast<long long>();
  const GmmRegion g = gmm_region(max_rows, max_k, max_n);
  if (lay.mega + g.total > lay.total) throw std::invalid_argument("the workspace is smaller than the GMM region");
  a.table_off = lay.mega + (gather ? g.table_a : g.table_b);
  a.data_off = lay.mega + (gather ? g.stage : g.recv);
  a.x = gptr<const __nv_bfloat16>(d, "x");
  a.counts = gptr<const int>(d, "counts");
  a.out = gptr<__nv_bfloat16>(d, "out");
  a.gathered = gptr<__nv_bfloat16>(d, "gathered");
  a.rows_in = gint(d, "rows_in"); a.E = gint(d, "experts"); a.K = gint(d, "k"); a.N = gint(d, "n");
  a.out_rows_cap = gint(d, "out_rows_cap"); a.gathered_cap = gather ? gint(d, "gathered_cap") : a.rows_in;
  a.max_tiles = gint(d, "max_tiles");
  a.tile_info = gptr<int>(d, "tile_info"); a.num_tiles = gptr<int>(d, "num_tiles"); a.pulled = gptr<int>(d, "pulled");
  a.error_flag = gptr<int>(d, "err");
  if (a.E < 1 || a.E > kMaxExperts || a.E % a.ctx.world) throw std::invalid_argument("experts must be in [1, 1024] and divisible by the world size");
  if (a.K < kGmmBK || a.K % kGmmBK || a.N < 64 || a.N % 64) throw std::invalid_argument("k and n must be positive multiples of 64");
  if (a.K > max_k || a.N > max_n) throw std::invalid_argument("k or n exceeds what the group was sized for");
  if (a.rows_in < 0 || a.out_rows_cap < 0) throw std::invalid_argument("negative row count");
  if ((gather ? a.rows_in : a.out_rows_cap) > max_rows) throw std::invalid_argument("more rows than the group was sized for");
  if (!a.counts || (a.out_rows_cap > 0 && !a.out) || !a.tile_info || !a.num_tiles || (a.rows_in > 0 && !a.x) || (gather && (!a.gathered || !a.pulled)))
    throw std::invalid_argument("missing tensor");
  const char* err = nullptr;
  const void* a_base = gather ? (const void*)a.gathered : (const void*)a.x;
  const long long a_rows = gather ? a.gathered_cap : a.rows_in;
  // an empty operand still needs a valid map: point it at the weights
  if (!encode_bf16_map(&a.tmap_a, a_rows > 0 ? a_base : (const void*)d["weight"].cast<uintptr_t>(), a_rows > 0 ? a_rows : 1, a.K, kGmmBM, &err))
    throw std::runtime_error(err);
  const long long L = a.E / a.ctx.world;
  if (!encode_bf16_map(&a.tmap_b, gptr<const void>(d, "weight"), L * a.K, a.N, kGmmBK, &err)) throw std::runtime_error(err);
}

void op(const WsLayout& lay, const std::vector<py::object>& sessions, const std::vector<py::dict>& args, int blocks, uintptr_t stream,
        bool gather) {
  GmmParams p{};
  p.lay = lay;
  const int n = (int)args.size();
  if (n < 1 || n > kMaxRanks || (int)sessions.size() != n) throw std::invalid_argument("1..8 rank argument blocks expected");
  for (int i = 0; i < n; ++i) fill(p.r[i], lay, args[i], sessions[i], gather);
  const cudaError_t e = gather ? launch_a2av_gmm(p, n, blocks, reinterpret_cast<cudaStream_t>(stream))
                               : launch_gmm_a2av(p, n, blocks, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) throw std::runtime_error(std::string(gather ? "a2av_gmm" : "gmm_a2av") + " launch: " + cudaGetErrorString(e));
}
}  // namespace

void bind_gmm(py::module_& m) {
  m.def("gmm_region_offsets", [](long long max_rows, long long max_k, long long max_n) {
    const GmmRegion g = gmm_region(max_rows, max_k, max_n);
    return std::vector<long long>{g.table_a, g.table_b, g.stage, g.recv, g.total};
  });
  m.def("gmm_region_bytes", [](long long max_rows, long long max_k, long long max_n) { return gmm_region(max_rows, max_k, max_n).total; });
  m.def("a2av_gmm", [](const WsLayout& lay, const std::vector<py::object>& sessions, const std::vector<py::dict>& args, int blocks,
                       uintptr_t stream) { op(lay, sessions, args, blocks, stream, true); });
  m.def("gmm_a2av", [](const WsLayout& lay, const std::vector<py::object>& sessions, const std::vector<py::dict>& args, int blocks,
                       uintptr_t stream) { op(lay, sessions, args, blocks, stream, false); });
}
