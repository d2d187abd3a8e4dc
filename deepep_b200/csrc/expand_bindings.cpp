// Python bindings of the local expand / aggregate operators.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <stdexcept>
#include <string>

#include "kernels/expand_api.h"

namespace py = pybind11;
using namespace dep;

namespace {
template <class T> T* eptr(const py::dict& d, const char* key) {
  if (!d.contains(key) || d[key].is_none()) return nullptr;
  return reinterpret_cast<T*>(d[key].cast<uintptr_t>());
}
void check_launch(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
}  // namespace

void bind_expand(py::module_& m) {
  m.attr("expand_tile") = kExpandTile;
  m.def("expand", [](const py::dict& d, int blocks, uintptr_t stream) {
    ExpandParams p{};
    p.x = eptr<const uint8_t>(d, "x"); p.x_sf = eptr<const float>(d, "x_sf");
    p.topk_idx = eptr<const long long>(d, "topk_idx"); p.topk_w = eptr<const float>(d, "topk_w");
    p.out = eptr<uint8_t>(d, "out"); p.out_sf = eptr<float>(d, "out_sf"); p.out_w = eptr<float>(d, "out_w");
    p.expert_offsets = eptr<int>(d, "expert_offsets"); p.actual_counts = eptr<int>(d, "actual_counts");
    p.mapping = eptr<int>(d, "mapping"); p.tile_counts = eptr<int>(d, "tile_counts"); p.error_flag = eptr<int>(d, "err");
    p.R = d["rows"].cast<int>(); p.K = d["topk"].cast<int>(); p.L = d["experts"].cast<int>(); p.N = d["expanded_rows"].cast<int>();
    p.row_bytes = d["row_bytes"].cast<int>(); p.num_sf = d["num_sf"].cast<int>(); p.cached = d["cached"].cast<int>();
    if (p.K < 1 || p.K > kMaxTopk) throw std::invalid_argument("num_topk must be in [1, 16]");
    if (p.L < 1 || p.L > kMaxExperts) throw std::invalid_argument("1..1024 local experts are supported");
    if (p.row_bytes <= 0 || p.row_bytes % 16) throw std::invalid_argument("a row must be a positive multiple of 16 bytes");
    if (p.R < 0 || p.N < 0) throw std::invalid_argument("negative row count");
    if (!p.expert_offsets || !p.actual_counts || !p.error_flag || (p.R > 0 && (!p.x || !p.mapping)) || (p.N > 0 && !p.out))
      throw std::invalid_argument("missing tensor");
    if (!p.cached && p.R > 0 && (!p.topk_idx || !p.tile_counts)) throw std::invalid_argument("expand needs topk_idx and its scratch");
    if ((p.x_sf == nullptr) != (p.out_sf == nullptr)) throw std::invalid_argument("scales need an input and an output");
    check_launch(launch_expand(p, blocks, reinterpret_cast<cudaStream_t>(stream)), "expand launch");
  });
  m.def("aggregate", [](const py::dict& d, int blocks, uintptr_t stream) {
    AggregateParams p{};
    p.x = eptr<const uint8_t>(d, "x"); p.row_w = eptr<const float>(d, "row_w"); p.values = eptr<const float>(d, "values");
    p.mapping = eptr<const int>(d, "mapping"); p.out = eptr<uint8_t>(d, "out"); p.out_values = eptr<float>(d, "out_values");
    p.R = d["rows"].cast<int>(); p.K = d["topk"].cast<int>(); p.H = d["hidden"].cast<int>(); p.N = d["expanded_rows"].cast<int>();
    p.is_half = d["is_half"].cast<int>();
    if (p.K < 1 || p.K > kMaxTopk) throw std::invalid_argument("num_topk must be in [1, 16]");
    if (p.H <= 0 || p.H % 8) throw std::invalid_argument("hidden must be a positive multiple of 8");
    if (p.R > 0 && (!p.mapping || !p.out || (p.N > 0 && !p.x))) throw std::invalid_argument("missing tensor");
    if (p.R == 0) return;
    check_launch(launch_aggregate(p, blocks, reinterpret_cast<cudaStream_t>(stream)), "aggregate launch");
  });
}
