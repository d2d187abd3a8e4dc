// Bindings of the low-latency dispatch/combine launchers (see kernels/ll_api.h).
// Parity: csrc/ops/low_latency.cpp:26-224 of the reference (layout probe, comm args, launch).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <stdexcept>
#include <string>

#include "kernels/ll_api.h"
#include "runtime/session.h"

namespace py = pybind11;
using namespace dep;

namespace {
void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    cudaGetLastError();
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
  }
}
template <class T> T* ptr(const py::dict& d, const char* key) {
  if (!d.contains(key) || d[key].is_none()) return nullptr;
  return reinterpret_cast<T*>(d[key].cast<uintptr_t>());
}
int geti(const py::dict& d, const char* key, int dflt = 0) { return d.contains(key) ? d[key].cast<int>() : dflt; }

void check_ll_shape(const WsLayout& lay) {
  if (lay.max_tokens > 256) throw std::invalid_argument("low-latency kernels serve at most 256 tokens per rank");
  if (lay.ll <= 0) throw std::invalid_argument("the workspace has no low-latency region");
}

void op_ll_dispatch(const WsLayout& lay, const std::vector<py::object>& sessions, const std::vector<py::dict>& args, int blocks,
                    uintptr_t stream, bool profile) {
  check_ll_shape(lay);
  LLDispatchParams p{};
  p.lay = lay;
  p.profile = profile ? 1 : 0;
  const int n = (int)args.size();
  if (n < 1 || n > kMaxRanks || (int)sessions.size() != n) throw std::invalid_argument("1..8 rank argument blocks expected");
  for (int i = 0; i < n; ++i) {
    const py::dict& d = args[i];
    LLDispatchArgs& a = p.r[i];
    Session& s = sessions[i].cast<Session&>();
    a.ctx = s.ctx();
    a.x = ptr<const void>(d, "x"); a.x_sf = ptr<const float>(d, "x_sf");
    a.topk_idx = ptr<const long long>(d, "topk_idx"); a.topk_w = ptr<const float>(d, "topk_w");
    a.T = geti(d, "T"); a.E = geti(d, "E"); a.mode = geti(d, "mode");
    a.recv_x = ptr<void>(d, "recv_x"); a.recv_sf = ptr<float>(d, "recv_sf"); a.recv_w = ptr<float>(d, "recv_w");
    a.recv_row_src = ptr<int>(d, "recv_row_src"); a.expert_counts = ptr<int>(d, "expert_counts");
    a.expert_offsets = ptr<int>(d, "expert_offsets"); a.num_rows = ptr<int>(d, "num_rows");
    a.mailbox = geti(d, "use_mailbox", 0) ? s.mailbox_device() : nullptr;
    a.capacity = d["capacity"].cast<long long>();
    if (a.T < 0 || a.T > lay.max_tokens) throw std::invalid_argument("token count exceeds num_max_tokens_per_rank");
    if (a.E < a.ctx.world || a.E > kMaxExperts || a.E % a.ctx.world) throw std::invalid_argument("num_experts must be a multiple of the world size and at most 1024");
    if (a.mode != 0 && lay.hidden % 128) throw std::invalid_argument("fp8 dispatch needs hidden % 128 == 0");
  }
  check(launch_ll_dispatch(p, n, blocks, reinterpret_cast<cudaStream_t>(stream)), "ep_dispatch_ll launch");
}

void op_ll_combine(const WsLayout& lay, const std::vector<py::object>& sessions, const std::vector<py::dict>& args, int blocks,
                   uintptr_t stream, bool profile) {
  check_ll_shape(lay);
  LLCombineParams p{};
  p.lay = lay;
  p.profile = profile ? 1 : 0;
  const int n = (int)args.size();
  if (n < 1 || n > kMaxRanks || (int)sessions.size() != n) throw std::invalid_argument("1..8 rank argument blocks expected");
  for (int i = 0; i < n; ++i) {
    const py::dict& d = args[i];
    LLCombineArgs& a = p.r[i];
    a.ctx = sessions[i].cast<Session&>().ctx();
    a.x = ptr<const __nv_bfloat16>(d, "x"); a.recv_row_src = ptr<const int>(d, "recv_row_src");
    a.num_rows = ptr<const int>(d, "num_rows"); a.topk_idx = ptr<const long long>(d, "topk_idx");
    a.topk_w = ptr<const float>(d, "topk_w"); a.T = geti(d, "T"); a.E = geti(d, "E");
    a.out = ptr<__nv_bfloat16>(d, "out");
  }
  check(launch_ll_combine(p, n, blocks, reinterpret_cast<cudaStream_t>(stream)), "ep_combine_ll launch");
}
}  // namespace

void bind_low_latency(py::module_& m) {
  m.def("ll_region_bytes", &ll_region_bytes, py::arg("world"), py::arg("max_tokens"), py::arg("topk"), py::arg("hidden"));
  m.def("ll_dispatch", &op_ll_dispatch, py::arg("layout"), py::arg("sessions"), py::arg("args"), py::arg("blocks"), py::arg("stream"),
        py::arg("profile") = false);
  m.def("ll_combine", &op_ll_combine, py::arg("layout"), py::arg("sessions"), py::arg("args"), py::arg("blocks"), py::arg("stream"),
        py::arg("profile") = false);
}
