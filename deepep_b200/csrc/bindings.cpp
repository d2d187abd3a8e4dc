// Python module `deepep_b200._C`: sessions, workspace layout and kernel launchers.
//
// Parity: csrc/bindings/module.cpp:17-95 of the reference (runtime factories + the
// notify/dispatch/combine/low-latency op families, `runtime_protocol`).  Tensors cross this
// boundary as raw device addresses (`tensor.data_ptr()`), so the module needs no libtorch.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <stdexcept>
#include <string>

#include "kernels/api.h"
#include "kernels/ll_api.h"
#include "kernels/mega_api.h"
#include "kernels/ws_layout.h"
#include "runtime/fake_cuda.h"
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
long long getl(const py::dict& d, const char* key, long long dflt = 0) { return d.contains(key) ? d[key].cast<long long>() : dflt; }

RankCtx ctx_of(const py::handle& session) { return session.cast<Session&>().ctx(); }

void op_notify(const WsLayout& lay, const std::vector<py::object>& sessions, const std::vector<py::dict>& args, int blocks,
               uintptr_t stream, bool profile) {
  NotifyParams p{};
  p.lay = lay;
  p.profile = profile ? 1 : 0;
  const int n = (int)args.size();
  if (n < 1 || n > kMaxRanks || (int)sessions.size() != n) throw std::invalid_argument("1..8 rank argument blocks expected");
  for (int i = 0; i < n; ++i) {
    const py::dict& d = args[i];
    NotifyArgs& a = p.r[i];
    a.ctx = ctx_of(sessions[i]);
    a.topk_idx = ptr<const long long>(d, "topk_idx");
    a.topk_w = ptr<const float>(d, "topk_w");
    a.T = geti(d, "T"); a.E = geti(d, "E"); a.K = geti(d, "K");
    a.expand = geti(d, "expand", 1); a.alignment = geti(d, "alignment", 1); a.meta_stride = geti(d, "meta_stride");
    a.hist = ptr<int>(d, "hist"); a.hits = ptr<int>(d, "hits"); a.own_hits = ptr<int>(d, "own_hits"); a.cnt = ptr<int>(d, "cnt");
    a.send_slot = ptr<int>(d, "send_slot"); a.slot_row = ptr<int>(d, "slot_row"); a.stage_meta = ptr<int>(d, "stage_meta");
    a.chunk_start = ptr<int>(d, "chunk_start"); a.rank_tokens = ptr<int>(d, "rank_tokens"); a.rank_rows = ptr<int>(d, "rank_rows");
    a.expert_counts = ptr<int>(d, "expert_counts"); a.expert_offsets = ptr<int>(d, "expert_offsets");
    a.recv_row_src = ptr<int>(d, "recv_row_src"); a.recv_w = ptr<float>(d, "recv_w"); a.recv_idx = ptr<long long>(d, "recv_idx");
    a.rank_matrix = ptr<int>(d, "rank_matrix");
    a.mailbox = sessions[i].cast<Session&>().mailbox_device();
    a.rcap = getl(d, "rcap");
    if (a.T < 0 || a.T > lay.max_tokens) throw std::invalid_argument("token count exceeds num_max_tokens_per_rank");
    if (a.K != lay.topk) throw std::invalid_argument("top-k width differs from the buffer's num_topk");
    if (a.E < a.ctx.world || a.E > kMaxExperts || a.E % a.ctx.world) throw std::invalid_argument("num_experts must be a multiple of the world size and at most 1024");
    if (a.alignment < 1) throw std::invalid_argument("expert_alignment must be positive");
  }
  check(launch_notify(p, n, blocks, reinterpret_cast<cudaStream_t>(stream)), "ep_notify launch");
}

void op_dispatch(const WsLayout& lay, const std::vector<py::object>& sessions, const std::vector<py::dict>& args, int send_blocks,
                 int recv_blocks, uintptr_t stream, bool local_direct, bool profile) {
  DispatchParams p{};
  p.lay = lay; p.send_blocks = send_blocks; p.recv_blocks = recv_blocks; p.local_direct = local_direct; p.profile = profile;
  const int n = (int)args.size();
  if (n < 1 || n > kMaxRanks || (int)sessions.size() != n) throw std::invalid_argument("1..8 rank argument blocks expected");
  if (send_blocks < 1 || recv_blocks < 0) throw std::invalid_argument("the sender block count must be positive, the receiver count nonnegative");
  if (recv_blocks == 0 && !(local_direct && lay.world == 1))
    throw std::invalid_argument("receiver blocks are only optional for one rank that writes its own rows directly");
  for (int i = 0; i < n; ++i) {
    const py::dict& d = args[i];
    DispatchArgs& a = p.r[i];
    a.ctx = ctx_of(sessions[i]);
    a.x = ptr<const void>(d, "x"); a.x_sf = ptr<const float>(d, "x_sf");
    a.T = geti(d, "T"); a.mode = geti(d, "mode");
    a.send_slot = ptr<const int>(d, "send_slot"); a.stage_meta = ptr<const int>(d, "stage_meta");
    a.slot_row = ptr<const int>(d, "slot_row"); a.topk_idx = ptr<const long long>(d, "topk_idx");
    a.rank_tokens = ptr<const int>(d, "rank_tokens"); a.rank_rows = ptr<const int>(d, "rank_rows");
    a.meta_stride = geti(d, "meta_stride");
    a.recv_rows = geti(d, "recv_rows", 0);
    a.K = geti(d, "K"); a.E = geti(d, "E"); a.expand = geti(d, "expand", 1);
    a.recv_x = ptr<void>(d, "recv_x"); a.recv_sf = ptr<float>(d, "recv_sf");
    a.prof = ptr<unsigned long long>(d, "prof");
    // (a rank without tokens, or without received rows, passes empty tensors whose address is null)
    if (!a.send_slot || !a.stage_meta || !a.rank_tokens || !a.rank_rows || (!a.x && a.T > 0))
      throw std::invalid_argument("dispatch: a required pointer is missing");
    if (local_direct && (!a.slot_row || (!a.topk_idx && a.T > 0) || a.E < a.ctx.world || a.K != lay.topk))
      throw std::invalid_argument("dispatch: direct local rows need slot_row, topk_idx, E and K");
    if (a.mode != p.r[0].mode) throw std::invalid_argument("all ranks must use the same dispatch mode");
    if (a.mode != kDispatchBf16 && lay.hidden % 128) throw std::invalid_argument("fp8 dispatch needs hidden % 128 == 0");
  }
  check(launch_dispatch(p, n, reinterpret_cast<cudaStream_t>(stream)), "ep_dispatch_ht launch");
}

void op_combine(const WsLayout& lay, const std::vector<py::object>& sessions, const std::vector<py::dict>& args, int send_blocks,
                int recv_blocks, uintptr_t stream, bool local_direct, bool profile, int t_begin, int t_end) {
  CombineParams p{};
  p.lay = lay; p.send_blocks = send_blocks; p.recv_blocks = recv_blocks; p.local_direct = local_direct; p.profile = profile;
  p.t_begin = t_begin; p.t_end = t_end < 0 ? lay.max_tokens : t_end;
  if (p.t_begin < 0 || p.t_end < p.t_begin || p.t_end - p.t_begin > lay.partial_tokens)
    throw std::invalid_argument("combine: the token window does not fit the workspace's partial area");
  const int n = (int)args.size();
  if (n < 1 || n > kMaxRanks || (int)sessions.size() != n) throw std::invalid_argument("1..8 rank argument blocks expected");
  if (send_blocks < 0 || recv_blocks < 1) throw std::invalid_argument("the source-side block count must be positive, the expert-side count nonnegative");
  if (send_blocks == 0 && !(local_direct && lay.world == 1))
    throw std::invalid_argument("expert-side blocks are only optional for one rank that reads its own rows directly");
  for (int i = 0; i < n; ++i) {
    const py::dict& d = args[i];
    CombineArgs& a = p.r[i];
    a.ctx = ctx_of(sessions[i]);
    a.x = ptr<const __nv_bfloat16>(d, "x"); a.w = ptr<const float>(d, "w");
    a.stage_meta = ptr<const int>(d, "stage_meta"); a.rank_rows = ptr<const int>(d, "rank_rows");
    a.rank_tokens = ptr<const int>(d, "rank_tokens"); a.send_slot = ptr<const int>(d, "send_slot");
    a.topk_idx = ptr<const long long>(d, "topk_idx");
    a.T = geti(d, "T"); a.meta_stride = geti(d, "meta_stride"); a.K = geti(d, "K"); a.E = geti(d, "E"); a.expand = geti(d, "expand", 1);
    a.x_rows = geti(d, "x_rows", 0);
    a.bias0 = ptr<const __nv_bfloat16>(d, "bias0"); a.bias1 = ptr<const __nv_bfloat16>(d, "bias1");
    a.out = ptr<__nv_bfloat16>(d, "out"); a.out_w = ptr<float>(d, "out_w");
    a.prof = ptr<unsigned long long>(d, "prof");
    if (!a.stage_meta || !a.rank_rows || !a.rank_tokens || !a.send_slot || ((!a.topk_idx || !a.out) && a.T > 0))
      throw std::invalid_argument("combine: a required pointer is missing");
    if (a.E < a.ctx.world) throw std::invalid_argument("combine: num_experts is missing");
  }
  check(launch_combine(p, n, reinterpret_cast<cudaStream_t>(stream)), "ep_combine_ht launch");
}

void op_barrier(const std::vector<py::object>& sessions, uintptr_t stream) {
  BarrierParams p{};
  const int n = (int)sessions.size();
  if (n < 1 || n > kMaxRanks) throw std::invalid_argument("1..8 sessions expected");
  for (int i = 0; i < n; ++i) p.r[i] = ctx_of(sessions[i]);
  check(launch_barrier(p, n, reinterpret_cast<cudaStream_t>(stream)), "ep_barrier launch");
}

}  // namespace

void bind_low_latency(py::module_& m);
void bind_mega(py::module_& m);
void bind_gmm(py::module_& m);
void bind_expand(py::module_& m);

PYBIND11_MODULE(_C, m) {
  m.attr("runtime_protocol") = 1;
  m.attr("max_ranks") = kMaxRanks;
  m.attr("chunk_tokens") = kChunkTokens;
  m.attr("max_topk") = kMaxTopk;
  m.attr("max_experts") = kMaxExperts;
  m.attr("control_bytes") = (long long)kControlBytes;
  m.attr("row_slot_shift") = kRowSlotShift;
  m.attr("control_dbg_offset") = (long long)offsetof(Control, dbg);
#ifdef DEEPEP_DEBUG_BOUNDS
  m.attr("debug_bounds") = true;
#else
  m.attr("debug_bounds") = false;
#endif

  py::class_<WsLayout>(m, "WsLayout")
      .def_readonly("gather_hdr", &WsLayout::gather_hdr).def_readonly("gather_idx", &WsLayout::gather_idx)
      .def_readonly("gather_w", &WsLayout::gather_w).def_readonly("stage", &WsLayout::stage)
      .def_readonly("partial", &WsLayout::partial).def_readonly("wret", &WsLayout::wret)
      .def_readonly("disp_flag", &WsLayout::disp_flag).def_readonly("comb_flag", &WsLayout::comb_flag)
      .def_readonly("ll", &WsLayout::ll).def_readonly("mega", &WsLayout::mega).def_readonly("total", &WsLayout::total)
      .def_readonly("max_tokens", &WsLayout::max_tokens).def_readonly("hidden", &WsLayout::hidden)
      .def_readonly("topk", &WsLayout::topk).def_readonly("world", &WsLayout::world)
      .def_readonly("stage_row_bytes", &WsLayout::stage_row_bytes).def_readonly("partial_tokens", &WsLayout::partial_tokens);
  m.def("make_mega_layout", &make_mega_layout);
  m.def("make_layout", &make_layout, py::arg("world"), py::arg("max_tokens"), py::arg("hidden"), py::arg("topk"),
        py::arg("ll_bytes") = 0, py::arg("mega_bytes") = 0, py::arg("partial_tokens") = 0);

  py::class_<Session>(m, "Session")
      .def(py::init<int, int, size_t, double, const std::string&>(), py::arg("rank"), py::arg("world"), py::arg("bytes"),
           py::arg("timeout"), py::arg("transport") = "auto")
      .def_property_readonly("transport", [](const Session& s) { return std::string(s.transport()); })
      .def("ipc_handle", [](const Session& s) { return py::bytes(s.ipc_handle()); })
      .def("export_fd", &Session::export_fd)
      .def("open_peer_fds", &Session::open_peer_fds)
      .def("close_peers", &Session::close_peers)
      .def("open_peers", [](Session& s, const std::vector<py::bytes>& hs) {
        std::vector<std::string> v;
        for (const auto& h : hs) v.push_back(std::string(h));
        s.open_peers(v);
      })
      .def("attach_peers", &Session::attach_peers)
      .def("close", &Session::close)
      .def("set_timeout", &Session::set_timeout)
      .def("clear_status", &Session::clear_status)
      .def("read_control", [](const Session& s) { return py::bytes(s.read_control()); })
      .def("guard_intact", &Session::guard_intact)
      .def("mapped", &Session::mapped)
      .def("peer", &Session::peer)
      .def_property_readonly("workspace", &Session::workspace)
      .def_property_readonly("bytes", &Session::bytes)
      .def_property_readonly("rank", &Session::rank)
      .def_property_readonly("world", &Session::world)
      .def_property_readonly("instance_id", &Session::instance_id)
      .def_property_readonly("poisoned", &Session::poisoned)
      .def_property_readonly("closed", &Session::closed)
      .def("status", [](const Session& s) {
        StatusBlock b = s.status();
        py::dict d;
        d["code"] = b.code; d["op"] = b.op; d["rank"] = b.rank; d["peer"] = b.peer; d["where"] = b.where;
        d["expected"] = b.expected; d["seen"] = b.seen;
        return d;
      })
      .def("mailbox", [](const Session& s, int n) {
        std::vector<int> v(s.mailbox_host(), s.mailbox_host() + std::min(n, kMailboxInts));
        return v;
      })
      .def("wait_probe", [](Session& s, uintptr_t stream) {
        check(launch_wait_probe(s.ctx(), reinterpret_cast<cudaStream_t>(stream)), "wait probe launch");
      });
  m.def("live_instances", &live_instances);
  m.def("vmm_supported", &vmm_supported_here);
  // host-memory doubles of the CUDA entry points behind the session (fault-injection tests; never used by the library itself)
  m.def("testing_install_fake_cuda", &fake::install, py::arg("vmm_supported") = true);
  m.def("testing_restore_cuda", &fake::restore);
  m.def("testing_fail", &fake::fail, py::arg("entry"), py::arg("nth") = 0, py::arg("code") = 1);
  m.def("testing_log", &fake::log);
  m.def("testing_clear", &fake::clear);
  m.def("testing_open_allocations", &fake::open_allocations);
  m.def("testing_poke", [](uintptr_t address, int value) { *reinterpret_cast<volatile int*>(address) = value; });
  m.def("testing_peek", [](uintptr_t address) { return *reinterpret_cast<volatile int*>(address); });

  m.def("layout", [](uintptr_t topk_idx, int T, int K, int E, int P, uintptr_t per_rank, uintptr_t per_expert, uintptr_t in_rank,
                     uintptr_t stream) {
    check(launch_layout(reinterpret_cast<const long long*>(topk_idx), T, K, E, P, reinterpret_cast<int*>(per_rank),
                        reinterpret_cast<int*>(per_expert), reinterpret_cast<bool*>(in_rank), reinterpret_cast<cudaStream_t>(stream)),
          "ep_layout launch");
  });
  m.def("notify", &op_notify, py::arg("layout"), py::arg("sessions"), py::arg("args"), py::arg("blocks"), py::arg("stream"),
        py::arg("profile") = false);
  m.def("dispatch", &op_dispatch, py::arg("layout"), py::arg("sessions"), py::arg("args"), py::arg("send_blocks"),
        py::arg("recv_blocks"), py::arg("stream"), py::arg("local_direct") = true, py::arg("profile") = false);
  m.def("combine", &op_combine, py::arg("layout"), py::arg("sessions"), py::arg("args"), py::arg("send_blocks"),
        py::arg("recv_blocks"), py::arg("stream"), py::arg("local_direct") = true, py::arg("profile") = false,
        py::arg("t_begin") = 0, py::arg("t_end") = -1);
  m.attr("group_tokens") = kGroupTokens;
  m.attr("row_block") = kRowBlock;
  m.attr("dispatch_prof_words") = kDispatchProfWords;
  m.attr("dispatch_threads") = kDispatchThreads;
  m.attr("combine_threads") = kCombineThreads;
  m.attr("combine_prof_words") = kCombineProfWords;
  m.def("barrier", &op_barrier);
  bind_low_latency(m);
  bind_mega(m);
  bind_gmm(m);
  bind_expand(m);
}
