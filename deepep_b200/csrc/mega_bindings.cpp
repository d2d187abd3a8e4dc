// Bindings of the fused-MoE kernels (see kernels/mega_api.h).
// Parity: experiments/megamoe/csrc/bindings.cpp:11-29 and forward.cpp:295-478 of the reference.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <stdexcept>
#include <string>

#include "kernels/mega_api.h"
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

// One grouped GEMM launch.  `d` carries operand pointers and shapes; `session` is needed only by the
// combine epilogue (peer workspaces).
void fill_gemm(MegaGemmParams& p, const py::dict& d, py::object session) {
  const long long rows_pad = getl(d, "rows_pad"), k = getl(d, "k"), b_rows = getl(d, "b_rows");
  if (rows_pad % kGemmBM || k % kGemmBK || b_rows % kGemmBN) throw std::invalid_argument("rows and K must be multiples of 128, weight rows of 256");
  const char* err = nullptr;
  if (!encode_operand_map(&p.tmap_a, ptr<const void>(d, "a"), rows_pad, k, false, &err)) throw std::runtime_error(err);
  // weights are stored tiled: every (128-row, 128-K) block is one contiguous run of 128 rows x 64 (e2m1) or 128 (e4m3) bytes
  p.b_fp8 = geti(d, "b_fp8", 0) ? 1 : 0;
  if (!encode_operand_map(&p.tmap_b, ptr<const void>(d, "b"), b_rows * (k / kGemmBK), kGemmBK, !p.b_fp8, &err)) throw std::runtime_error(err);
  p.sfa = ptr<const uint8_t>(d, "sfa"); p.sfb = ptr<const uint8_t>(d, "sfb");
  if (!encode_sf_map(&p.tmap_sfa, p.sfa, (rows_pad / kGemmBM) * (k / kGemmBK), &err)) throw std::runtime_error(err);
  if (!encode_sf_map(&p.tmap_sfb, p.sfb, (b_rows / 128) * (k / kGemmBK), &err)) throw std::runtime_error(err);
  p.mtile_expert = ptr<const int>(d, "mtile_expert"); p.num_mtiles = ptr<const int>(d, "num_mtiles");
  p.a_ready = ptr<const int>(d, "a_ready");
  p.max_mtiles = (int)(rows_pad / kGemmBM);
  p.n_total = geti(d, "n_total"); p.n_tiles = p.n_total / kGemmBN; p.k_steps = (int)(k / kGemmBK);
  if (p.n_total % kGemmBN) throw std::invalid_argument("output width must be a multiple of 256");
  p.epi = geti(d, "epi");
  p.pair = geti(d, "pair", 0) ? 1 : 0;
  p.stages = geti(d, "stages", 0); p.commit_every = geti(d, "commit_every", 0);
  if (p.stages < 0 || p.stages > kGemmMaxStagesHost || p.stages == 1 || p.commit_every < 0 || p.commit_every > 2)
    throw std::invalid_argument("stages must be 0 or 2..6, commit_every 0, 1 or 2");
  p.b_tx_bytes = geti(d, "b_tx_bytes", p.b_fp8 ? 128 * kGemmBK : 128 * kGemmBK / 2);   // bytes counted per 128-row box of weights
  p.c = ptr<float>(d, "c"); p.ldc = geti(d, "ldc");
  p.a2 = ptr<uint8_t>(d, "a2"); p.a2_sf = ptr<uint8_t>(d, "a2_sf"); p.inter = geti(d, "inter");
  p.row_src = ptr<const int>(d, "row_src");
  p.comb_off = getl(d, "comb_off"); p.max_tokens = geti(d, "max_tokens"); p.topk = geti(d, "topk"); p.hidden = geti(d, "hidden");
  p.error_flag = ptr<int>(d, "error_flag");
  p.debug = ptr<long long>(d, "debug");
  if (p.epi == kEpiCombine) {
    RankCtx ctx = session.cast<Session&>().ctx();
    for (int r = 0; r < ctx.world; ++r) p.ws[r] = ctx.ws[r];
  }
}

void op_mega_gemm(const py::dict& d, py::object session, int blocks, uintptr_t stream) {
  MegaGemmParams p{};
  fill_gemm(p, d, session);
  check(launch_mega_gemm(p, blocks, reinterpret_cast<cudaStream_t>(stream)), "mega_gemm launch");
}

void fill_route(MegaRouteArgs& a, const py::dict& d, py::object session) {
  a.ctx = session.cast<Session&>().ctx();
  a.in_off = getl(d, "in_off"); a.T = geti(d, "T"); a.E = geti(d, "E"); a.K = geti(d, "K"); a.H = geti(d, "H");
  a.max_tokens = geti(d, "max_tokens"); a.max_mtiles = geti(d, "max_mtiles");
  a.a1 = ptr<uint8_t>(d, "a1"); a.a1_sf = ptr<uint8_t>(d, "a1_sf"); a.row_src = ptr<int>(d, "row_src");
  a.mtile_expert = ptr<int>(d, "mtile_expert"); a.num_mtiles = ptr<int>(d, "num_mtiles");
  a.expert_rows = ptr<int>(d, "expert_rows"); a.expert_list = ptr<int>(d, "expert_list");
  a.pulled = ptr<int>(d, "pulled");
  a.S = geti(d, "S", 0);
  a.tile_pairs = geti(d, "tile_pairs", 0) ? 1 : 0;
  a.x_bf16 = ptr<const __nv_bfloat16>(d, "x_bf16");
  a.timer = ptr<unsigned long long>(d, "timer");
  if (a.S < 0 || a.K + a.S > kMaxTopk || a.E / a.ctx.world + a.S > kMaxExperts)
    throw std::invalid_argument("top-k plus shared experts must not exceed 16, local plus shared experts 1024");
  if (a.H % 128 || a.E % a.ctx.world || a.E > kMaxExperts) throw std::invalid_argument("hidden % 128 == 0 and experts % world == 0 are required");
}

void fill_finish(MegaFinishArgs& a, const py::dict& d, py::object session) {
  a.ctx = session.cast<Session&>().ctx();
  a.in_off = getl(d, "in_off"); a.comb_off = getl(d, "comb_off");
  a.T = geti(d, "T"); a.E = geti(d, "E"); a.K = geti(d, "K"); a.H = geti(d, "H"); a.max_tokens = geti(d, "max_tokens");
  a.y = ptr<__nv_bfloat16>(d, "y");
  a.S = geti(d, "S", 0);
  a.timer = ptr<unsigned long long>(d, "timer");
}

// One persistent launch for the whole layer: args[i] = {"route": {...}, "gemm1": {...}, "gemm2": {...}, "finish": {...}, "ready": ptr}
void op_mega_fused(const WsLayout& lay, const std::vector<py::object>& sessions, const std::vector<py::dict>& args, int blocks,
                   uintptr_t stream) {
  static MegaFusedParams p;   // ~10 KB: kept off the stack; launches are issued by one thread at a time under the GIL
  p = MegaFusedParams{};
  p.lay = lay;
  const int n = (int)args.size();
  if (n < 1 || n > kMaxRanks || (int)sessions.size() != n) throw std::invalid_argument("1..8 rank argument blocks expected");
  for (int i = 0; i < n; ++i) {
    const py::dict& d = args[i];
    fill_route(p.r[i].route, d["route"].cast<py::dict>(), sessions[i]);
    fill_finish(p.r[i].finish, d["finish"].cast<py::dict>(), sessions[i]);
    fill_gemm(p.r[i].g1, d["gemm1"].cast<py::dict>(), sessions[i]);
    fill_gemm(p.r[i].g2, d["gemm2"].cast<py::dict>(), sessions[i]);
    p.r[i].ready = ptr<int>(d, "ready");
    p.r[i].tile_counter = ptr<int>(d, "tile_counter");
    p.r[i].interleave = geti(d, "interleave", 1);
    p.r[i].pair = geti(d, "pair", 0) ? 1 : 0;
    if (p.r[i].pair && n > 1) throw std::invalid_argument("CTA pairs are for one rank per GPU (virtual ranks share the SMs)");
    if (!p.r[i].ready || !p.r[i].route.pulled) throw std::invalid_argument("the fused kernel needs the ready and pulled counter arrays");
  }
  check(launch_mega_fused(p, n, blocks, reinterpret_cast<cudaStream_t>(stream)), "mega_moe launch");
}

void op_mega_route(const WsLayout& lay, const std::vector<py::object>& sessions, const std::vector<py::dict>& args, int blocks,
                   uintptr_t stream) {
  MegaRouteParams p{};
  p.lay = lay;
  const int n = (int)args.size();
  if (n < 1 || n > kMaxRanks || (int)sessions.size() != n) throw std::invalid_argument("1..8 rank argument blocks expected");
  for (int i = 0; i < n; ++i) fill_route(p.r[i], args[i], sessions[i]);
  check(launch_mega_route(p, n, blocks, reinterpret_cast<cudaStream_t>(stream)), "mega_route launch");
}

void op_mega_finish(const WsLayout& lay, const std::vector<py::object>& sessions, const std::vector<py::dict>& args, int blocks,
                    uintptr_t stream) {
  MegaFinishParams p{};
  p.lay = lay;
  const int n = (int)args.size();
  if (n < 1 || n > kMaxRanks || (int)sessions.size() != n) throw std::invalid_argument("1..8 rank argument blocks expected");
  for (int i = 0; i < n; ++i) fill_finish(p.r[i], args[i], sessions[i]);
  check(launch_mega_finish(p, n, blocks, reinterpret_cast<cudaStream_t>(stream)), "mega_finish launch");
}
}  // namespace

void bind_mega(py::module_& m) {
  m.attr("gemm_tile") = kGemmBM;
  m.attr("gemm_tile_n") = kGemmBN;
  m.attr("sf_chunk") = kSfChunk;
  m.attr("mega_timer_words") = kMegaTimerWords;
  m.def("mega_input_offsets", [](int max_tokens, int hidden, int topk) {
    long long o[6];
    mega_input_offsets(max_tokens, hidden, topk, o);
    return std::vector<long long>(o, o + 6);
  });
  m.def("mega_gemm", &op_mega_gemm);
  m.def("mega_route", &op_mega_route);
  m.def("mega_finish", &op_mega_finish);
  m.def("mega_fused", &op_mega_fused);
}
