// Workspace layouts (host side): byte offsets of every region of a symmetric workspace, identical on every rank.
// Plain C++ so that host code, the Python bindings and stand-alone host tests (compiled with g++, no GPU) share them;
// `parallel/layout.py` mirrors the sizes and is checked against these functions.
// Parity: csrc/kernels/notify/tiling.hpp:136-244 / csrc/kernels/dispatch/tiling.hpp / csrc/kernels/combine/tiling.hpp of the
// reference (host+device tiling structs with `Make...Tiling`), tested there through tests/utils/cpp.py.
#pragma once
#include <stdexcept>

#include "common.cuh"

namespace dep {

constexpr long long align_up(long long v, long long a) { return (v + a - 1) / a * a; }

// `partial_tokens` (0 = max_tokens): tokens whose combine partials fit the workspace at a time; a smaller window makes the
// combine run in several passes over the tokens (capacity fallback for callers that cap the workspace).
inline WsLayout make_layout(int world, int max_tokens, int hidden, int topk, long long ll_bytes, long long mega_bytes,
                            int partial_tokens = 0) {
  if (world < 1 || world > kMaxRanks) throw std::invalid_argument("world size must be in [1, 8]");
  if (max_tokens < 1 || max_tokens > kChunkTokens * kMaxChunks) throw std::invalid_argument("num_max_tokens_per_rank must be in [1, 16384]");
  if (topk < 1 || topk > kMaxTopk) throw std::invalid_argument("num_topk must be in [1, 16]");
  if (hidden < 8 || hidden % 8) throw std::invalid_argument("hidden must be a positive multiple of 8");
  if (partial_tokens < 0 || partial_tokens > max_tokens) throw std::invalid_argument("the combine window must be in [1, num_max_tokens_per_rank]");
  WsLayout l{};
  l.world = world; l.max_tokens = max_tokens; l.hidden = hidden; l.topk = topk;
  l.partial_tokens = partial_tokens > 0 ? partial_tokens : max_tokens;
  l.stage_row_bytes = (int)align_up((long long)hidden * 2, 128);
  long long at = kControlBytes;
  auto take = [&](long long bytes) { long long o = at; at = align_up(at + bytes, 1024); return o; };
  l.gather_hdr = take((long long)world * 4 * sizeof(int));
  l.gather_idx = take((long long)world * max_tokens * topk * sizeof(int));
  l.gather_w = take((long long)world * max_tokens * topk * sizeof(float));
  l.stage = take((long long)world * max_tokens * l.stage_row_bytes);
  l.partial = take((long long)l.partial_tokens * world * hidden * 2);
  l.wret = take((long long)max_tokens * topk * sizeof(float));
  l.disp_flag = take((long long)world * ((max_tokens + kGroupTokens - 1) / kGroupTokens) * 8);
  l.comb_flag = take((long long)world * ((max_tokens + kRowBlock - 1) / kRowBlock) * 8);
  l.ll = take(ll_bytes);
  l.mega = take(mega_bytes);
  l.total = align_up(at, 2 << 20);
  return l;
}

// Workspace that only carries the control block and the fused-MoE region (dispatch/combine regions are empty).
inline WsLayout make_mega_layout(int world, int max_tokens, int hidden, int topk, long long mega_bytes) {
  if (world < 1 || world > kMaxRanks) throw std::invalid_argument("world size must be in [1, 8]");
  if (topk < 1 || topk > kMaxTopk) throw std::invalid_argument("num_topk must be in [1, 16]");
  if (hidden < 128 || hidden % 128) throw std::invalid_argument("hidden must be a positive multiple of 128");
  WsLayout l{};
  l.world = world; l.max_tokens = max_tokens; l.hidden = hidden; l.topk = topk;
  l.partial_tokens = max_tokens;
  l.stage_row_bytes = hidden * 2;
  l.gather_hdr = l.gather_idx = l.gather_w = l.stage = l.partial = l.wret = l.disp_flag = l.comb_flag = l.ll = kControlBytes;
  l.mega = kControlBytes;
  l.total = align_up(kControlBytes + mega_bytes, 2 << 20);
  return l;
}

}  // namespace dep
