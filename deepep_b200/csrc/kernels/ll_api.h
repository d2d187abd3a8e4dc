// Low-latency (decode) dispatch/combine: argument blocks, region layout and launchers.
//
// Counterpart of the reference's low-latency kernels (csrc/kernels/dispatch/low_latency.cpp:17-66 and
// csrc/kernels/combine/low_latency.cpp:17-45): no separate notify, fixed pre-allocated receive
// slots, per-message flags that are polled, two banks selected by call parity, every piece of
// state device-resident so the launch can be captured in a CUDA graph and replayed.
#pragma once
#include "common.cuh"

namespace dep {

constexpr int kLLParts = 4;   // column parts of a row, each with its own completion flag

// Offsets inside the low-latency region of a workspace (relative to WsLayout::ll), for one bank.
struct LLLayout {
  long long gather_hdr;   // int   [P][4]
  long long gather_idx;   // int   [P][M][K]
  long long gather_w;     // float [P][M][K]
  long long idx_flag;     // u64   [P]        routing table of source r has landed
  long long row_flag;     // u64   [P][M][kLLParts]  part p of staged row j of source r has landed
  long long stage;        // byte  [P][M][msg_bytes]
  long long ret_flag;     // u64   [M][K][kLLParts]  part p of the returned row of (token, slot) has landed
  long long ret;          // bf16  [M][K][H]
  long long bank_bytes;   // size of one bank; bank b starts at b * bank_bytes
  int msg_bytes, pad;
};

__host__ __device__ inline long long ll_align(long long v) { return (v + 1023) / 1024 * 1024; }

__host__ __device__ inline LLLayout make_ll_layout(int P, int M, int K, int H) {
  LLLayout l{};
  l.msg_bytes = (H * 2 + 127) / 128 * 128;
  long long at = 0;
  l.gather_hdr = at; at = ll_align(at + (long long)P * 4 * 4);
  l.gather_idx = at; at = ll_align(at + (long long)P * M * K * 4);
  l.gather_w = at;   at = ll_align(at + (long long)P * M * K * 4);
  l.idx_flag = at;   at = ll_align(at + (long long)P * 8);
  l.row_flag = at;   at = ll_align(at + (long long)P * M * kLLParts * 8);
  l.stage = at;      at = ll_align(at + (long long)P * M * l.msg_bytes);
  l.ret_flag = at;   at = ll_align(at + (long long)M * K * kLLParts * 8);
  l.ret = at;        at = ll_align(at + (long long)M * K * H * 2);
  l.bank_bytes = at;
  return l;
}
inline long long ll_region_bytes(int P, int M, int K, int H) { return 2 * make_ll_layout(P, M, K, H).bank_bytes; }

struct LLDispatchArgs {
  RankCtx ctx;
  const void* x;               // [T][H] bf16 (modes 0, 2) or e4m3 (mode 1)
  const float* x_sf;           // [T][H/128] (mode 1)
  const long long* topk_idx;   // [T][K]
  const float* topk_w;         // [T][K]
  int T, E, mode, pad;
  void* recv_x;                // [C][H]
  float* recv_sf;              // [C][H/128] or null
  float* recv_w;               // [C]
  int* recv_row_src;           // [C] (source * M + token) * K + slot
  int* expert_counts;          // [L]
  int* expert_offsets;         // [L + 1]
  int* num_rows;               // [1] device copy of the row count
  int* mailbox;                // mapped host memory (may be null): [0] rows, [3] epoch, [4..] counts
  long long capacity;          // rows available in recv_x
};
struct LLDispatchParams { WsLayout lay; int profile, pad; LLDispatchArgs r[kMaxRanks]; };   // profile: block 0 stamps its phases into Control::dbg[0..7]
cudaError_t launch_ll_dispatch(const LLDispatchParams& p, int nranks, int blocks, cudaStream_t stream);

struct LLCombineArgs {
  RankCtx ctx;
  const __nv_bfloat16* x;      // [rows][H] expert outputs
  const int* recv_row_src;     // [rows]
  const int* num_rows;         // [1]
  const long long* topk_idx;   // [T][K] of this rank's tokens
  const float* topk_w;         // [T][K] weights applied here, at the source
  int T, E;
  __nv_bfloat16* out;          // [T][H]
};
struct LLCombineParams { WsLayout lay; int profile, pad; LLCombineArgs r[kMaxRanks]; };     // profile: the same into Control::dbg[8..15]
cudaError_t launch_ll_combine(const LLCombineParams& p, int nranks, int blocks, cudaStream_t stream);

}  // namespace dep
