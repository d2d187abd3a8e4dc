// Host-callable launchers of the expert-parallel kernels and their argument blocks.
//
// Every launcher takes `nranks` argument blocks: 1 in production (one process
// per GPU) or several virtual ranks that share one GPU (single-launch protocol
// test).  Pointers are device pointers valid on the current device.
#pragma once
#include "common.cuh"

namespace dep {

// ---------------------------------------------------------------- notify (routing layout)
// Counterpart of the reference's notify kernel (csrc/kernels/notify/notify.cpp:1426-1970):
// counts, prefix offsets, rank-level dedup map and receive-side expansion lists.
struct NotifyArgs {
  RankCtx ctx;
  const long long* topk_idx;   // [T][K]; <0 or >=E marks an empty slot
  const float* topk_w;         // [T][K] or null
  int T, E, K;
  int expand;                  // 1: rows per (token, slot) sorted by local expert; 0: rows per (source, token)
  int alignment;               // every local expert's row block starts at a multiple of this
  int meta_stride;             // ints per stage_meta record: 2 + max(2, min(K, E / world))
  // scratch owned by the buffer
  int* hist;                   // [P][NT][E]
  int* hits;                   // [P][NT]
  int* own_hits;               // [NT][P]
  int* cnt;                    // [P][E]
  // outputs owned by the handle
  int* send_slot;              // [T][P]  staging index on each destination, -1 if not routed there
  int* slot_row;               // [T][K]  row on the destination rank (expanded layout), -1 if empty
  int* stage_meta;             // [P * Tmax][meta_stride]: token, n, n x (row | slot << 27); rank layout: token, 1, row, slot mask
  int* chunk_start;            // [P][NT + 1] staged-row index at the start of every source chunk
  int* rank_tokens;            // [P] tokens each source holds
  int* rank_rows;              // [P + 1] exclusive prefix of staged rows per source
  int* expert_counts;          // [L] unaligned rows per local expert
  int* expert_offsets;         // [L + 1] aligned exclusive prefix
  int* recv_row_src;           // [rcap] (source * Tmax + token) * K + slot of every output row, -1 for padding
  float* recv_w;               // [rcap] (expanded) or [rcap][K] (rank layout); may be null
  long long* recv_idx;         // [rcap][K] destination-local expert ids (rank layout) or null
  int* rank_matrix;            // optional [P][P], zeroed by the caller: tokens that source i sends to rank j (every rank computes all of it)
  int* mailbox;                // mapped host memory: [0] rows, [1] staged rows, [2] max tokens, [3] epoch, [4..] counts
  long long rcap;
};
struct NotifyParams { WsLayout lay; int profile, pad; NotifyArgs r[kMaxRanks]; };   // profile: block 0 stamps its phases into Control::dbg[16..23]
cudaError_t launch_notify(const NotifyParams& p, int nranks, int blocks, cudaStream_t stream);

// ---------------------------------------------------------------- high-throughput dispatch
// Counterpart of csrc/kernels/dispatch/dispatch.cpp:463-590 of the reference: payload scatter
// + receive-side expansion + completion flags, here with an optional fused bf16 -> e4m3 quantiser.
enum DispatchMode : int { kDispatchBf16 = 0, kDispatchFp8Given = 1, kDispatchFp8Fused = 2 };
struct DispatchArgs {
  RankCtx ctx;
  const void* x;               // [T][H] bf16/fp16 (modes 0, 2) or e4m3 (mode 1)
  const float* x_sf;           // [T][H/128] (mode 1)
  int T, mode;
  const int* send_slot;        // [T][P]
  const int* slot_row;         // [T][K] output row of every slot on its destination (expanded layout)
  const long long* topk_idx;   // [T][K] of this rank's tokens (which slots are local)
  const int* stage_meta;
  const int* rank_tokens;
  const int* rank_rows;        // [P + 1] exclusive prefix of the staged rows per source (rank layout: first output row of a source)
  int meta_stride, recv_rows;  // recv_rows: rows of recv_x (only read by the optional index checks; 0 = unknown)
  int K, E, expand;
  void* recv_x;                // [R][H] 2-byte (mode 0) or e4m3 (modes 1, 2)
  float* recv_sf;              // [R][H/128] or null
  unsigned long long* prof;    // profile build only: kDispatchProfWords words per block, or null
};
// local_direct: rows whose destination is the sending rank itself are written straight into recv_x by the sender
// blocks (no staging, no flag); 0 sends them through the staging area like remote rows.
struct DispatchParams { WsLayout lay; int send_blocks, recv_blocks, local_direct, profile; DispatchArgs r[kMaxRanks]; };
// per block: role (0 sender, 1 receiver), start ns, end ns, then summed over the block's warps: cycles spent reading
// routing records, waiting for flags, moving rows, publishing flags; rows moved
constexpr int kDispatchProfWords = 8;
constexpr int kDispatchThreads = 512;   // 16 independent warps per block
cudaError_t launch_dispatch(const DispatchParams& p, int nranks, cudaStream_t stream);

// ---------------------------------------------------------------- high-throughput combine
// Counterpart of csrc/kernels/combine/combine.cpp:2224-2917 (EP8 form): expert ranks reduce the
// rows of one (source token, this rank) in fp32, return one bf16 partial, the source reduces
// the partials of its destinations in rank order and adds the optional biases.
struct CombineArgs {
  RankCtx ctx;
  const __nv_bfloat16* x;      // [R][H] expert outputs
  const float* w;              // [R] (expanded) / [R][K] (rank layout) value channel, or null
  const int* stage_meta;
  const int* rank_tokens;
  const int* rank_rows;        // [P + 1] exclusive prefix of the staged rows per source
  const int* send_slot;        // [T][P]
  const long long* topk_idx;   // [T][K] of the source tokens (validity of returned weights)
  int T, meta_stride, K, E, expand, x_rows;   // x_rows: rows of x (only read by the optional index checks; 0 = unknown)
  const __nv_bfloat16* bias0;  // [T][H] or null
  const __nv_bfloat16* bias1;
  __nv_bfloat16* out;          // [T][H]
  float* out_w;                // [T][K] or null
  unsigned long long* prof;    // profile build only: kCombineProfWords words per block, or null
};
// local_direct: the source side sums the rows of its own rank straight from x (same rounding: fp32 sum -> bf16 ->
// fp32), so no local partial is written and no flag is needed for it.
// t_begin / t_end: the token window of this pass (all tokens unless the workspace holds the partials of fewer tokens than
// num_max_tokens_per_rank: the combine then runs one launch per window, every rank with the same window).
struct CombineParams { WsLayout lay; int send_blocks, recv_blocks, local_direct, profile; int t_begin, t_end; CombineArgs r[kMaxRanks]; };
// per block: role (0 expert side, 1 source side), start ns, end ns, then summed over the block's warps: cycles spent
// reading routing records, waiting for flags, reducing rows, publishing flags; rows read
constexpr int kCombineProfWords = 8;
constexpr int kCombineThreads = 384;    // 12 warps: up to 168 registers per thread, which the source side needs for 8 partials in flight
cudaError_t launch_combine(const CombineParams& p, int nranks, cudaStream_t stream);

// ---------------------------------------------------------------- V1 routing summary (get_dispatch_layout)
cudaError_t launch_layout(const long long* topk_idx, int T, int K, int E, int P, int* tokens_per_rank, int* tokens_per_expert,
                          bool* is_token_in_rank, cudaStream_t stream);

// ---------------------------------------------------------------- barrier
struct BarrierParams { RankCtx r[kMaxRanks]; };
cudaError_t launch_barrier(const BarrierParams& p, int nranks, cudaStream_t stream);
// Waits on a flag nobody writes: exercises the bounded-wait + status path without a fault.
cudaError_t launch_wait_probe(const RankCtx& ctx, cudaStream_t stream);

}  // namespace dep
