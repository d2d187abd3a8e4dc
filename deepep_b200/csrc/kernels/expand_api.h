// Local layout operators of the V1 interface: expand (rank-deduplicated rows -> expert-major rows) and
// aggregate (expert-major rows -> rank-deduplicated rows).  No communication.
//
// Counterpart of the reference's expand_kernel (csrc/direct/kernels/expand/expand.cpp:110) and
// aggregate_kernel (csrc/direct/kernels/aggregate/aggregate.cpp:21) with their host ops
// (csrc/direct/ops/expand.cpp, aggregate.cpp).
#pragma once
#include "common.cuh"

namespace dep {

constexpr int kExpandTile = 64;    // rows per ranking tile (two 32-bit mask words per expert)

struct ExpandParams {
  const uint8_t* x;            // [R][row_bytes]
  const float* x_sf;           // [R][num_sf] or null
  const long long* topk_idx;   // [R][K] local expert id, anything outside [0, L) is an empty slot; null in cached mode
  const float* topk_w;         // [R][K] or null
  uint8_t* out;                // [N][row_bytes]
  float* out_sf;               // [N][num_sf] or null
  float* out_w;                // [N] or null
  int* expert_offsets;         // [L + 1] exclusive prefix of the capacities (input)
  int* actual_counts;          // [L] rows really routed to each expert (output; input in cached mode)
  int* mapping;                // [R][K] expanded row of every slot, -1 for empty (output; input in cached mode)
  int* tile_counts;            // scratch [tiles][L]
  int* error_flag;             // set to 1 when an expert receives more rows than its capacity
  int R, K, L, N, row_bytes, num_sf, cached, pad;
};
cudaError_t launch_expand(const ExpandParams& p, int blocks, cudaStream_t stream);

struct AggregateParams {
  const uint8_t* x;            // [N][H] bf16 or fp16
  const float* row_w;          // [N] or null: every expanded row is multiplied by its weight
  const float* values;         // [N] or null: independent fp32 channel
  const int* mapping;          // [R][K]
  uint8_t* out;                // [R][H]
  float* out_values;           // [R][K] or null
  int R, K, H, N, is_half, pad;
};
cudaError_t launch_aggregate(const AggregateParams& p, int blocks, cudaStream_t stream);

}  // namespace dep
