// ep_layout: the routing summary of upstream DeepEP's V1 `get_dispatch_layout`.
//
// From topk_idx [T, K] (int64, < 0 or >= E marks an empty slot): tokens per destination rank, tokens per expert,
// and is_token_in_rank [T, P].  One thread per token; a block accumulates its counts in shared memory and
// adds them to the global counters once.  Integer atomics: the result does not depend on the order of arrival.
// Counterpart of the reference's dispatch_layout_kernel (csrc/direct/kernels/dispatch/dispatch_layout.cpp:35),
// which builds the same three outputs from per-core partial counts.
#include "api.h"

namespace dep {

constexpr int kLayoutThreads = 256;

__global__ void __launch_bounds__(kLayoutThreads) ep_layout_kernel(const long long* __restrict__ topk_idx, int T, int K, int E, int P,
                                                                   int* __restrict__ tokens_per_rank, int* __restrict__ tokens_per_expert,
                                                                   bool* __restrict__ is_token_in_rank) {
  __shared__ int s_expert[kMaxExperts];
  __shared__ int s_rank[kMaxRanks];
  for (int e = threadIdx.x; e < E; e += kLayoutThreads) s_expert[e] = 0;
  if (threadIdx.x < kMaxRanks) s_rank[threadIdx.x] = 0;
  __syncthreads();
  const int Lx = E / P;
  for (int t = blockIdx.x * kLayoutThreads + threadIdx.x; t < T; t += gridDim.x * kLayoutThreads) {
    unsigned rank_mask = 0;
    for (int k = 0; k < K; ++k) {
      const long long e = topk_idx[(size_t)t * K + k];
      if (e < 0 || e >= E) continue;
      atomicAdd(&s_expert[(int)e], 1);              // per-expert counts include every valid slot, as upstream counts them
      rank_mask |= 1u << ((int)e / Lx);
    }
    for (int r = 0; r < P; ++r) {
      const bool in = (rank_mask >> r) & 1u;
      is_token_in_rank[(size_t)t * P + r] = in;
      if (in) atomicAdd(&s_rank[r], 1);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += kLayoutThreads)
    if (s_expert[e]) atomicAdd(&tokens_per_expert[e], s_expert[e]);
  if (threadIdx.x < P && s_rank[threadIdx.x]) atomicAdd(&tokens_per_rank[threadIdx.x], s_rank[threadIdx.x]);
}

// Outputs must be zeroed by the caller (tokens_per_rank [P], tokens_per_expert [E]); is_token_in_rank is fully written.
cudaError_t launch_layout(const long long* topk_idx, int T, int K, int E, int P, int* tokens_per_rank, int* tokens_per_expert,
                          bool* is_token_in_rank, cudaStream_t stream) {
  if (T <= 0) return cudaSuccess;
  if (K < 1 || K > kMaxTopk || E < P || E > kMaxExperts || E % P || P < 1 || P > kMaxRanks) return cudaErrorInvalidValue;
  const int blocks = (T + kLayoutThreads - 1) / kLayoutThreads;
  ep_layout_kernel<<<blocks < 148 ? blocks : 148, kLayoutThreads, 0, stream>>>(topk_idx, T, K, E, P, tokens_per_rank, tokens_per_expert,
                                                                             is_token_in_rank);
  return cudaGetLastError();
}

}  // namespace dep
