// ep_expand / ep_aggregate: the V1 interface's local layout operators (see expand_api.h).
//
// expand: rows of the rank-deduplicated layout carry up to K local expert ids; every (row, slot) gets its own row
// in the expert-major output, ordered inside an expert by (row, slot).  Ranking is deterministic: per 64-row tile
// a bit mask per expert, ranks from popcounts, tile bases from an exclusive scan over the tiles.  The phases are
// separated by grid barriers (cooperative launch).  Rows between an expert's real count and its capacity are zeroed.
// aggregate: out[r] = sum over the slots of row r of (w *) x[mapping[r][k]], fp32 in slot order, one warp per row.
#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include "expand_api.h"

namespace cg = cooperative_groups;

namespace dep {

constexpr int kExpandThreads = 256;

__global__ void __launch_bounds__(kExpandThreads) ep_expand_kernel(const __grid_constant__ ExpandParams p) {
  cg::grid_group grid = cg::this_grid();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = kExpandThreads / 32;
  const int gw = blockIdx.x * nwarps + warp, total_warps = gridDim.x * nwarps;
  const int tiles = (p.R + kExpandTile - 1) / kExpandTile, L = p.L, K = p.K;
  __shared__ unsigned s_mask[kMaxExperts][2];

  if (!p.cached) {
    // ---- pass 1: rows per (tile, expert)
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
      for (int i = threadIdx.x; i < L * 2; i += kExpandThreads) (&s_mask[0][0])[i] = 0u;
      __syncthreads();
      for (int i = threadIdx.x; i < kExpandTile * K; i += kExpandThreads) {
        const int r = tile * kExpandTile + i / K;
        if (r >= p.R) continue;
        const long long e = p.topk_idx[(size_t)r * K + i % K];
        if (e >= 0 && e < L) atomicOr(&s_mask[e][(i / K) >> 5], 1u << ((i / K) & 31));
      }
      __syncthreads();
      for (int e = threadIdx.x; e < L; e += kExpandThreads) p.tile_counts[(size_t)tile * L + e] = __popc(s_mask[e][0]) + __popc(s_mask[e][1]);
      __syncthreads();
    }
    __threadfence();
    grid.sync();
    // ---- pass 2: exclusive scan over the tiles, one thread per expert
    for (int e = blockIdx.x * kExpandThreads + threadIdx.x; e < L; e += gridDim.x * kExpandThreads) {
      int run = 0;
      for (int t = 0; t < tiles; ++t) { const int c = p.tile_counts[(size_t)t * L + e]; p.tile_counts[(size_t)t * L + e] = run; run += c; }
      p.actual_counts[e] = run;
      if (run > p.expert_offsets[e + 1] - p.expert_offsets[e]) *p.error_flag = 1;
    }
    __threadfence();
    grid.sync();
    // ---- pass 3: the mapping
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
      for (int i = threadIdx.x; i < L * 2; i += kExpandThreads) (&s_mask[0][0])[i] = 0u;
      __syncthreads();
      for (int i = threadIdx.x; i < kExpandTile * K; i += kExpandThreads) {
        const int r = tile * kExpandTile + i / K;
        if (r >= p.R) continue;
        const long long e = p.topk_idx[(size_t)r * K + i % K];
        if (e >= 0 && e < L) atomicOr(&s_mask[e][(i / K) >> 5], 1u << ((i / K) & 31));
      }
      __syncthreads();
      for (int i = threadIdx.x; i < kExpandTile * K; i += kExpandThreads) {
        const int rt = i / K, r = tile * kExpandTile + rt;
        if (r >= p.R) continue;
        const long long e = p.topk_idx[(size_t)r * K + i % K];
        int dst = -1;
        if (e >= 0 && e < L) {
          bool first = true;                 // a repeated id inside a row keeps its first slot only
          for (int k = 0; k < i % K; ++k) first = first && p.topk_idx[(size_t)r * K + k] != e;
          if (first) {
            const int below = rt < 32 ? __popc(s_mask[e][0] & ((1u << rt) - 1u)) : __popc(s_mask[e][0]) + __popc(s_mask[e][1] & ((1u << (rt - 32)) - 1u));
            const int pos = p.tile_counts[(size_t)tile * L + e] + below;
            if (pos < p.expert_offsets[e + 1] - p.expert_offsets[e]) dst = p.expert_offsets[e] + pos;
          }
        }
        p.mapping[(size_t)r * K + i % K] = dst;
      }
      __syncthreads();
    }
    __threadfence();
    grid.sync();
  }

  // ---- copy: one warp per input row, all its destinations at once
  const int units = p.row_bytes / 16;
  for (int r = gw; r < p.R; r += total_warps) {
    int4* dst[kMaxTopk];
    int n = 0;
    for (int k = 0; k < K; ++k) {
      const int d = p.mapping[(size_t)r * K + k];
      if (d < 0 || d >= p.N) continue;
      if (n < kMaxTopk) dst[n++] = reinterpret_cast<int4*>(p.out + (size_t)d * p.row_bytes);
      if (p.out_sf) for (int q = lane; q < p.num_sf; q += 32) p.out_sf[(size_t)d * p.num_sf + q] = p.x_sf[(size_t)r * p.num_sf + q];
      if (p.out_w && lane == 0) p.out_w[d] = p.topk_w ? p.topk_w[(size_t)r * K + k] : 0.f;
    }
    if (n) warp_copy_row<8>(dst, n, reinterpret_cast<const int4*>(p.x + (size_t)r * p.row_bytes), units, lane);
  }
  // ---- padding rows between an expert's real count and its capacity
  for (int e = 0; e < L; ++e) {
    const int begin = p.expert_offsets[e] + min(p.actual_counts[e], p.expert_offsets[e + 1] - p.expert_offsets[e]), end = p.expert_offsets[e + 1];
    for (int d = begin + gw; d < end; d += total_warps) {
      int4* row = reinterpret_cast<int4*>(p.out + (size_t)d * p.row_bytes);
      for (int u = lane; u < units; u += 32) row[u] = make_int4(0, 0, 0, 0);
      if (p.out_sf) for (int q = lane; q < p.num_sf; q += 32) p.out_sf[(size_t)d * p.num_sf + q] = 0.f;
      if (p.out_w && lane == 0) p.out_w[d] = 0.f;
    }
  }
}

cudaError_t launch_expand(const ExpandParams& p, int blocks, cudaStream_t stream) {
  void* args[] = {const_cast<ExpandParams*>(&p)};
  return cudaLaunchCooperativeKernel((const void*)ep_expand_kernel, dim3(blocks), dim3(kExpandThreads), args, 0, stream);
}

template <class T2> __device__ __forceinline__ float2 to_float2(uint32_t v);
template <> __device__ __forceinline__ float2 to_float2<__nv_bfloat162>(uint32_t v) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v)); }
template <> __device__ __forceinline__ float2 to_float2<__half2>(uint32_t v) { return __half22float2(*reinterpret_cast<__half2*>(&v)); }
template <class T2> __device__ __forceinline__ uint32_t from_float2(float a, float b);
template <> __device__ __forceinline__ uint32_t from_float2<__nv_bfloat162>(float a, float b) { __nv_bfloat162 h = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&h); }
template <> __device__ __forceinline__ uint32_t from_float2<__half2>(float a, float b) { __half2 h = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&h); }

template <class T2>
__global__ void __launch_bounds__(kExpandThreads) ep_aggregate_kernel(const __grid_constant__ AggregateParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = kExpandThreads / 32;
  const int units = p.H / 8;
  for (int r = blockIdx.x * nwarps + warp; r < p.R; r += gridDim.x * nwarps) {
    int src[kMaxTopk];
    float w[kMaxTopk];
    int n = 0;
    for (int k = 0; k < p.K; ++k) {
      const int d = p.mapping[(size_t)r * p.K + k];
      const bool valid = d >= 0 && d < p.N;
      if (p.out_values && lane == 0) p.out_values[(size_t)r * p.K + k] = valid && p.values ? p.values[d] : 0.f;
      if (valid && n < kMaxTopk) { src[n] = d; w[n] = p.row_w ? p.row_w[d] : 1.f; ++n; }
    }
    for (int u = lane; u < units; u += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      int4 v[kMaxTopk];
#pragma unroll
      for (int i = 0; i < kMaxTopk; ++i)
        if (i < n) v[i] = __ldg(reinterpret_cast<const int4*>(p.x + (size_t)src[i] * p.H * 2) + u);
#pragma unroll
      for (int i = 0; i < kMaxTopk; ++i) {
        if (i < n) {
          const uint32_t* q = reinterpret_cast<const uint32_t*>(&v[i]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {        // product and sum rounded separately (slot order)
            const float2 f = to_float2<T2>(q[j]);
            acc[2 * j] = __fadd_rn(acc[2 * j], __fmul_rn(w[i], f.x));
            acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], __fmul_rn(w[i], f.y));
          }
        }
      }
      reinterpret_cast<int4*>(p.out + (size_t)r * p.H * 2)[u] =
          make_int4((int)from_float2<T2>(acc[0], acc[1]), (int)from_float2<T2>(acc[2], acc[3]), (int)from_float2<T2>(acc[4], acc[5]),
                    (int)from_float2<T2>(acc[6], acc[7]));
    }
  }
}

cudaError_t launch_aggregate(const AggregateParams& p, int blocks, cudaStream_t stream) {
  if (p.is_half) ep_aggregate_kernel<__half2><<<blocks, kExpandThreads, 0, stream>>>(p);
  else ep_aggregate_kernel<__nv_bfloat162><<<blocks, kExpandThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace dep
