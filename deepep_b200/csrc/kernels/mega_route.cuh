// MegaMoE routing + token pull, and the final weighted reduction.
//
// mega_route: after a cross-rank "inputs ready" handshake every rank reads all ranks' routing
// tables straight from peer memory, counts the rows of its local experts, lays the experts out
// as 128-row tiles, and pulls the e4m3 token rows and their ue8m0 scales from the owners'
// symmetric input blocks into expert-major operands (scales in the tensor-memory chunk layout).
// Row order inside an expert is arbitrary (atomic tickets): rows are independent in the GEMMs
// and the final reduction is ordered by top-k slot at the source, so results stay deterministic.
//
// mega_finish: tells the peers that this rank's GEMM2 rows have been written, waits for the
// same from everybody, then y[t] = sum_k w[t, k] * row[t, k] (fp32, slot order) -> bf16.
//
// Parity: stage/route_compact, stage/token_dispatch, CrossRankSync and stage/unpermute of the
// reference's MegaMoE kernel (experiments/megamoe/csrc/kernels/mega_moe/mega_moe_arch35.hpp:852-1006).
#include <cooperative_groups.h>

#pragma once
#include "mega_api.h"

namespace cg = cooperative_groups;

namespace dep {

struct MegaInput {  // offsets inside the input block of a workspace
  long long x, x_sf, idx, w, hdr, total;
};
__host__ __device__ inline MegaInput mega_input_layout(int M, int H, int K) {
  MegaInput l;
  long long at = 0;
  auto take = [&](long long b) { long long o = at; at = (at + b + 1023) / 1024 * 1024; return o; };
  l.hdr = take(64);
  l.x = take((long long)M * H);
  l.x_sf = take((long long)M * (H / 32));
  l.idx = take((long long)M * K * 4);
  l.w = take((long long)M * K * 4);
  l.total = at;
  return l;
}

#ifdef __CUDACC__
__device__ __forceinline__ void route_phase(const MegaRouteArgs& a, cg::grid_group& grid) {
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, me = ctx.rank, K = a.K, H = a.H, E = a.E, Lx = E / P, M = a.max_tokens;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gtid = blockIdx.x * (int)blockDim.x + threadIdx.x, gstride = gridDim.x * (int)blockDim.x;
  const int gw = blockIdx.x * ((int)blockDim.x / 32) + warp, total_warps = gridDim.x * ((int)blockDim.x / 32);
  Control* ctl = control_of(ctx.ws[me]);
  const unsigned long long epoch = ctl->epoch[kOpMega] + 1;
  const MegaInput in = mega_input_layout(M, H, K);

  __shared__ int s_T[kMaxRanks];
  __shared__ int s_base[kMaxExperts];   // first row of every local expert (multiple of 128)

  // ---- handshake: my inputs are in place (stream order), tell everybody, wait for everybody
  if (blockIdx.x == 0 && threadIdx.x < P) {
    if (threadIdx.x == 0) reinterpret_cast<int*>(ctx.ws[me] + a.in_off + in.hdr)[0] = a.T;
    __threadfence_system();
  }
  grid.sync();
  if (blockIdx.x == 0 && threadIdx.x < P) st_release_sys(&control_of(ctx.ws[threadIdx.x])->mega_flag[me][0], epoch);
  int ok = 1;
  if (threadIdx.x < P) ok = wait_flag_ge(&ctl->mega_flag[threadIdx.x][0], epoch, ctx, kOpMega, 0, threadIdx.x);
  const int alive = __syncthreads_and(ok);
  if (threadIdx.x < kMaxRanks)
    s_T[threadIdx.x] = (alive && threadIdx.x < P) ? __ldcg(reinterpret_cast<const int*>(ctx.ws[threadIdx.x] + a.in_off + in.hdr)) : 0;
  // zero the per-expert counters
  if (blockIdx.x == 0) for (int l = threadIdx.x; l < Lx; l += (int)blockDim.x) a.expert_rows[l] = 0;
  __syncthreads();
  grid.sync();

  // ---- pass 1: rows per local expert
  for (int r = 0; r < P; ++r) {
    const int* idx = reinterpret_cast<const int*>(ctx.ws[r] + a.in_off + in.idx);
    const int n = s_T[r] * K;
    for (int i = gtid; i < n; i += gstride) {
      const int e = __ldcg(idx + i);
      if (e >= me * Lx && e < (me + 1) * Lx) atomicAdd(&a.expert_rows[e - me * Lx], 1);
    }
  }
  __threadfence();
  grid.sync();

  // ---- tile layout: every expert starts at a multiple of 128 rows
  if (threadIdx.x == 0) {
    int run = 0;
    for (int l = 0; l < Lx; ++l) {
      s_base[l] = run;
      const int tiles = (a.expert_rows[l] + kGemmBM - 1) / kGemmBM;
      if (blockIdx.x == 0)
        for (int t = 0; t < tiles && run / kGemmBM + t < a.max_mtiles; ++t) a.mtile_expert[run / kGemmBM + t] = l;
      run += tiles * kGemmBM;
    }
    if (blockIdx.x == 0) *a.num_mtiles = min(run / kGemmBM, a.max_mtiles);
  }
  __syncthreads();
  const int rows_cap = a.max_mtiles * kGemmBM;
  // padding rows carry no source; their payload is never read back (tile rows are independent in the GEMMs)
  for (int l = blockIdx.x; l < Lx; l += gridDim.x) {
    const int c = a.expert_rows[l], end = (c + kGemmBM - 1) / kGemmBM * kGemmBM;
    for (int rr = c + threadIdx.x; rr < end; rr += (int)blockDim.x)
      if (s_base[l] + rr < rows_cap) a.row_src[s_base[l] + rr] = -1;
  }
  int* ticket = a.ticket;   // zeroed by the previous call's pass 2 epilogue (and at allocation)

  // ---- pass 2: hand out rows and pull the tokens (one warp per routed slot)
  if (alive) {
    for (int r0 = 0; r0 < P; ++r0) {
      const int r = (me + r0) % P;
      const uint8_t* peer = ctx.ws[r] + a.in_off;
      const int* idx = reinterpret_cast<const int*>(peer + in.idx);
      const int n = s_T[r] * K;
      for (int i0 = gw * 32; i0 < n; i0 += total_warps * 32) {
        const int i = i0 + lane;
        const int e = i < n ? __ldcg(idx + i) : -1;
        const bool mine = e >= me * Lx && e < (me + 1) * Lx;
        int my_row = -1;
        if (mine) my_row = s_base[e - me * Lx] + atomicAdd(&ticket[e - me * Lx], 1);
        unsigned todo = __ballot_sync(0xffffffffu, mine && my_row < rows_cap);
        while (todo) {
          const int src_lane = __ffs(todo) - 1;
          todo &= todo - 1;
          const long long row = __shfl_sync(0xffffffffu, my_row, src_lane);
          const int slot_i = i0 + src_lane, t = slot_i / K;
          const int4* from = reinterpret_cast<const int4*>(peer + in.x + (size_t)t * H);
          int4* to = reinterpret_cast<int4*>(a.a1 + row * H);
          { int4* one[1] = {to}; warp_copy_row<14>(one, 1, from, H / 16, lane); }
          const uint32_t* sf = reinterpret_cast<const uint32_t*>(peer + in.x_sf + (size_t)t * (H / 32));
          for (int g = lane; g < H / 128; g += 32)
            *reinterpret_cast<uint32_t*>(a.a1_sf + sf_offset(row, (long long)g * 128, H)) = __ldcg(sf + g);
          if (lane == 0) a.row_src[row] = (r * M + t) * K + (slot_i - t * K);
        }
      }
    }
  }
  grid.sync();
  if (blockIdx.x == 0) for (int l = threadIdx.x; l < Lx; l += (int)blockDim.x) ticket[l] = 0;   // ready for the next call
}


__device__ __forceinline__ void finish_phase(const MegaFinishArgs& a, bool bump_epoch) {
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, me = ctx.rank, K = a.K, H = a.H, M = a.max_tokens;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gw = blockIdx.x * ((int)blockDim.x / 32) + warp, total_warps = gridDim.x * ((int)blockDim.x / 32);
  Control* ctl = control_of(ctx.ws[me]);
  const unsigned long long epoch = ctl->epoch[kOpMega] + 1;
  const MegaInput in = mega_input_layout(M, H, K);

  // my GEMM2 finished before this kernel started (stream order, its remote writes were fenced)
  if (blockIdx.x == 0 && threadIdx.x < P) {
    __threadfence_system();
    st_release_sys(&control_of(ctx.ws[threadIdx.x])->mega_flag[me][1], epoch);
  }
  int ok = 1;
  if (threadIdx.x < P) ok = wait_flag_ge(&ctl->mega_flag[threadIdx.x][1], epoch, ctx, kOpMega, 1, threadIdx.x);
  const int alive = __syncthreads_and(ok);
  if (alive) {
    const int* idx = reinterpret_cast<const int*>(ctx.ws[me] + a.in_off + in.idx);
    const float* w = reinterpret_cast<const float*>(ctx.ws[me] + a.in_off + in.w);
    const uint8_t* comb = ctx.ws[me] + a.comb_off;
    for (int t = gw; t < a.T; t += total_warps) {
      float wk[kMaxTopk];
      unsigned valid = 0;
      for (int k = 0; k < K; ++k) {
        const int e = idx[(size_t)t * K + k];
        wk[k] = w[(size_t)t * K + k];
        if (e >= 0 && e < a.E) valid |= 1u << k;
      }
      int4* out = reinterpret_cast<int4*>(reinterpret_cast<uint8_t*>(a.y) + (size_t)t * H * 2);
      const uint8_t* rows = comb + (size_t)t * K * H * 2;
      for (int u0 = lane; u0 < H / 8; u0 += 64) {      // two 16-byte columns per step, all slots' loads issued first
        const bool two = u0 + 32 < H / 8;
        int4 v0[kMaxTopk], v1[kMaxTopk];
#pragma unroll
        for (int k = 0; k < kMaxTopk; ++k) {
          if (k < K && ((valid >> k) & 1u)) {
            v0[k] = ld_cg_int4(rows + (size_t)k * H * 2 + (size_t)u0 * 16);
            if (two) v1[k] = ld_cg_int4(rows + (size_t)k * H * 2 + (size_t)(u0 + 32) * 16);
          }
        }
        float a0[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, a1[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int k = 0; k < kMaxTopk; ++k) {
          if (k < K && ((valid >> k) & 1u)) {
            const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&v0[k]);
            const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&v1[k]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {   // product and sum rounded separately, as the CPU oracle does
              a0[2 * i] = __fadd_rn(a0[2 * i], __fmul_rn(wk[k], __low2float(h0[i])));
              a0[2 * i + 1] = __fadd_rn(a0[2 * i + 1], __fmul_rn(wk[k], __high2float(h0[i])));
              if (two) {
                a1[2 * i] = __fadd_rn(a1[2 * i], __fmul_rn(wk[k], __low2float(h1[i])));
                a1[2 * i + 1] = __fadd_rn(a1[2 * i + 1], __fmul_rn(wk[k], __high2float(h1[i])));
              }
            }
          }
        }
        int4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) oh[i] = __floats2bfloat162_rn(a0[2 * i], a0[2 * i + 1]);
        out[u0] = o;
        if (two) {
#pragma unroll
          for (int i = 0; i < 4; ++i) oh[i] = __floats2bfloat162_rn(a1[2 * i], a1[2 * i + 1]);
          out[u0 + 32] = o;
        }
      }
    }
  }
  if (bump_epoch && last_block_of_rank(ctl, kOpMega, gridDim.x)) {
    if (threadIdx.x == 0) ctl->epoch[kOpMega] = epoch;
  }
}

#endif  // __CUDACC__

}  // namespace dep
