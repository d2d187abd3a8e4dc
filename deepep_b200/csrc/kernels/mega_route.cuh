// MegaMoE routing + token pull, and the final weighted reduction.
//
// mega_route: after a cross-rank "inputs ready" handshake every rank reads all ranks' routing
// tables straight from peer memory, counts the rows of its local experts, lays the experts out
// as 128-row tiles, and pulls the e4m3 token rows and their ue8m0 scales from the owners'
// symmetric input blocks into expert-major operands (scales in the tensor-memory chunk layout).
// Row order inside an expert is arbitrary (arrival order of an atomic counter): rows are independent in the GEMMs
// and the final reduction is ordered by top-k slot at the source, so results stay deterministic.
//
// mega_finish: tells the peers that this rank's GEMM2 rows have been written, waits for the
// same from everybody, then y[t] = sum_k w[t, k] * row[t, k] (fp32, slot order) -> bf16.
//
// Parity: stage/route_compact, stage/token_dispatch, CrossRankSync and stage/unpermute of the
// reference's MegaMoE kernel (experiments/megamoe/csrc/kernels/mega_moe/mega_moe_arch35.hpp:852-1006).
#pragma once
#ifdef __CUDACC__
#include <cooperative_groups.h>
namespace cg = cooperative_groups;
#endif
#include "mega_api.h"

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
struct RouteShared {
  int T[kMaxRanks];          // tokens of every rank
  int base[kMaxExperts];     // first row of every local expert (multiple of 128)
  int rows[kMaxExperts];     // rows of every local expert
  int alive, total_rows;
};

constexpr int kPullChunk = 8;   // consecutive rows one warp pulls before it moves on

__device__ __forceinline__ void mega_stamp(unsigned long long* timer, int slot) {
  if (timer != nullptr && threadIdx.x == 0) timer[(size_t)blockIdx.x * kMegaTimerWords + slot] = global_timer_ns();
}

// bf16 [T, H] -> e4m3 codes and one ue8m0 exponent per 32 values, written into this rank's symmetric input block.
// Block scale 2^(floor(log2(amax)) - 8) (amax clamped to 2^-119, exponent to -127), values clamped to +-448: the
// quantiser of the reference's token-quant stage (stage/mega_moe_token_quant.hpp; oracle: reference.py:44-54).
// One lane per 32-value block.
__device__ __forceinline__ void quantize_inputs_phase(const MegaRouteArgs& a, uint8_t* x_out, uint8_t* sf_out) {
  const int blocks_per_row = a.H / 32;
  const long long total = (long long)a.T * blocks_per_row;
  for (long long b = blockIdx.x * (long long)blockDim.x + threadIdx.x; b < total; b += (long long)gridDim.x * blockDim.x) {
    const int4* src = reinterpret_cast<const int4*>(a.x_bf16) + b * 4;
    int4 raw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) raw[i] = __ldg(src + i);
    float v[32];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[8 * i + 2 * j] = __low2float(h[j]); v[8 * i + 2 * j + 1] = __high2float(h[j]);
        amax = fmaxf(amax, fmaxf(fabsf(v[8 * i + 2 * j]), fabsf(v[8 * i + 2 * j + 1])));
      }
    }
    amax = fmaxf(amax, __uint_as_float((127u - 119u) << 23));                       // 2^-119
    const int exponent = max((int)((__float_as_uint(amax) >> 23) & 0xffu) - 127 - 8, -127);
    const float inv = __uint_as_float((unsigned)(127 - exponent) << 23);          // 2^-exponent, exact
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint32_t word = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float scaled = fminf(fmaxf(v[4 * i + j] * inv, -448.f), 448.f);
        word |= (uint32_t)__nv_cvt_float_to_fp8(scaled, __NV_SATFINITE, __NV_E4M3) << (8 * j);
      }
      w[i] = word;
    }
    int4* dst = reinterpret_cast<int4*>(x_out) + b * 2;
    dst[0] = make_int4((int)w[0], (int)w[1], (int)w[2], (int)w[3]);
    dst[1] = make_int4((int)w[4], (int)w[5], (int)w[6], (int)w[7]);
    sf_out[b] = (uint8_t)(exponent + 127);
  }
}

// Handshake, per-expert entry lists, 128-row tile layout (tile -> expert).
// expert_list[l * cap + j] (cap = world * max_tokens) = (source * M + token) * (K + S) + slot of the j-th routed slot of
// local expert l, in arrival order; the S shared experts follow the routed ones and take every token of this rank
// (slot K + s).
__device__ __forceinline__ void route_layout_phase(const MegaRouteArgs& a, cg::grid_group& grid, RouteShared& sh) {
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, me = ctx.rank, K = a.K, E = a.E, Lx = E / P, M = a.max_tokens;
  const int gtid = blockIdx.x * (int)blockDim.x + threadIdx.x, gstride = gridDim.x * (int)blockDim.x;
  Control* ctl = control_of(ctx.ws[me]);
  const unsigned long long epoch = ctl->epoch[kOpMega] + 1;
  const MegaInput in = mega_input_layout(M, a.H, K);
  const int cap = P * M, S = a.S, Kp = K + S;     // Kp: combine slots per token (top-k slots, then one per shared expert)

  mega_stamp(a.timer, kTimStart);
  if (a.x_bf16 != nullptr)   // the caller passed bf16 activations: quantise them into the symmetric input block first
    quantize_inputs_phase(a, ctx.ws[me] + a.in_off + in.x, ctx.ws[me] + a.in_off + in.x_sf);
  // ---- handshake: my inputs are in place (stream order, or just written above), tell everybody, wait for everybody
  __threadfence_system();
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
    sh.T[threadIdx.x] = (alive && threadIdx.x < P) ? __ldcg(reinterpret_cast<const int*>(ctx.ws[threadIdx.x] + a.in_off + in.hdr)) : 0;
  if (threadIdx.x == 0) sh.alive = alive;
  // zero the per-expert counters
  if (blockIdx.x == 0) for (int l = threadIdx.x; l < Lx + S; l += (int)blockDim.x) a.expert_rows[l] = 0;
  __syncthreads();
  grid.sync();
  mega_stamp(a.timer, kTimHandshake);

  // ---- pass 1: the routed slots of every local expert (own rank first, then the peers in ring order)
  for (int r0 = 0; r0 < P; ++r0) {
    const int r = (me + r0) % P;
    const int* idx = reinterpret_cast<const int*>(ctx.ws[r] + a.in_off + in.idx);
    const int n = sh.T[r] * K;
    for (int i = gtid; i < n; i += gstride) {
      const int e = __ldcg(idx + i);
      if (e >= me * Lx && e < (me + 1) * Lx) {
        const int j = atomicAdd(&a.expert_rows[e - me * Lx], 1);
        if (j < cap) a.expert_list[(size_t)(e - me * Lx) * cap + j] = (r * M + i / K) * Kp + i % K;
      }
    }
  }
  // shared experts: every token of this rank, in order, into combine slot K + s
  for (int s = 0; s < S; ++s) {
    for (int t = gtid; t < a.T; t += gstride) a.expert_list[(size_t)(Lx + s) * cap + t] = (me * M + t) * Kp + K + s;
    if (gtid == 0) a.expert_rows[Lx + s] = a.T;
  }
  __threadfence();
  grid.sync();

  // ---- tile layout: every expert starts at a multiple of 128 rows (256 with CTA pairs)
  for (int l = threadIdx.x; l < Lx + S; l += (int)blockDim.x) sh.rows[l] = min(__ldcg(a.expert_rows + l), cap);   // parallel loads
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int l = 0; l < Lx + S; ++l) {
      const int c = sh.rows[l];
      sh.base[l] = run;
      const int unit = a.tile_pairs ? 2 * kGemmBM : kGemmBM;      // with CTA pairs an expert owns whole pairs of tiles
      const int tiles = (c + unit - 1) / unit * (unit / kGemmBM);
      if (blockIdx.x == 0)
        for (int t = 0; t < tiles && run / kGemmBM + t < a.max_mtiles; ++t) a.mtile_expert[run / kGemmBM + t] = l;
      run += tiles * kGemmBM;
    }
    sh.total_rows = min(run, a.max_mtiles * kGemmBM);
    if (blockIdx.x == 0) *a.num_mtiles = sh.total_rows / kGemmBM;
  }
  __syncthreads();
  mega_stamp(a.timer, kTimLayout);
}

// Pulls the routed tokens from their owners in row order (tile by tile, so that the first tiles are complete first);
// warp `gw` of `total_warps` warps.  Padding rows get row_src = -1; their payload is never read back (tile rows are
// independent in the GEMMs).
__device__ __forceinline__ void route_pull_phase(const MegaRouteArgs& a, const RouteShared& sh, int gw, int total_warps) {
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, K = a.K, H = a.H, M = a.max_tokens;
  const int lane = threadIdx.x & 31;
  const MegaInput in = mega_input_layout(M, H, K);
  const int cap = P * M, Kp = K + a.S;
  if (!sh.alive) return;
  for (int row0 = gw * kPullChunk; row0 < sh.total_rows; row0 += total_warps * kPullChunk) {
    // lane j < kPullChunk looks up row row0 + j
    int entry = -1;
    if (lane < kPullChunk && row0 + lane < sh.total_rows) {
      const int row = row0 + lane, l = __ldcg(a.mtile_expert + row / kGemmBM), j = row - sh.base[l];
      if (j < sh.rows[l]) entry = __ldcg(a.expert_list + (size_t)l * cap + j);
      a.row_src[row] = entry;
    }
#pragma unroll 1
    for (int c = 0; c < kPullChunk; ++c) {
      const int en = __shfl_sync(0xffffffffu, entry, c);
      if (en < 0) continue;
      const long long row = row0 + c;
      const int r = en / (M * Kp), t = (en - r * M * Kp) / Kp;
      const uint8_t* peer = ctx.ws[r] + a.in_off;
      const int4* from = reinterpret_cast<const int4*>(peer + in.x + (size_t)t * H);
      int4* to = reinterpret_cast<int4*>(a.a1 + row * H);
      { int4* one[1] = {to}; warp_copy_row<14>(one, 1, from, H / 16, lane); }
      const uint32_t* sf = reinterpret_cast<const uint32_t*>(peer + in.x_sf + (size_t)t * (H / 32));
      for (int g = lane; g < H / 128; g += 32)
        *reinterpret_cast<uint32_t*>(a.a1_sf + sf_offset(row, (long long)g * 128, H)) = __ldcg(sf + g);
    }
    if (a.pulled) {            // tell the GEMM that these rows of the tile (payload or padding mark) are in place
      __threadfence();
      __syncwarp();
      if (lane == 0) atomicAdd(a.pulled + row0 / kGemmBM, min(kPullChunk, sh.total_rows - row0));
    }
  }
  if (a.timer != nullptr && lane == 0)     // the CTA's pull warps all write this word; the last one to finish wins
    a.timer[(size_t)blockIdx.x * kMegaTimerWords + kTimPull] = global_timer_ns();
}

// The whole routing step as one phase (all warps of the grid pull).
__device__ __forceinline__ void route_phase(const MegaRouteArgs& a, cg::grid_group& grid) {
  __shared__ RouteShared sh;
  route_layout_phase(a, grid, sh);
  const int warps = (int)blockDim.x / 32;
  route_pull_phase(a, sh, blockIdx.x * warps + (threadIdx.x >> 5), gridDim.x * warps);
}

__device__ __forceinline__ void finish_phase(const MegaFinishArgs& a, bool bump_epoch) {
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, me = ctx.rank, K = a.K, H = a.H, M = a.max_tokens, Kp = a.K + a.S;
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
  mega_stamp(a.timer, kTimFinishSync);
  if (alive) {
    const int* idx = reinterpret_cast<const int*>(ctx.ws[me] + a.in_off + in.idx);
    const float* w = reinterpret_cast<const float*>(ctx.ws[me] + a.in_off + in.w);
    const uint8_t* comb = ctx.ws[me] + a.comb_off;
    // small batches: several warps share a token, each reduces a span of columns (a multiple of the 64-piece step)
    const int units = H / 8;
    const int parts = max(1, min(8, total_warps / max(a.T, 1)));
    const int span = ((units + parts * 64 - 1) / (parts * 64)) * 64;
    for (int item = gw; item < a.T * parts; item += total_warps) {
      const int t = item / parts, part = item - t * parts;
      if (part * span >= units) continue;
      const int u_end = min(units, (part + 1) * span);
      // lane k holds slot k: its weight and whether it counts (shared experts: every token, weight one)
      float w_mine = 0.f;
      bool counts = false;
      if (lane < K) {
        const int e = idx[(size_t)t * K + lane];
        w_mine = w[(size_t)t * K + lane];
        counts = e >= 0 && e < a.E;
      } else if (lane < Kp) {
        w_mine = 1.f;
        counts = true;
      }
      const unsigned valid = __ballot_sync(0xffffffffu, counts);
      int4* out = reinterpret_cast<int4*>(reinterpret_cast<uint8_t*>(a.y) + (size_t)t * H * 2);
      const uint8_t* rows = comb + (size_t)t * Kp * H * 2;
      // two 16-byte columns per lane and step; the trip count is the same for every lane, which all take part in the shuffles
      for (int ub = part * span; ub < u_end; ub += 64) {
        const int u0 = ub + lane;
        const bool one = u0 < u_end, two = u0 + 32 < u_end;
        float a0[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, a1[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int kb = 0; kb < Kp; kb += 8) {     // eight slots' loads in flight at a time
          int4 v0[8], v1[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            if (kb + k < Kp && ((valid >> (kb + k)) & 1u)) {
              if (one) v0[k] = ld_cg_int4(rows + (size_t)(kb + k) * H * 2 + (size_t)u0 * 16);
              if (two) v1[k] = ld_cg_int4(rows + (size_t)(kb + k) * H * 2 + (size_t)(u0 + 32) * 16);
            }
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            if (kb + k < Kp && ((valid >> (kb + k)) & 1u)) {     // warp-uniform
              const float wk = __shfl_sync(0xffffffffu, w_mine, kb + k);
              const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&v0[k]);
              const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&v1[k]);
#pragma unroll
              for (int i = 0; i < 4; ++i) {   // product and sum rounded separately, as the CPU oracle does
                if (one) {
                  a0[2 * i] = __fadd_rn(a0[2 * i], __fmul_rn(wk, __low2float(h0[i])));
                  a0[2 * i + 1] = __fadd_rn(a0[2 * i + 1], __fmul_rn(wk, __high2float(h0[i])));
                }
                if (two) {
                  a1[2 * i] = __fadd_rn(a1[2 * i], __fmul_rn(wk, __low2float(h1[i])));
                  a1[2 * i + 1] = __fadd_rn(a1[2 * i + 1], __fmul_rn(wk, __high2float(h1[i])));
                }
              }
            }
          }
        }
        int4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
        if (one) {
#pragma unroll
          for (int i = 0; i < 4; ++i) oh[i] = __floats2bfloat162_rn(a0[2 * i], a0[2 * i + 1]);
          out[u0] = o;
        }
        if (two) {
#pragma unroll
          for (int i = 0; i < 4; ++i) oh[i] = __floats2bfloat162_rn(a1[2 * i], a1[2 * i + 1]);
          out[u0 + 32] = o;
        }
      }
    }
  }
  mega_stamp(a.timer, kTimEnd);
  if (bump_epoch && last_block_of_rank(ctl, kOpMega, gridDim.x)) {
    if (threadIdx.x == 0) ctl->epoch[kOpMega] = epoch;
  }
}

#endif  // __CUDACC__

}  // namespace dep
