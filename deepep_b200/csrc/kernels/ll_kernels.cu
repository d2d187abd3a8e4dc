// ep_dispatch_ll / ep_combine_ll: latency-oriented dispatch and combine for decode batches
// (at most 256 tokens per rank).
//
// One kernel per direction and no separate layout pass.  Dispatch: every rank pushes its tiny
// routing table ([T, K] expert ids and weights) to all peers and, at the same time, pushes each
// token row once per destination GPU into a fixed staging slot there, followed by a per-row
// release flag.  A receiver derives the expert-major layout (sorted by local expert, source rank,
// source token, slot) from the gathered tables with bit masks and popcounts in shared memory,
// then polls row flags and writes every output row.  Combine returns each expert row to a fixed
// (token, slot) slot at its source with a per-row flag; the source waits and computes
// sum_k w_k * row_k in slot order in fp32.
//
// Re-entrancy: epochs live in device memory and select one of two banks, flags hold epochs and
// are never cleared, a bank is reused only after the peers acknowledged the call before last.
// Nothing depends on host state, so both kernels can be captured in a CUDA graph.
//
// Parity: csrc/kernels/dispatch/low_latency/dispatch_server_dedup_kernel.h:37-58 and
// csrc/kernels/combine/low_latency/combine_server_dedup_kernel.h:102-127 of the reference
// (count exchange, cumsum, flagged packets, ping-pong banks; weights applied at the source).
#include <cooperative_groups.h>

#include "ll_api.h"

namespace dep {

constexpr int kLLThreads = 256;
constexpr int kLLWords = 8;  // 256 tokens as 8 x 32-bit masks

__device__ __forceinline__ int below8(const unsigned* m, int t) {
  int n = 0;
  const int w = t >> 5;
  for (int i = 0; i < w; ++i) n += __popc(m[i]);
  return n + __popc(m[w] & ((1u << (t & 31)) - 1u));
}
__device__ __forceinline__ int popc8(const unsigned* m) {
  int n = 0;
  for (int i = 0; i < kLLWords; ++i) n += __popc(m[i]);
  return n;
}
__device__ __forceinline__ bool counts_ll(const int* row, int k, int E) {
  int e = row[k];
  if (e < 0 || e >= E) return false;
  for (int j = 0; j < k; ++j)
    if (row[j] == e) return false;
  return true;
}

// ------------------------------------------------------------------------------------------ dispatch
__global__ void __launch_bounds__(kLLThreads) ep_dispatch_ll_kernel(const __grid_constant__ LLDispatchParams p) {
  const LLDispatchArgs& a = p.r[blockIdx.y];
  const WsLayout& lay = p.lay;
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, me = ctx.rank, M = lay.max_tokens, K = lay.topk, H = lay.hidden, E = a.E, Lx = E / P;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = kLLThreads / 32;
  const int gw = blockIdx.x * nwarps + warp, total_warps = gridDim.x * nwarps;
  Control* ctl = control_of(ctx.ws[me]);
  const unsigned long long epoch = ctl->epoch[kOpLLDispatch] + 1;
  const LLLayout ll = make_ll_layout(P, M, K, H);
  const long long bank_off = lay.ll + (long long)(epoch & 1) * ll.bank_bytes;
  const bool fp8 = a.mode != 0;
  const int nsf = H / 128, row_bytes = fp8 ? H : H * 2;

  __shared__ unsigned s_emask[kMaxExperts][kLLWords];   // [(source, local expert)] -> tokens
  __shared__ unsigned s_hit[kMaxRanks][kLLWords];       // tokens of source r that reach this rank
  __shared__ unsigned s_own[kMaxRanks][kLLWords];       // my tokens that reach rank d
  __shared__ int s_off[kMaxExperts];                    // first output row of (source, local expert)
  __shared__ int s_tot[kMaxExperts];
  __shared__ int s_T[kMaxRanks];
  __shared__ int s_rows;

  // phase stamps (nanoseconds since kernel start) of block 0, for diagnostics: Control::dbg[0..7]
  const unsigned long long t_start = global_timer_ns();
  auto stamp = [&](int i) { if (blockIdx.x == 0 && threadIdx.x == 0) ctl->dbg[i] = global_timer_ns() - t_start; };

  // ---- bank reuse: the call before last must have been consumed everywhere
  int ok = 1;
  if (threadIdx.x < P && epoch > 2)
    ok = wait_flag_ge(&ctl->ll_disp_ack[threadIdx.x], epoch - 2, ctx, kOpLLDispatch, 0, threadIdx.x);
  int alive = __syncthreads_and(ok);

  // ---- my own routing: which destinations does each token reach
  for (int i = threadIdx.x; i < kMaxRanks * kLLWords; i += kLLThreads) (&s_own[0][0])[i] = 0u;
  __syncthreads();
  for (int t = threadIdx.x; t < a.T; t += kLLThreads) {   // one thread per token: K independent loads, dedup in registers
    int row[kMaxTopk];
#pragma unroll
    for (int k = 0; k < kMaxTopk; ++k) {
      long long v = k < K ? a.topk_idx[(size_t)t * K + k] : -1;
      row[k] = (v < 0 || v >= E) ? -1 : (int)v;
    }
#pragma unroll
    for (int k = 0; k < kMaxTopk; ++k)
      if (k < K && counts_ll(row, k, E)) atomicOr(&s_own[row[k] / Lx][t >> 5], 1u << (t & 31));
  }
  __syncthreads();

  stamp(0);
  if (alive) {
    // ---- routing table to every peer (block 0), rows to their destinations (all warps)
    if (blockIdx.x == 0) {
      const int n = a.T * K;
      for (int i = threadIdx.x; i < P * n; i += kLLThreads) {
        const int d = i / n, j = i - d * n;
        long long v = a.topk_idx[j];
        uint8_t* base = ctx.ws[d] + bank_off;
        reinterpret_cast<int*>(base + ll.gather_idx)[(size_t)me * M * K + j] = (v < 0 || v >= E) ? -1 : (int)v;
        reinterpret_cast<float*>(base + ll.gather_w)[(size_t)me * M * K + j] = a.topk_w ? a.topk_w[j] : 0.f;
      }
      if (threadIdx.x < P) reinterpret_cast<int*>(ctx.ws[threadIdx.x] + bank_off + ll.gather_hdr)[me * 4] = a.T;
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x < P)
        st_release_sys(reinterpret_cast<unsigned long long*>(ctx.ws[threadIdx.x] + bank_off + ll.idx_flag) + me, epoch);
    }
    // with more than one block, block 0 only publishes the routing table so that it leaves as early as possible
    const int send_first = gridDim.x > 1 ? 1 : 0;
    const int send_warps = (gridDim.x - send_first) * nwarps;
    for (int item = (blockIdx.x - send_first) * nwarps + warp; item < a.T * P && (int)blockIdx.x >= send_first; item += send_warps) {
      const int t = item / P, d = (me + item % P) % P;
      if (!((s_own[d][t >> 5] >> (t & 31)) & 1u)) continue;
      const int j = below8(s_own[d], t);
      uint8_t* base = ctx.ws[d] + bank_off;
      uint8_t* dst = base + ll.stage + ((size_t)me * M + j) * ll.msg_bytes;
      if (a.mode == 2) {  // bf16 -> e4m3 with one fp32 scale per 128 values, straight into the peer
        // a lane owns 8 consecutive values (16 B); 16 lanes cover one 128-value block, a warp step covers two blocks
        const int4* src = reinterpret_cast<const int4*>(reinterpret_cast<const uint8_t*>(a.x) + (size_t)t * H * 2);
        const int units = H / 8, half = lane >> 4;
        constexpr int U = 8;
        for (int u0 = 0; u0 < units; u0 += 32 * U) {
          int4 v[U];
#pragma unroll
          for (int i = 0; i < U; ++i) {
            const int u = u0 + i * 32 + lane;
            if (u < units) v[i] = __ldg(src + u);
          }
#pragma unroll
          for (int i = 0; i < U; ++i) {
            const int u = u0 + i * 32 + lane;
            if (u0 + i * 32 >= units) break;           // warp-uniform: H is a multiple of 128, so steps are all-or-nothing per half
            float f[8];
            const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
            for (int j = 0; j < 4; ++j) { f[2 * j] = __low2float(hh[j]); f[2 * j + 1] = __high2float(hh[j]); }
            float amax = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            amax = fmaxf(amax, 1e-4f);
            const float inv = __frcp_rn(amax) * 448.0f;   // torch evaluates `448 / amax` (scalar / tensor) as reciprocal, then multiply
            uint32_t q[2] = {0u, 0u};
#pragma unroll
            for (int j = 0; j < 8; ++j)
              q[j >> 2] |= (uint32_t)__nv_cvt_float_to_fp8(f[j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * (j & 3));
            if (u < units) {
              *reinterpret_cast<uint2*>(dst + (size_t)u * 8) = make_uint2(q[0], q[1]);
              if ((lane & 15) == 0) reinterpret_cast<float*>(dst + H)[(u0 + i * 32) / 16 + half] = amax / 448.0f;
            }
          }
        }
      } else {
        warp_copy_row1(reinterpret_cast<int4*>(dst), reinterpret_cast<const int4*>(reinterpret_cast<const uint8_t*>(a.x) + (size_t)t * row_bytes),
                       row_bytes / 16, lane);
        if (a.mode == 1)
          for (int q = lane; q < nsf; q += 32) reinterpret_cast<float*>(dst + H)[q] = a.x_sf[(size_t)t * nsf + q];
      }
      __threadfence_system();
      __syncwarp();
      if (lane == 0) st_release_sys(reinterpret_cast<unsigned long long*>(base + ll.row_flag) + (size_t)me * M + j, epoch);
    }

    stamp(1);
    // ---- receive: wait for all routing tables, derive the layout
    uint8_t* mine = ctx.ws[me] + bank_off;
    ok = 1;
    if (threadIdx.x < P)
      ok = wait_flag_ge(reinterpret_cast<unsigned long long*>(mine + ll.idx_flag) + threadIdx.x, epoch, ctx, kOpLLDispatch, 1, threadIdx.x);
    alive = __syncthreads_and(ok);
  }
  if (alive) {
    uint8_t* mine = ctx.ws[me] + bank_off;
    const int* gidx = reinterpret_cast<const int*>(mine + ll.gather_idx);
    const float* gw_ = reinterpret_cast<const float*>(mine + ll.gather_w);
    stamp(2);
    if (threadIdx.x < kMaxRanks)
      s_T[threadIdx.x] = threadIdx.x < P ? __ldcg(reinterpret_cast<const int*>(mine + ll.gather_hdr) + threadIdx.x * 4) : 0;
    for (int i = threadIdx.x; i < E * kLLWords; i += kLLThreads) (&s_emask[0][0])[i] = 0u;
    for (int i = threadIdx.x; i < kMaxRanks * kLLWords; i += kLLThreads) (&s_hit[0][0])[i] = 0u;
    __syncthreads();
    for (int i = threadIdx.x; i < P * M; i += kLLThreads) {   // one thread per (source, token)
      const int r = i / M, t = i - r * M;
      if (t >= s_T[r]) continue;
      int row[kMaxTopk];
#pragma unroll
      for (int k = 0; k < kMaxTopk; ++k) row[k] = k < K ? __ldcg(gidx + ((size_t)r * M + t) * K + k) : -1;
#pragma unroll
      for (int k = 0; k < kMaxTopk; ++k) {
        if (k < K && counts_ll(row, k, E) && row[k] / Lx == me) {
          atomicOr(&s_emask[r * Lx + (row[k] - me * Lx)][t >> 5], 1u << (t & 31));
          atomicOr(&s_hit[r][t >> 5], 1u << (t & 31));
        }
      }
    }
    __syncthreads();
    for (int l = threadIdx.x; l < Lx; l += kLLThreads) {
      int tot = 0;
      for (int r = 0; r < P; ++r) tot += popc8(s_emask[r * Lx + l]);
      s_tot[l] = tot;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int run = 0;
      for (int l = 0; l < Lx; ++l) { int v = s_tot[l]; s_tot[l] = run; run += v; }
      s_rows = run;
    }
    __syncthreads();
    for (int l = threadIdx.x; l < Lx; l += kLLThreads) {
      int run = s_tot[l];
      for (int r = 0; r < P; ++r) { s_off[r * Lx + l] = run; run += popc8(s_emask[r * Lx + l]); }
      if (blockIdx.x == 0) {
        a.expert_offsets[l] = s_tot[l];
        a.expert_counts[l] = run - s_tot[l];
        if (a.mailbox) a.mailbox[4 + l] = run - s_tot[l];
      }
    }
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      a.expert_offsets[Lx] = s_rows;
      *a.num_rows = s_rows;
      if (a.mailbox) {
        a.mailbox[0] = s_rows;
        __threadfence_system();
        a.mailbox[3] = (int)(epoch & 0x7fffffff);
      }
    }

    stamp(3);
    // ---- poll row flags and write the output rows
    const uint8_t* stage = mine + ll.stage;
    uint8_t* recv_x = reinterpret_cast<uint8_t*>(a.recv_x);
    for (int item = gw; item < P * M; item += total_warps) {
      const int r = (me + item / M) % P, t = item % M;
      if (t >= s_T[r] || !((s_hit[r][t >> 5] >> (t & 31)) & 1u)) continue;
      const int j = below8(s_hit[r], t);
      int got = 1;
      if (lane == 0)
        got = wait_flag_ge(reinterpret_cast<unsigned long long*>(mine + ll.row_flag) + (size_t)r * M + j, epoch, ctx, kOpLLDispatch, 2, r);
      if (!__shfl_sync(0xffffffffu, got, 0)) break;
      int idx_row[kMaxTopk], rows[kMaxTopk], n = 0;
      for (int k = 0; k < K; ++k) idx_row[k] = __ldcg(gidx + ((size_t)r * M + t) * K + k);
      for (int k = 0; k < K; ++k) {
        if (!counts_ll(idx_row, k, E) || idx_row[k] / Lx != me) continue;
        const int el = idx_row[k] - me * Lx;
        const int out_row = s_off[r * Lx + el] + below8(s_emask[r * Lx + el], t);
        if (out_row >= a.capacity) continue;
        rows[n++] = out_row;
        if (lane == 0) {
          a.recv_row_src[out_row] = (r * M + t) * K + k;
          a.recv_w[out_row] = __ldcg(gw_ + ((size_t)r * M + t) * K + k);
        }
      }
      const uint8_t* src = stage + ((size_t)r * M + j) * ll.msg_bytes;
      int4* outs[kMaxTopk];
      for (int i = 0; i < n; ++i) outs[i] = reinterpret_cast<int4*>(recv_x + (size_t)rows[i] * row_bytes);
      warp_copy_row<8>(outs, n, reinterpret_cast<const int4*>(src), row_bytes / 16, lane);
      if (fp8)
        for (int q = lane; q < nsf; q += 32) {
          const float v = __ldcg(reinterpret_cast<const float*>(src + H) + q);
          for (int i = 0; i < n; ++i) a.recv_sf[(size_t)rows[i] * nsf + q] = v;
        }
    }
  }

  stamp(4);
  if (last_block_of_rank(ctl, kOpLLDispatch, gridDim.x)) {
    stamp(5);
    if (!ld_volatile_int(&ctl->abort) && threadIdx.x < P)
      st_release_sys(&control_of(ctx.ws[threadIdx.x])->ll_disp_ack[me], epoch);
    if (threadIdx.x == 0) ctl->epoch[kOpLLDispatch] = epoch;
  }
}

cudaError_t launch_ll_dispatch(const LLDispatchParams& p, int nranks, int blocks, cudaStream_t stream) {
  dim3 grid(blocks, nranks), block(kLLThreads);
  void* args[] = {const_cast<LLDispatchParams*>(&p)};
  return cudaLaunchCooperativeKernel((const void*)ep_dispatch_ll_kernel, grid, block, args, 0, stream);
}

// ------------------------------------------------------------------------------------------ combine
__global__ void __launch_bounds__(kLLThreads) ep_combine_ll_kernel(const __grid_constant__ LLCombineParams p) {
  const LLCombineArgs& a = p.r[blockIdx.y];
  const WsLayout& lay = p.lay;
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, me = ctx.rank, M = lay.max_tokens, K = lay.topk, H = lay.hidden;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = kLLThreads / 32;
  const int gw = blockIdx.x * nwarps + warp, total_warps = gridDim.x * nwarps;
  Control* ctl = control_of(ctx.ws[me]);
  const unsigned long long epoch = ctl->epoch[kOpLLCombine] + 1;
  const LLLayout ll = make_ll_layout(P, M, K, H);
  const long long bank_off = lay.ll + (long long)(epoch & 1) * ll.bank_bytes;
  const int row_bytes = H * 2, units = H / 8;

  int ok = 1;
  if (threadIdx.x < P && epoch > 2)
    ok = wait_flag_ge(&ctl->ll_comb_ack[threadIdx.x], epoch - 2, ctx, kOpLLCombine, 0, threadIdx.x);
  const int alive = __syncthreads_and(ok);

  if (alive) {
    // ---- return every expert row to its (token, slot) slot at the source
    const int R = *a.num_rows;
    for (int r = gw; r < R; r += total_warps) {
      const int code = a.recv_row_src[r];
      if (code < 0) continue;
      const int src = code / (M * K), rem = code - src * M * K;
      uint8_t* base = ctx.ws[src] + bank_off;
      int4* dst = reinterpret_cast<int4*>(base + ll.ret + (size_t)rem * row_bytes);
      const int4* from = reinterpret_cast<const int4*>(reinterpret_cast<const uint8_t*>(a.x) + (size_t)r * row_bytes);
      warp_copy_row1(dst, from, units, lane);
      __threadfence_system();
      __syncwarp();
      if (lane == 0) st_release_sys(reinterpret_cast<unsigned long long*>(base + ll.ret_flag) + rem, epoch);
    }
    // ---- weighted sum at the source, slot order, fp32
    uint8_t* mine = ctx.ws[me] + bank_off;
    const unsigned long long* flags = reinterpret_cast<const unsigned long long*>(mine + ll.ret_flag);
    constexpr int kSplit = 4;                      // warps per token: each reduces a quarter of the columns
    const int span = ((units + kSplit * 64 - 1) / (kSplit * 64)) * 64;   // columns per warp, a multiple of the 64-unit step
    for (int item = gw; item < a.T * kSplit; item += total_warps) {
      const int t = item / kSplit, part = item - t * kSplit;
      int idx_row[kMaxTopk];
      float w_row[kMaxTopk];
      unsigned valid = 0;
      for (int k = 0; k < K; ++k) {
        long long v = a.topk_idx[(size_t)t * K + k];
        idx_row[k] = (v < 0 || v >= a.E) ? -1 : (int)v;
        w_row[k] = a.topk_w[(size_t)t * K + k];
      }
      for (int k = 0; k < K; ++k)
        if (counts_ll(idx_row, k, a.E)) valid |= 1u << k;
      int got = 1;
      if (lane == 0)
        for (unsigned m = valid; m && got; m &= m - 1)
          got = wait_flag_ge(flags + (size_t)t * K + (__ffs(m) - 1), epoch, ctx, kOpLLCombine, 1, me);
      if (!__shfl_sync(0xffffffffu, got, 0)) break;
      const uint8_t* rows = mine + ll.ret + (size_t)t * K * row_bytes;
      int4* out = reinterpret_cast<int4*>(reinterpret_cast<uint8_t*>(a.out) + (size_t)t * row_bytes);
      const int u_end = min(units, (part + 1) * span);
      for (int u0 = part * span + lane; u0 < u_end; u0 += 64) {     // two 16-byte columns per step; all slots' loads issued first
        const bool two = u0 + 32 < u_end;
        int4 v0[kMaxTopk], v1[kMaxTopk];
#pragma unroll
        for (int k = 0; k < kMaxTopk; ++k) {
          if (k < K && ((valid >> k) & 1u)) {
            v0[k] = ld_cg_int4(rows + (size_t)k * row_bytes + (size_t)u0 * 16);
            if (two) v1[k] = ld_cg_int4(rows + (size_t)k * row_bytes + (size_t)(u0 + 32) * 16);
          }
        }
        float a0[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, a1[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int k = 0; k < kMaxTopk; ++k) {
          if (k < K && ((valid >> k) & 1u)) {
            const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&v0[k]);
            const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&v1[k]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              // product and sum are rounded separately (no fused multiply-add), as the CPU oracle does
              a0[2 * i] = __fadd_rn(a0[2 * i], __fmul_rn(w_row[k], __low2float(h0[i])));
              a0[2 * i + 1] = __fadd_rn(a0[2 * i + 1], __fmul_rn(w_row[k], __high2float(h0[i])));
              if (two) {
                a1[2 * i] = __fadd_rn(a1[2 * i], __fmul_rn(w_row[k], __low2float(h1[i])));
                a1[2 * i + 1] = __fadd_rn(a1[2 * i + 1], __fmul_rn(w_row[k], __high2float(h1[i])));
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

  if (last_block_of_rank(ctl, kOpLLCombine, gridDim.x)) {
    if (!ld_volatile_int(&ctl->abort) && threadIdx.x < P)
      st_release_sys(&control_of(ctx.ws[threadIdx.x])->ll_comb_ack[me], epoch);
    if (threadIdx.x == 0) ctl->epoch[kOpLLCombine] = epoch;
  }
}

cudaError_t launch_ll_combine(const LLCombineParams& p, int nranks, int blocks, cudaStream_t stream) {
  dim3 grid(blocks, nranks), block(kLLThreads);
  void* args[] = {const_cast<LLCombineParams*>(&p)};
  return cudaLaunchCooperativeKernel((const void*)ep_combine_ll_kernel, grid, block, args, 0, stream);
}

}  // namespace dep
