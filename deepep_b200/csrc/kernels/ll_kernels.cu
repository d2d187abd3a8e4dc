// ep_dispatch_ll / ep_combine_ll: latency-oriented dispatch and combine for decode batches
// (at most 256 tokens per rank).
//
// One kernel per direction and no separate layout pass.  Dispatch: every rank pushes its tiny
// routing table ([T, K] expert ids and weights) to all peers (one block per peer, 16-byte stores)
// and, at the same time, pushes each token row once per destination GPU into a fixed staging slot
// there, as four column parts that different warps carry, each followed by its own release flag.
// A receiver derives the expert-major layout (sorted by local expert, source rank, source token,
// slot) from the gathered tables with bit masks and popcounts in shared memory, then polls the
// part flags and writes every output row.  Combine returns each expert row, again part by part, to
// a fixed (token, slot) slot at its source; the source waits per part and computes
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

constexpr int kLLThreads = 512;
constexpr int kLLSendWarps = 8;      // dispatch: warps that push rows; the other warps of the block derive the layout meanwhile
constexpr int kLLWords = 8;  // 256 tokens as 8 x 32-bit masks

// A row travels as kLLParts column parts, each with its own flag, so that a row is spread over several warps on both
// sides.  Parts are whole groups of 128 values (the granularity of the fp8 scales): part p covers values [v0, v1).
struct LLPart { int v0, v1, b0, b1; };
__device__ __forceinline__ LLPart ll_part(int H, int p) {
  const int nblk = (H + 127) / 128, bpp = (nblk + kLLParts - 1) / kLLParts;
  LLPart r;
  r.b0 = min(nblk, p * bpp); r.b1 = min(nblk, (p + 1) * bpp);
  r.v0 = min(H, r.b0 * 128); r.v1 = min(H, r.b1 * 128);
  return r;
}

// Flags of finished parts are published together: lane i of the warp keeps the address of the i-th pending flag.
struct PendingFlags {
  unsigned long long* mine = nullptr;
  int count = 0;
  __device__ __forceinline__ void add(unsigned long long* flag, unsigned long long epoch, int lane) {
    if (count == 32) publish(epoch, lane);
    if (lane == count) mine = flag;
    ++count;
  }
  // every lane's stores are ordered before the flags by the warp barrier + release
  __device__ __forceinline__ void publish(unsigned long long epoch, int lane) {
    __syncwarp();
    if (lane < count) st_release_sys(mine, epoch);
    count = 0;
  }
};

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
template <bool kProfile>
__global__ void __launch_bounds__(kLLThreads) ep_dispatch_ll_kernel(const __grid_constant__ LLDispatchParams p) {
  const LLDispatchArgs& a = p.r[blockIdx.y];
  const WsLayout& lay = p.lay;
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, me = ctx.rank, M = lay.max_tokens, K = lay.topk, H = lay.hidden, E = a.E, Lx = E / P;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = kLLThreads / 32;
  // consecutive work items go to different SMs, so a short list of items spreads over the whole GPU
  const int gw = warp * gridDim.x + blockIdx.x, total_warps = gridDim.x * nwarps;
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
  __shared__ int s_fail;                                // a wait of the layout warps ran out

  // profile instantiation only: phase stamps (nanoseconds since kernel start) of block 0 in Control::dbg[0..7]; the
  // first thread of the sending warps and the first thread of the layout warps stamp their own phases
  unsigned long long t_start = 0;
  if constexpr (kProfile) t_start = global_timer_ns();
  auto stamp = [&](int i, int who = 0) {
    if constexpr (kProfile)
      if (blockIdx.x == 0 && (int)threadIdx.x == who) ctl->dbg[i] = global_timer_ns() - t_start;
  };
  constexpr int kLayoutFirst = kLLSendWarps * 32, LT = kLLThreads - kLayoutFirst;   // the layout warps and their thread count
  const int lt = (int)threadIdx.x - kLayoutFirst;
  auto layout_sync = [&]() { asm volatile("bar.sync 1, %0;" ::"n"(LT) : "memory"); };
  if (threadIdx.x == 0) s_fail = 0;

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
    // ---- routing table: block b writes it to peer (me + b) % P (16-byte stores when the table allows), so all peers are
    // served at once and the table leaves in a couple of microseconds; rows to their destinations (all warps)
    {
      const int n = a.T * K;
      const bool vec = ((M * K) & 3) == 0 && (reinterpret_cast<uintptr_t>(a.topk_idx) & 15) == 0 &&
                       (!a.topk_w || (reinterpret_cast<uintptr_t>(a.topk_w) & 15) == 0);
      for (int s = blockIdx.x; s < P; s += gridDim.x) {
        const int d = (me + s) % P;
        uint8_t* base = ctx.ws[d] + bank_off;
        int* gi = reinterpret_cast<int*>(base + ll.gather_idx) + (size_t)me * M * K;
        float* gwt = reinterpret_cast<float*>(base + ll.gather_w) + (size_t)me * M * K;
        const int n4 = vec ? n / 4 : 0;
        for (int i = threadIdx.x; i < n4; i += kLLThreads) {
          const longlong2 lo = __ldg(reinterpret_cast<const longlong2*>(a.topk_idx) + 2 * i);
          const longlong2 hi = __ldg(reinterpret_cast<const longlong2*>(a.topk_idx) + 2 * i + 1);
          const long long v[4] = {lo.x, lo.y, hi.x, hi.y};
          int o[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) o[j] = (v[j] < 0 || v[j] >= E) ? -1 : (int)v[j];
          reinterpret_cast<int4*>(gi)[i] = make_int4(o[0], o[1], o[2], o[3]);
          reinterpret_cast<float4*>(gwt)[i] = a.topk_w ? __ldg(reinterpret_cast<const float4*>(a.topk_w) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        for (int j = n4 * 4 + threadIdx.x; j < n; j += kLLThreads) {
          const long long v = a.topk_idx[j];
          gi[j] = (v < 0 || v >= E) ? -1 : (int)v;
          gwt[j] = a.topk_w ? a.topk_w[j] : 0.f;
        }
        if (threadIdx.x == 0) reinterpret_cast<int*>(base + ll.gather_hdr)[me * 4] = a.T;
        __syncthreads();   // the block's stores are ordered before the flag by the block barrier + release
        if (threadIdx.x == 0) st_release_sys(reinterpret_cast<unsigned long long*>(base + ll.idx_flag) + me, epoch);
      }
    }
    stamp(6);
    uint8_t* mine = ctx.ws[me] + bank_off;
    const int* gidx = reinterpret_cast<const int*>(mine + ll.gather_idx);
    if (warp < kLLSendWarps) {
    // ================================================================ sending warps: every row part to its destination
    PendingFlags pending;
    for (int item = warp * gridDim.x + blockIdx.x; item < a.T * P * kLLParts; item += gridDim.x * kLLSendWarps) {
      const int part = item % kLLParts, td = item / kLLParts;
      const int t = td / P, d = (me + td % P) % P;
      if (!((s_own[d][t >> 5] >> (t & 31)) & 1u)) continue;
      const LLPart pr = ll_part(H, part);
      if (pr.v0 >= pr.v1) continue;
      const int j = below8(s_own[d], t);
      uint8_t* base = ctx.ws[d] + bank_off;
      uint8_t* dst = base + ll.stage + ((size_t)me * M + j) * ll.msg_bytes;
      if (a.mode == 2) {  // bf16 -> e4m3 with one fp32 scale per 128 values, straight into the peer
        // a lane owns 8 consecutive values (16 B); 16 lanes cover one 128-value group, a warp step covers two groups
        const int4* src = reinterpret_cast<const int4*>(reinterpret_cast<const uint8_t*>(a.x) + (size_t)t * H * 2);
        const int u_lo = pr.v0 / 8, u_hi = pr.v1 / 8, half = lane >> 4;
        constexpr int U = 8;
        for (int u0 = u_lo; u0 < u_hi; u0 += 32 * U) {
          int4 v[U];
#pragma unroll
          for (int i = 0; i < U; ++i) {
            const int u = u0 + i * 32 + lane;
            if (u < u_hi) v[i] = __ldg(src + u);
          }
#pragma unroll
          for (int i = 0; i < U; ++i) {
            const int u = u0 + i * 32 + lane;
            if (u0 + i * 32 >= u_hi) break;           // warp-uniform
            float f[8];
            if (u >= u_hi) v[i] = make_int4(0, 0, 0, 0);   // groups are whole, so a step is all-or-nothing per half warp
            const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
            for (int q = 0; q < 4; ++q) { f[2 * q] = __low2float(hh[q]); f[2 * q + 1] = __high2float(hh[q]); }
            float amax = 0.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) amax = fmaxf(amax, fabsf(f[q]));
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            amax = fmaxf(amax, 1e-4f);
            const float inv = __frcp_rn(amax) * 448.0f;   // torch evaluates `448 / amax` (scalar / tensor) as reciprocal, then multiply
            uint32_t q2[2] = {0u, 0u};
#pragma unroll
            for (int q = 0; q < 8; ++q)
              q2[q >> 2] |= (uint32_t)__nv_cvt_float_to_fp8(f[q] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * (q & 3));
            if (u < u_hi) {
              *reinterpret_cast<uint2*>(dst + (size_t)u * 8) = make_uint2(q2[0], q2[1]);
              if ((lane & 15) == 0) reinterpret_cast<float*>(dst + H)[(u0 + i * 32) / 16 + half] = amax / 448.0f;
            }
          }
        }
      } else {
        const int b_lo = fp8 ? pr.v0 : pr.v0 * 2, b_hi = fp8 ? pr.v1 : pr.v1 * 2;   // byte range of the part in the row
        warp_copy_row1(reinterpret_cast<int4*>(dst + b_lo),
                       reinterpret_cast<const int4*>(reinterpret_cast<const uint8_t*>(a.x) + (size_t)t * row_bytes + b_lo),
                       (b_hi - b_lo) / 16, lane);
        if (a.mode == 1)
          for (int q = pr.b0 + lane; q < pr.b1; q += 32) reinterpret_cast<float*>(dst + H)[q] = a.x_sf[(size_t)t * nsf + q];
      }
      stamp(7);
      pending.add(reinterpret_cast<unsigned long long*>(base + ll.row_flag) + ((size_t)me * M + j) * kLLParts + part, epoch, lane);
    }
    pending.publish(epoch, lane);
    stamp(1);
    } else {
    // ================================================================ layout warps: wait for all routing tables, derive the layout
    int ok = 1;
    if (lt < P)
      ok = wait_flag_ge(reinterpret_cast<unsigned long long*>(mine + ll.idx_flag) + lt, epoch, ctx, kOpLLDispatch, 1, lt);
    if (!ok) s_fail = 1;
    layout_sync();
    stamp(2, kLayoutFirst);
    if (!s_fail) {
    if (lt < kMaxRanks)
      s_T[lt] = lt < P ? __ldcg(reinterpret_cast<const int*>(mine + ll.gather_hdr) + lt * 4) : 0;
    for (int i = lt; i < E * kLLWords; i += LT) (&s_emask[0][0])[i] = 0u;
    for (int i = lt; i < kMaxRanks * kLLWords; i += LT) (&s_hit[0][0])[i] = 0u;
    layout_sync();
    int maxT = 1;
    for (int r = 0; r < P; ++r) maxT = max(maxT, min(s_T[r], M));
    // one thread per (source, token); the loads of four items are issued before the first of them is used
    constexpr int kBatch = 4;
    for (int i0 = lt; i0 < P * maxT; i0 += LT * kBatch) {
      int row[kBatch][kMaxTopk];
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        const int i = i0 + b * LT, r = i / maxT, t = i - r * maxT;
        const bool live = i < P * maxT && t < s_T[r];
#pragma unroll
        for (int k = 0; k < kMaxTopk; ++k) row[b][k] = (live && k < K) ? __ldcg(gidx + ((size_t)r * M + t) * K + k) : -1;
      }
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        const int i = i0 + b * LT, r = i / maxT, t = i - r * maxT;
        if (i >= P * maxT) break;
#pragma unroll
        for (int k = 0; k < kMaxTopk; ++k) {
          if (k < K && counts_ll(row[b], k, E) && row[b][k] / Lx == me) {
            atomicOr(&s_emask[r * Lx + (row[b][k] - me * Lx)][t >> 5], 1u << (t & 31));
            atomicOr(&s_hit[r][t >> 5], 1u << (t & 31));
          }
        }
      }
    }
    layout_sync();
    for (int l = lt; l < Lx; l += LT) {
      int tot = 0;
      for (int r = 0; r < P; ++r) tot += popc8(s_emask[r * Lx + l]);
      s_tot[l] = tot;
    }
    layout_sync();
    if (lt == 0) {
      int run = 0;
      for (int l = 0; l < Lx; ++l) { int v = s_tot[l]; s_tot[l] = run; run += v; }
      s_rows = run;
    }
    layout_sync();
    for (int l = lt; l < Lx; l += LT) {
      int run = s_tot[l];
      for (int r = 0; r < P; ++r) { s_off[r * Lx + l] = run; run += popc8(s_emask[r * Lx + l]); }
      if (blockIdx.x == 0) {
        a.expert_offsets[l] = s_tot[l];
        a.expert_counts[l] = run - s_tot[l];
        if (a.mailbox) a.mailbox[4 + l] = run - s_tot[l];
      }
    }
    layout_sync();
    if (blockIdx.x == 0 && lt == 0) {
      a.expert_offsets[Lx] = s_rows;
      *a.num_rows = s_rows;
      if (a.mailbox) {
        a.mailbox[0] = s_rows;
        __threadfence_system();
        a.mailbox[3] = (int)(epoch & 0x7fffffff);
      }
    }

    }
    stamp(3, kLayoutFirst);
    }
    // ---- both halves of the block meet: the rows are on their way and the layout is known
    __syncthreads();
    alive = !s_fail;
  }
  if (alive) {
    uint8_t* mine = ctx.ws[me] + bank_off;
    const int* gidx = reinterpret_cast<const int*>(mine + ll.gather_idx);
    const float* gw_ = reinterpret_cast<const float*>(mine + ll.gather_w);
    int maxT = 1;
    for (int r = 0; r < P; ++r) maxT = max(maxT, min(s_T[r], M));

    // ---- poll row flags and write the output rows
    const uint8_t* stage = mine + ll.stage;
    uint8_t* recv_x = reinterpret_cast<uint8_t*>(a.recv_x);
    // a staged row is materialised part by part, by whichever warp draws the part
    for (int item = gw; item < P * maxT * kLLParts; item += total_warps) {
      const int part = item % kLLParts, it = item / kLLParts;
      const int r = (me + it / maxT) % P, t = it % maxT;
      if (t >= s_T[r] || !((s_hit[r][t >> 5] >> (t & 31)) & 1u)) continue;
      const LLPart pr = ll_part(H, part);
      if (pr.v0 >= pr.v1) continue;
      const int j = below8(s_hit[r], t);
      int idx_row[kMaxTopk], rows[kMaxTopk], n = 0;
      for (int k = 0; k < K; ++k) idx_row[k] = __ldcg(gidx + ((size_t)r * M + t) * K + k);   // issued before the flag wait
      int got = 1;
      if (lane == 0)
        got = wait_flag_ge(reinterpret_cast<unsigned long long*>(mine + ll.row_flag) + ((size_t)r * M + j) * kLLParts + part, epoch,
                           ctx, kOpLLDispatch, 2, r);
      if (!__shfl_sync(0xffffffffu, got, 0)) break;
      for (int k = 0; k < K; ++k) {
        if (!counts_ll(idx_row, k, E) || idx_row[k] / Lx != me) continue;
        const int el = idx_row[k] - me * Lx;
        const int out_row = s_off[r * Lx + el] + below8(s_emask[r * Lx + el], t);
        if (out_row >= a.capacity) continue;
        rows[n++] = out_row;
        if (lane == 0 && part == 0) {
          a.recv_row_src[out_row] = (r * M + t) * K + k;
          a.recv_w[out_row] = __ldcg(gw_ + ((size_t)r * M + t) * K + k);
        }
      }
      const uint8_t* src = stage + ((size_t)r * M + j) * ll.msg_bytes;
      const int b_lo = fp8 ? pr.v0 : pr.v0 * 2, b_hi = fp8 ? pr.v1 : pr.v1 * 2;
      int4* outs[kMaxTopk];
      for (int i = 0; i < n; ++i) outs[i] = reinterpret_cast<int4*>(recv_x + (size_t)rows[i] * row_bytes + b_lo);
      warp_copy_row<8>(outs, n, reinterpret_cast<const int4*>(src + b_lo), (b_hi - b_lo) / 16, lane);
      if (fp8)
        for (int q = pr.b0 + lane; q < pr.b1; q += 32) {
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
  const void* fn = p.profile ? (const void*)ep_dispatch_ll_kernel<true> : (const void*)ep_dispatch_ll_kernel<false>;
  return cudaLaunchCooperativeKernel(fn, grid, block, args, 0, stream);
}

// ------------------------------------------------------------------------------------------ combine
template <bool kProfile>
__global__ void __launch_bounds__(kLLThreads) ep_combine_ll_kernel(const __grid_constant__ LLCombineParams p) {
  const LLCombineArgs& a = p.r[blockIdx.y];
  const WsLayout& lay = p.lay;
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, me = ctx.rank, M = lay.max_tokens, K = lay.topk, H = lay.hidden;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = kLLThreads / 32;
  // consecutive work items go to different SMs, so a short list of items spreads over the whole GPU
  const int gw = warp * gridDim.x + blockIdx.x, total_warps = gridDim.x * nwarps;
  Control* ctl = control_of(ctx.ws[me]);
  const unsigned long long epoch = ctl->epoch[kOpLLCombine] + 1;
  const LLLayout ll = make_ll_layout(P, M, K, H);
  const long long bank_off = lay.ll + (long long)(epoch & 1) * ll.bank_bytes;
  const int row_bytes = H * 2;
  // profile instantiation only: phase stamps (nanoseconds since kernel start) of block 0 in Control::dbg[8..15]
  unsigned long long t_start = 0;
  if constexpr (kProfile) t_start = global_timer_ns();
  auto stamp = [&](int i) {
    if constexpr (kProfile)
      if (blockIdx.x == 0 && threadIdx.x == 0) ctl->dbg[8 + i] = global_timer_ns() - t_start;
  };

  int ok = 1;
  if (threadIdx.x < P && epoch > 2)
    ok = wait_flag_ge(&ctl->ll_comb_ack[threadIdx.x], epoch - 2, ctx, kOpLLCombine, 0, threadIdx.x);
  const int alive = __syncthreads_and(ok);
  stamp(0);

  if (alive) {
    // ---- return every expert row, part by part, to its (token, slot) slot at the source
    const int R = *a.num_rows;
    PendingFlags pending;
    for (int item = gw; item < R * kLLParts; item += total_warps) {
      const int r = item / kLLParts, part = item % kLLParts;
      const int code = a.recv_row_src[r];
      if (code < 0) continue;
      const LLPart pr = ll_part(H, part);
      if (pr.v0 >= pr.v1) continue;
      const int src = code / (M * K), rem = code - src * M * K;
      uint8_t* base = ctx.ws[src] + bank_off;
      int4* dst = reinterpret_cast<int4*>(base + ll.ret + (size_t)rem * row_bytes + (size_t)pr.v0 * 2);
      const int4* from = reinterpret_cast<const int4*>(reinterpret_cast<const uint8_t*>(a.x) + (size_t)r * row_bytes + (size_t)pr.v0 * 2);
      warp_copy_row1(dst, from, (pr.v1 - pr.v0) / 8, lane);
      pending.add(reinterpret_cast<unsigned long long*>(base + ll.ret_flag) + (size_t)rem * kLLParts + part, epoch, lane);
    }
    pending.publish(epoch, lane);
    stamp(1);
    // ---- weighted sum at the source, slot order, fp32: two warps per (token, part), each a half of the part's columns
    uint8_t* mine = ctx.ws[me] + bank_off;
    const unsigned long long* flags = reinterpret_cast<const unsigned long long*>(mine + ll.ret_flag);
    for (int item = gw; item < a.T * kLLParts * 2; item += total_warps) {
      const int t = item / (kLLParts * 2), sub = item % (kLLParts * 2), part = sub >> 1, half = sub & 1;
      const LLPart pr = ll_part(H, part);
      if (pr.v0 >= pr.v1) continue;
      // lane k holds slot k: expert, weight, whether it counts (in range, first occurrence)
      long long e = -1;
      float w = 0.f;
      if (lane < K) {
        e = a.topk_idx[(size_t)t * K + lane];
        w = a.topk_w[(size_t)t * K + lane];
      }
      bool counts = lane < K && e >= 0 && e < a.E;
      for (int z = 0; z < K; ++z) {
        const long long ez = __shfl_sync(0xffffffffu, e, z);
        if (z < lane && ez == e) counts = false;
      }
      const unsigned valid = __ballot_sync(0xffffffffu, counts);
      int got = 1;
      if (counts) got = wait_flag_ge(flags + ((size_t)t * K + lane) * kLLParts + part, epoch, ctx, kOpLLCombine, 1, me);
      if (!__all_sync(0xffffffffu, got)) break;
      const uint8_t* rows = mine + ll.ret + (size_t)t * K * row_bytes;
      int4* out = reinterpret_cast<int4*>(reinterpret_cast<uint8_t*>(a.out) + (size_t)t * row_bytes);
      const int u_lo = pr.v0 / 8, u_hi = pr.v1 / 8, hs = (u_hi - u_lo + 1) / 2;
      const int u_begin = u_lo + half * hs, u_end = min(u_hi, u_begin + hs);
      // two 16-byte columns per lane and step; the trip count is the same for every lane, which all take part in the shuffles
      for (int ub = u_begin; ub < u_end; ub += 64) {
        const int u0 = ub + lane;
        const bool one = u0 < u_end, two = u0 + 32 < u_end;
        float a0[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, a1[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int kb = 0; kb < K; kb += 8) {    // eight slots' loads in flight at a time
          int4 v0[8], v1[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            if (kb + k < K && ((valid >> (kb + k)) & 1u)) {
              if (one) v0[k] = ld_cg_int4(rows + (size_t)(kb + k) * row_bytes + (size_t)u0 * 16);
              if (two) v1[k] = ld_cg_int4(rows + (size_t)(kb + k) * row_bytes + (size_t)(u0 + 32) * 16);
            }
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            if (kb + k < K && ((valid >> (kb + k)) & 1u)) {      // warp-uniform
              const float wk = __shfl_sync(0xffffffffu, w, kb + k);
              const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&v0[k]);
              const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&v1[k]);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                // product and sum are rounded separately (no fused multiply-add), as the CPU oracle does
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

  stamp(2);
  if (last_block_of_rank(ctl, kOpLLCombine, gridDim.x)) {
    stamp(3);
    if (!ld_volatile_int(&ctl->abort) && threadIdx.x < P)
      st_release_sys(&control_of(ctx.ws[threadIdx.x])->ll_comb_ack[me], epoch);
    if (threadIdx.x == 0) ctl->epoch[kOpLLCombine] = epoch;
  }
}

cudaError_t launch_ll_combine(const LLCombineParams& p, int nranks, int blocks, cudaStream_t stream) {
  dim3 grid(blocks, nranks), block(kLLThreads);
  void* args[] = {const_cast<LLCombineParams*>(&p)};
  const void* fn = p.profile ? (const void*)ep_combine_ll_kernel<true> : (const void*)ep_combine_ll_kernel<false>;
  return cudaLaunchCooperativeKernel(fn, grid, block, args, 0, stream);
}

}  // namespace dep
