// ep_combine_ht: all-to-all-v return of expert outputs fused with the top-k reduction.
//
// Every warp works on its own, there is no block-wide step inside the kernel.
//   Expert-side warps walk the staged-row records that dispatch used, a block of kRowBlock records
//   of one source at a time: for one (source token, this rank) they sum the token's rows on this
//   rank in slot order in fp32, round once to bf16 and store that single partial into the source
//   rank's workspace through the peer mapping (NVLink); a release flag per (source, block) follows.
//   Source-side warps take one token each: they wait for the flags of the blocks that hold the
//   token's staged row on the ranks it was sent to (the send-slot table names the row), sum the
//   partials in rank order in fp32, add the optional biases and write bf16 into the caller's tensor.  The rows that stayed on the source rank itself are summed straight from the
//   expert output (same rounding: fp32 sum -> bf16 -> fp32), so the local share never takes the detour
//   through a partial.
// The optional fp32 value channel (used for dispatch-backward) is returned per slot and is never
// multiplied into the payload.
//
// Parity: csrc/kernels/combine/combine.cpp:2224-2917 of the reference in its EP8 form (rank-level dedup,
// no gateway stage): same numeric contract (fp32 sum -> bf16 partial -> fp32 sum -> bf16), but no
// entry/exit device barriers, no prepare kernel and no final device-to-device copy, because flags are
// epochs and the output is written in place.
#include "api.h"

namespace dep {

constexpr int kSumUnroll = 4;      // 16-byte pieces per lane and pass, times up to four rows in flight

__device__ __forceinline__ void add_bf16x8(float acc[8], const int4& v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[2 * i] += __low2float(h[i]);
    acc[2 * i + 1] += __high2float(h[i]);
  }
}
__device__ __forceinline__ int4 pack_bf16x8(const float acc[8]) {
  int4 out;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
  return out;
}

// acc[i] += sum over the n rows (slot order, fp32) of pieces u0 + i * 32 + lane; lane q < n holds row q in `my_row`.
// Four rows are fetched at a time so that their loads overlap.
template <int U>
__device__ __forceinline__ void sum_rows(const uint8_t* x, int row_bytes, int units, int my_row, int n, int u0, int lane,
                                         float acc[U][8]) {
  for (int q0 = 0; q0 < n; q0 += 4) {
    int4 v[4][U];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (q0 + q < n) {
        const int4* src = reinterpret_cast<const int4*>(x + (size_t)__shfl_sync(0xffffffffu, my_row, q0 + q) * row_bytes);
#pragma unroll
        for (int i = 0; i < U; ++i) {
          const int u = u0 + i * 32 + lane;
          if (u < units) v[q][i] = __ldg(src + u);
        }
      }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (q0 + q < n) {
#pragma unroll
        for (int i = 0; i < U; ++i)
          if (u0 + i * 32 + lane < units) add_bf16x8(acc[i], v[q][i]);
      }
    }
  }
}

// One row with n == 1: the partial is the row itself.  Adding +0 in bf16 keeps every value and turns -0 into +0, which is
// what the fp32 sum that starts from zero gives.
__device__ __forceinline__ void copy_row_as_partial(const int4* src, int4* dst, int units, int lane) {
  const __nv_bfloat162 zero = __floats2bfloat162_rn(0.f, 0.f);
  for (int u0 = 0; u0 < units; u0 += 32 * 8) {
    int4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int u = u0 + i * 32 + lane;
      if (u < units) v[i] = __ldg(src + u);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int u = u0 + i * 32 + lane;
      if (u < units) {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v[i]);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __hadd2(h[e], zero);
        dst[u] = v[i];
      }
    }
  }
}

// One partial and nothing else to add: the result is the partial itself (with -0 turned into +0, as above).
__device__ __forceinline__ void copy_partial_as_result(const int4* src, int4* dst, int units, int lane) {
  const __nv_bfloat162 zero = __floats2bfloat162_rn(0.f, 0.f);
  for (int u0 = 0; u0 < units; u0 += 32 * 8) {
    int4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int u = u0 + i * 32 + lane;
      if (u < units) v[i] = __ldcg(src + u);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int u = u0 + i * 32 + lane;
      if (u < units) {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v[i]);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __hadd2(h[e], zero);
        dst[u] = v[i];
      }
    }
  }
}

template <bool kProfile>
__global__ void __launch_bounds__(kCombineThreads, 1) ep_combine_ht_kernel(const __grid_constant__ CombineParams p) {
  const CombineArgs& a = p.r[blockIdx.y];
  const WsLayout& lay = p.lay;
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, me = ctx.rank, Tmax = lay.max_tokens, H = lay.hidden, K = a.K;
  const int NB = (Tmax + kRowBlock - 1) / kRowBlock;   // completion flags per expert rank
  const int lane = threadIdx.x & 31;
  const int q = lane >> 3, c = lane & 7;      // metadata of a group is fetched by lane = (record of the group) * 8 + field
  const int row_bytes = H * 2, units = H / 8;  // 16-byte units per row
  Control* ctl = control_of(ctx.ws[me]);
  const unsigned long long epoch = ctl->epoch[kOpCombine] + 1;
  const uint8_t* x = reinterpret_cast<const uint8_t*>(a.x);
  const bool expert_side = (int)blockIdx.x < p.send_blocks;
  PhaseClock<kProfile> clk;
  clk.start();

  if (expert_side) {
    // ================================================================ expert side: reduce + return
    int ok = 1;
    if (lane < P) ok = wait_flag_ge(&ctl->comb_ack[lane], epoch - 1, ctx, kOpCombine, 0, lane);
    const bool alive = __all_sync(0xffffffffu, ok);
    clk.mark(kProfWait);
    // the sources whose rows are returned through a partial: all ranks, or all but this one
    const int S = p.local_direct ? P - 1 : P, first = p.local_direct ? 1 : 0;
    int max_nb = 0;
    for (int s = 0; s < S; ++s) {
      const int r = (me + first + s) % P;
      max_nb = max(max_nb, (a.rank_rows[r + 1] - a.rank_rows[r] + kRowBlock - 1) / kRowBlock);
    }
    // items are blocks of kRowBlock staged-row records of one source, handed out in order by a shared counter
    for (int item = next_ticket(&ctl->ticket[kOpCombine][0], lane); item < max_nb * S && alive;
         item = next_ticket(&ctl->ticket[kOpCombine][0], lane)) {
      const int r = (me + first + item % S) % P, jb = item / S, j0 = jb * kRowBlock;
      const int rows_r = min(a.rank_rows[r + 1] - a.rank_rows[r], Tmax);
      if (j0 >= rows_r) continue;
      const int cnt = min(kRowBlock, rows_r - j0);
      // the block's records in one round of loads: lane (q, c) holds fields c, 8 + c, 16 + c of record j0 + q
      int f0 = 0, f1 = 0, f2 = 0;
      if (q < cnt) {
        const int* rec = a.stage_meta + ((size_t)r * Tmax + j0 + q) * a.meta_stride;
        if (c < a.meta_stride) f0 = rec[c];
        if (8 + c < a.meta_stride) f1 = rec[8 + c];
        if (16 + c < a.meta_stride) f2 = rec[16 + c];
      }
      uint8_t* partial = ctx.ws[r] + lay.partial;
      float* wret = reinterpret_cast<float*>(ctx.ws[r] + lay.wret);
      clk.mark(kProfMeta);
      bool any = false;    // a record of this block belongs to the pass's token window
      for (int qq = 0; qq < cnt; ++qq) {
        const int t = __shfl_sync(0xffffffffu, f0, qq * 8), n = min(__shfl_sync(0xffffffffu, f0, qq * 8 + 1), kMaxTopk);
        const int rec3 = __shfl_sync(0xffffffffu, f0, qq * 8 + 3);
        const int fi = 2 + lane, from = qq * 8 + (fi & 7);
        const int e0 = __shfl_sync(0xffffffffu, f0, from), e1 = __shfl_sync(0xffffffffu, f1, from), e2 = __shfl_sync(0xffffffffu, f2, from);
        const int entry = lane < n ? ((fi >> 3) == 0 ? e0 : (fi >> 3) == 1 ? e1 : e2) : 0;
        int my_row = entry & kRowMask;
        if (lane < n && a.x_rows > 0 && !DEP_INDEX_OK(ctx, my_row, a.x_rows, kOpCombine, 0)) my_row = 0;
        const int my_row0 = __shfl_sync(0xffffffffu, my_row, 0);
        if (t < p.t_begin || t >= min(p.t_end, Tmax)) continue;
        any = true;
        int4* dst = reinterpret_cast<int4*>(partial + ((size_t)(t - p.t_begin) * P + me) * row_bytes);
        if (n == 1) {
          copy_row_as_partial(reinterpret_cast<const int4*>(x + (size_t)my_row0 * row_bytes), dst, units, lane);
        } else {
          for (int u0 = 0; u0 < units; u0 += 32 * kSumUnroll) {
            float acc[kSumUnroll][8];
#pragma unroll
            for (int i = 0; i < kSumUnroll; ++i)
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
            sum_rows<kSumUnroll>(x, row_bytes, units, my_row, n, u0, lane, acc);
#pragma unroll
            for (int i = 0; i < kSumUnroll; ++i) {
              const int u = u0 + i * 32 + lane;
              if (u < units) dst[u] = pack_bf16x8(acc[i]);
            }
          }
        }
        if (a.w) {
          if (a.expand) {
            if (lane < n) wret[(size_t)t * K + (entry >> kRowSlotShift)] = a.w[my_row];
          } else if (lane < K && ((rec3 >> lane) & 1)) {
            wret[(size_t)t * K + lane] = a.w[(size_t)my_row0 * K + lane];
          }
        }
        clk.add_rows(n);
      }
      clk.mark(kProfData);
      // publish the block: every lane's stores are ordered before the flag by the warp barrier + release
      __syncwarp();
      if (lane == 0 && any)
        st_release_sys(reinterpret_cast<unsigned long long*>(ctx.ws[r] + lay.comb_flag) + (size_t)me * NB + jb, epoch);
      clk.mark(kProfPublish);
    }
  }
  {
    // ================================================================ source side: final reduction (expert-side warps join
    // once every partial of this rank is on its way)
    const uint8_t* partial = ctx.ws[me] + lay.partial;
    const float* wret = reinterpret_cast<const float*>(ctx.ws[me] + lay.wret);
    const unsigned long long* flags = reinterpret_cast<const unsigned long long*>(ctx.ws[me] + lay.comb_flag);
    const int Lx = a.E / P;
    const int t_stop = min(a.T, p.t_end);
    for (int t = p.t_begin + next_ticket(&ctl->ticket[kOpCombine][1], lane); t < t_stop;
         t = p.t_begin + next_ticket(&ctl->ticket[kOpCombine][1], lane)) {
      const int ss = lane < P ? a.send_slot[(size_t)t * P + lane] : -1;
      const unsigned dmask = __ballot_sync(0xffffffffu, ss >= 0);
      const bool local = p.local_direct && ((dmask >> me) & 1u);
      const int j_me = __shfl_sync(0xffffffffu, ss, me);
      // the record of the rows that stayed on this rank: lane l holds field l
      int f = 0;
      if (local && j_me < Tmax && lane < a.meta_stride) f = a.stage_meta[((size_t)me * Tmax + j_me) * a.meta_stride + lane];
      clk.mark(kProfMeta);
      int ok = 1;
      if (((dmask >> lane) & 1u) && !(local && lane == me))   // the partial of rank `lane` belongs to the block of its staged row
        ok = wait_flag_ge(flags + (size_t)lane * NB + min(ss, Tmax - 1) / kRowBlock, epoch, ctx, kOpCombine, 1, lane);
      ok = __all_sync(0xffffffffu, ok);
      clk.mark(kProfWait);
      if (!ok) break;
      const int n_local = local ? min(__shfl_sync(0xffffffffu, f, 1), kMaxTopk) : 0;
      const int l_rec3 = __shfl_sync(0xffffffffu, f, 3);
      const int l_entry_raw = __shfl_sync(0xffffffffu, f, (2 + lane) & 31);
      const int l_entry = lane < n_local ? l_entry_raw : 0;
      int l_row = l_entry & kRowMask;
      if (lane < n_local && a.x_rows > 0 && !DEP_INDEX_OK(ctx, l_row, a.x_rows, kOpCombine, 0)) l_row = 0;
      const int l_row0 = __shfl_sync(0xffffffffu, l_row, 0);   // rank layout: the token's single row on this rank
      // Operands in summation order: partials of the ranks below this one, the local rows (slot order; their fp32 sum is
      // rounded to bf16 like a partial before it joins), partials of the ranks above.  Lane o holds operand o.
      const unsigned rmask = local ? (dmask & ~(1u << me)) : dmask;
      const int nlow = local ? __popc(rmask & ((1u << me) - 1u)) : __popc(rmask), nops = __popc(rmask) + n_local;
      const int l_row_o = __shfl_sync(0xffffffffu, l_row, (lane - nlow) & 31);
      unsigned long long my_op = 0;
      if (lane < nops) {
        if (lane >= nlow && lane < nlow + n_local) {
          my_op = reinterpret_cast<unsigned long long>(x + (size_t)l_row_o * row_bytes);
        } else {
          const int d = __fns(rmask, 0, (lane < nlow ? lane : lane - n_local) + 1);
          my_op = reinterpret_cast<unsigned long long>(partial + ((size_t)(t - p.t_begin) * P + d) * row_bytes);
        }
      }
      const int4* b0 = a.bias0 ? reinterpret_cast<const int4*>(a.bias0 + (size_t)t * H) : nullptr;
      const int4* b1 = a.bias1 ? reinterpret_cast<const int4*>(a.bias1 + (size_t)t * H) : nullptr;
      int4* out = reinterpret_cast<int4*>(reinterpret_cast<uint8_t*>(a.out) + (size_t)t * row_bytes);
      if (nops == 1 && n_local == 0 && !b0 && !b1) {
        copy_partial_as_result(reinterpret_cast<const int4*>(__shfl_sync(0xffffffffu, my_op, 0)), out, units, lane);
      } else {
        for (int u0 = 0; u0 < units; u0 += 32 * kSumUnroll) {
          float acc[kSumUnroll][8], lsum[kSumUnroll][8];
#pragma unroll
          for (int i = 0; i < kSumUnroll; ++i)
#pragma unroll
            for (int e = 0; e < 8; ++e) { acc[i][e] = 0.f; lsum[i][e] = 0.f; }
          for (int o0 = 0; o0 < nops; o0 += 4) {
            int4 v[4][kSumUnroll];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              if (o0 + b < nops) {
                const int4* src = reinterpret_cast<const int4*>(__shfl_sync(0xffffffffu, my_op, o0 + b));
                const bool is_row = o0 + b >= nlow && o0 + b < nlow + n_local;
#pragma unroll
                for (int i = 0; i < kSumUnroll; ++i) {
                  const int u = u0 + i * 32 + lane;
                  if (u < units) v[b][i] = is_row ? __ldg(src + u) : __ldcg(src + u);
                }
              }
            }
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              if (o0 + b < nops) {
                const int o = o0 + b;
                const bool is_row = o >= nlow && o < nlow + n_local;
#pragma unroll
                for (int i = 0; i < kSumUnroll; ++i) {
                  if (u0 + i * 32 + lane >= units) continue;
                  if (is_row) add_bf16x8(lsum[i], v[b][i]);
                  else add_bf16x8(acc[i], v[b][i]);
                  // the last local row: the local partial is complete, it joins the sum rounded like a remote one
                  if (is_row && o == nlow + n_local - 1) add_bf16x8(acc[i], pack_bf16x8(lsum[i]));
                }
              }
            }
          }
#pragma unroll
          for (int i = 0; i < kSumUnroll; ++i) {
            const int u = u0 + i * 32 + lane;
            if (u >= units) continue;
            if (b0) add_bf16x8(acc[i], __ldg(b0 + u));
            if (b1) add_bf16x8(acc[i], __ldg(b1 + u));
            out[u] = pack_bf16x8(acc[i]);
          }
        }
      }
      if (a.out_w) {
        // lane k: the value of slot k (zero for empty or repeated experts); local slots are read from the caller's tensor
        long long e = lane < K ? a.topk_idx[(size_t)t * K + lane] : -1;
        bool valid = lane < K && e >= 0 && e < a.E;
        for (int z = 0; z < K; ++z) {
          const long long ez = __shfl_sync(0xffffffffu, e, z);
          if (z < lane && ez == e) valid = false;
        }
        float value = 0.f;
        const bool mine = valid && local && (int)(e / Lx) == me;
        if (a.expand) {
          for (int i = 0; i < n_local; ++i) {
            const int ei = __shfl_sync(0xffffffffu, l_entry, i);
            if (mine && (ei >> kRowSlotShift) == lane) value = a.w ? a.w[ei & kRowMask] : 0.f;
          }
        } else if (mine && ((l_rec3 >> lane) & 1)) {
          value = a.w ? a.w[(size_t)l_row0 * K + lane] : 0.f;
        }
        if (valid && !mine) value = __ldcg(wret + (size_t)t * K + lane);
        if (lane < K) a.out_w[(size_t)t * K + lane] = valid ? value : 0.f;
      }
      clk.add_rows(nops);
      clk.mark(kProfData);
    }
  }

  clk.finish(a.prof ? a.prof + (size_t)blockIdx.x * kCombineProfWords : nullptr, expert_side ? 0 : 1);

  if (last_block_of_rank(ctl, kOpCombine, gridDim.x)) {
    if (!ld_volatile_int(&ctl->abort) && threadIdx.x < P)
      st_release_sys(&control_of(ctx.ws[threadIdx.x])->comb_ack[me], epoch);
    if (threadIdx.x == 0) { ctl->ticket[kOpCombine][0] = 0; ctl->ticket[kOpCombine][1] = 0; ctl->epoch[kOpCombine] = epoch; }
  }
}

cudaError_t launch_combine(const CombineParams& p, int nranks, cudaStream_t stream) {
  dim3 grid(p.send_blocks + p.recv_blocks, nranks), block(kCombineThreads);
  void* args[] = {const_cast<CombineParams*>(&p)};
  const void* fn = p.profile ? (const void*)ep_combine_ht_kernel<true> : (const void*)ep_combine_ht_kernel<false>;
  return cudaLaunchCooperativeKernel(fn, grid, block, args, 0, stream);
}

}  // namespace dep
