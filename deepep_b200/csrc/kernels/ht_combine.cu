// ep_combine_ht: all-to-all-v return of expert outputs fused with the top-k reduction.
//
// Every warp works on its own, there is no block-wide step inside the kernel.
//   Expert-side warps walk the staged-row records that dispatch used, (source, group of kGroupTokens
//   tokens) by (source, group): for one (source token, this rank) they sum the token's rows on this
//   rank in slot order in fp32, round once to bf16 and store that single partial into the source
//   rank's workspace through the peer mapping (NVLink); a release flag per (source, group) follows.
//   Source-side warps take one token each: they wait for the group flags of the ranks the token was
//   sent to, sum the partials in rank order in fp32, add the optional biases and write bf16 into the
//   caller's tensor.  The rows that stayed on the source rank itself are summed straight from the
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

constexpr int kHtThreads = 512;
constexpr int kSumUnroll = 4;      // expert side: 16-byte pieces per lane and pass
constexpr int kSrcUnroll = 2;      // source side: pieces per lane and pass (times up to 8 partials in flight)

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

template <bool kProfile>
__global__ void __launch_bounds__(kHtThreads, 1) ep_combine_ht_kernel(const __grid_constant__ CombineParams p) {
  const CombineArgs& a = p.r[blockIdx.y];
  const WsLayout& lay = p.lay;
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, me = ctx.rank, Tmax = lay.max_tokens, H = lay.hidden, K = a.K;
  const int NG = (Tmax + kGroupTokens - 1) / kGroupTokens;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int row_bytes = H * 2, units = H / 8;  // 16-byte units per row
  Control* ctl = control_of(ctx.ws[me]);
  const unsigned long long epoch = ctl->epoch[kOpCombine] + 1;
  const uint8_t* x = reinterpret_cast<const uint8_t*>(a.x);
  const bool expert_side = (int)blockIdx.x < p.send_blocks;
  unsigned long long t_begin = 0, t_wait = 0, n_rows = 0;
  if (kProfile) t_begin = global_timer_ns();

  if (expert_side) {
    // ================================================================ expert side: reduce + return
    int ok = 1;
    if (lane < P) ok = wait_flag_ge(&ctl->comb_ack[lane], epoch - 1, ctx, kOpCombine, 0, lane);
    const bool alive = __all_sync(0xffffffffu, ok);
    int max_ng = 0;
    for (int r = 0; r < P; ++r) max_ng = max(max_ng, (a.rank_tokens[r] + kGroupTokens - 1) / kGroupTokens);
    const int nsend = p.send_blocks * nwarps, w = blockIdx.x * nwarps + warp;
    for (int item = w; item < max_ng * P && alive; item += nsend) {
      const int gi = item / P, r = (me + item % P) % P;
      if ((p.local_direct && r == me) || gi * kGroupTokens >= a.rank_tokens[r]) continue;
      const int j0 = a.group_start[r * (NG + 1) + gi], j1 = a.group_start[r * (NG + 1) + gi + 1];
      if (j0 >= j1) continue;
      if (j0 < 0 || j1 - j0 > kGroupTokens || j1 > Tmax) {   // a group stages at most one row per token: the plan is damaged
        if (lane == 0) report_failure(ctx, kStatusBadArgument, kOpCombine, 3, r, kGroupTokens, (unsigned long long)(j1 - j0));
        break;
      }
      uint8_t* partial = ctx.ws[r] + lay.partial;
      float* wret = reinterpret_cast<float*>(ctx.ws[r] + lay.wret);
      for (int j = j0; j < j1; ++j) {
        if (!DEP_INDEX_OK(ctx, j, Tmax, kOpCombine, 2)) continue;
        const int* rec = a.stage_meta + ((size_t)r * Tmax + j) * a.meta_stride;
        const int t = rec[0], n = min(rec[1], kMaxTopk);
        int entry = lane < n ? rec[2 + lane] : 0;
        int my_row = entry & kRowMask;
        if (lane < n && a.x_rows > 0 && !DEP_INDEX_OK(ctx, my_row, a.x_rows, kOpCombine, 0)) my_row = 0;
        int4* dst = reinterpret_cast<int4*>(partial + ((size_t)t * P + me) * row_bytes);
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
        if (a.w) {
          if (a.expand) {
            if (lane < n) wret[(size_t)t * K + (entry >> kRowSlotShift)] = a.w[my_row];
          } else if (lane < K && ((rec[3] >> lane) & 1)) {
            wret[(size_t)t * K + lane] = a.w[(size_t)(rec[2] & kRowMask) * K + lane];
          }
        }
        if (kProfile) n_rows += n;
      }
      // publish the group: every lane's stores are ordered before the flag by the warp barrier + release
      __syncwarp();
      if (lane == 0)
        st_release_sys(reinterpret_cast<unsigned long long*>(ctx.ws[r] + lay.comb_flag) + (size_t)me * NG + gi, epoch);
    }
  } else {
    // ================================================================ source side: final reduction
    const int nsrc = p.recv_blocks * nwarps, w = (blockIdx.x - p.send_blocks) * nwarps + warp;
    const uint8_t* partial = ctx.ws[me] + lay.partial;
    const float* wret = reinterpret_cast<const float*>(ctx.ws[me] + lay.wret);
    const unsigned long long* flags = reinterpret_cast<const unsigned long long*>(ctx.ws[me] + lay.comb_flag);
    const int Lx = a.E / P;
    for (int t = w; t < a.T; t += nsrc) {
      const int slot = lane < P ? a.send_slot[(size_t)t * P + lane] : -1;
      const unsigned dmask = __ballot_sync(0xffffffffu, slot >= 0);
      const bool local = p.local_direct && ((dmask >> me) & 1u);
      int ok = 1;
      if (((dmask >> lane) & 1u) && !(local && lane == me)) {
        unsigned long long t0 = 0;
        if (kProfile) t0 = global_timer_ns();
        ok = wait_flag_ge(flags + (size_t)lane * NG + t / kGroupTokens, epoch, ctx, kOpCombine, 1, lane);
        if (kProfile && lane == 0) t_wait += global_timer_ns() - t0;
      }
      if (!__all_sync(0xffffffffu, ok)) break;
      // the rows of this token that stayed on this rank
      int n_local = 0, l_entry = 0, l_row = 0, l_rec3 = 0;
      if (local) {
        const int* rec = a.stage_meta + ((size_t)me * Tmax + __shfl_sync(0xffffffffu, slot, me)) * a.meta_stride;
        n_local = min(rec[1], kMaxTopk);
        l_entry = lane < n_local ? rec[2 + lane] : 0;
        l_row = l_entry & kRowMask;
        if (lane < n_local && a.x_rows > 0 && !DEP_INDEX_OK(ctx, l_row, a.x_rows, kOpCombine, 0)) l_row = 0;
        if (!a.expand) l_rec3 = rec[3];
      }
      const int l_row0 = __shfl_sync(0xffffffffu, l_row, 0);   // rank layout: the token's single row on this rank
      const int4* b0 = a.bias0 ? reinterpret_cast<const int4*>(a.bias0 + (size_t)t * H) : nullptr;
      const int4* b1 = a.bias1 ? reinterpret_cast<const int4*>(a.bias1 + (size_t)t * H) : nullptr;
      int4* out = reinterpret_cast<int4*>(reinterpret_cast<uint8_t*>(a.out) + (size_t)t * row_bytes);
      for (int u0 = 0; u0 < units; u0 += 32 * kSrcUnroll) {
        // all remote partials of the pass are fetched before the first addition
        int4 v[kMaxRanks][kSrcUnroll];
#pragma unroll
        for (int d = 0; d < kMaxRanks; ++d) {
          if (((dmask >> d) & 1u) && !(local && d == me)) {
            const int4* src = reinterpret_cast<const int4*>(partial + ((size_t)t * P + d) * row_bytes);
#pragma unroll
            for (int i = 0; i < kSrcUnroll; ++i) {
              const int u = u0 + i * 32 + lane;
              if (u < units) v[d][i] = __ldcg(src + u);
            }
          }
        }
        float lsum[kSrcUnroll][8];
#pragma unroll
        for (int i = 0; i < kSrcUnroll; ++i)
#pragma unroll
          for (int e = 0; e < 8; ++e) lsum[i][e] = 0.f;
        if (local) sum_rows<kSrcUnroll>(x, row_bytes, units, l_row, n_local, u0, lane, lsum);
        float acc[kSrcUnroll][8];
#pragma unroll
        for (int i = 0; i < kSrcUnroll; ++i)
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
#pragma unroll
        for (int d = 0; d < kMaxRanks; ++d) {
          if ((dmask >> d) & 1u) {
#pragma unroll
            for (int i = 0; i < kSrcUnroll; ++i) {
              if (u0 + i * 32 + lane >= units) continue;
              if (local && d == me) add_bf16x8(acc[i], pack_bf16x8(lsum[i]));   // the local partial, rounded like a remote one
              else add_bf16x8(acc[i], v[d][i]);
            }
          }
        }
#pragma unroll
        for (int i = 0; i < kSrcUnroll; ++i) {
          const int u = u0 + i * 32 + lane;
          if (u >= units) continue;
          if (b0) add_bf16x8(acc[i], __ldg(b0 + u));
          if (b1) add_bf16x8(acc[i], __ldg(b1 + u));
          out[u] = pack_bf16x8(acc[i]);
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
      if (kProfile) n_rows += __popc(dmask);
    }
  }

  if (kProfile && a.prof != nullptr && threadIdx.x == 0) {
    unsigned long long* rec = a.prof + (size_t)blockIdx.x * kCombineProfWords;
    rec[0] = expert_side ? 0 : 1; rec[1] = t_begin; rec[2] = global_timer_ns(); rec[3] = t_wait; rec[4] = n_rows;
  }

  if (last_block_of_rank(ctl, kOpCombine, gridDim.x)) {
    if (!ld_volatile_int(&ctl->abort) && threadIdx.x < P)
      st_release_sys(&control_of(ctx.ws[threadIdx.x])->comb_ack[me], epoch);
    if (threadIdx.x == 0) ctl->epoch[kOpCombine] = epoch;
  }
}

cudaError_t launch_combine(const CombineParams& p, int nranks, cudaStream_t stream) {
  dim3 grid(p.send_blocks + p.recv_blocks, nranks), block(kHtThreads);
  void* args[] = {const_cast<CombineParams*>(&p)};
  const void* fn = p.profile ? (const void*)ep_combine_ht_kernel<true> : (const void*)ep_combine_ht_kernel<false>;
  return cudaLaunchCooperativeKernel(fn, grid, block, args, 0, stream);
}

}  // namespace dep
