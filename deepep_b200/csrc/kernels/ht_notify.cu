// ep_notify: routing layout of one dispatch, computed identically on every rank.
//
// Design (differs from the reference's 47-phase notify, csrc/kernels/notify/notify.cpp:1426-1970,
// which exchanges count tables, forward packets and backward packets in three rounds):
// on one NVSwitch domain the routing table itself is tiny, so every rank pushes its
// [T, K] expert ids and weights to every peer once (P2P stores + one release flag per
// peer), and each rank then derives *all* metadata locally from the gathered table:
//   - per-(source, expert) counts  -> expert row offsets, ordered (expert, source, token, slot)
//   - rank-level dedup             -> one staged row per (source token, destination rank)
//   - receive-side expansion lists -> stage_meta[(source, staged row)] = rows to materialise
// Offsets come from prefix sums over 64-token tiles (bit masks + popcounts), never from
// atomics, so the layout is deterministic and equal to the CPU oracle bit for bit.
#include <cooperative_groups.h>

#include "api.h"

namespace cg = cooperative_groups;

namespace dep {

constexpr int kNotifyThreads = 256;

struct TileMasks {
  unsigned expert[kMaxExperts][2];   // bit t: token t of the tile routes to this expert
  unsigned rank[kMaxRanks][2];       // bit t: token t of the tile routes to this rank
};

__device__ __forceinline__ int below(const unsigned m[2], int tl) {
  unsigned lo = tl < 32 ? ((1u << tl) - 1u) : 0xffffffffu;
  unsigned hi = tl < 32 ? 0u : ((1u << (tl - 32)) - 1u);
  return __popc(m[0] & lo) + __popc(m[1] & hi);
}

// A slot counts when its expert id is in range and no earlier slot of the token names the same expert.
__device__ __forceinline__ bool slot_counts(const int* row, int k, int E) {
  int e = row[k];
  if (e < 0 || e >= E) return false;
  for (int j = 0; j < k; ++j)
    if (row[j] == e) return false;
  return true;
}

// One thread per token of the tile: the K ids of a row are fetched once (independent loads), duplicates
// are resolved in registers, then the masks are updated with shared-memory atomics.
__device__ void build_masks(TileMasks& m, const int* gidx_src, int tile, int T_r, int K, int E, int Lx) {
  for (int i = threadIdx.x; i < E * 2; i += blockDim.x) (&m.expert[0][0])[i] = 0u;
  if (threadIdx.x < kMaxRanks * 2) (&m.rank[0][0])[threadIdx.x] = 0u;
  __syncthreads();
  const int tl = threadIdx.x, t = tile * kChunkTokens + tl;
  if (tl < kChunkTokens && t < T_r) {
    int row[kMaxTopk];
    const int* src = gidx_src + (size_t)t * K;
#pragma unroll
    for (int k = 0; k < kMaxTopk; ++k) row[k] = k < K ? __ldcg(src + k) : -1;
#pragma unroll
    for (int k = 0; k < kMaxTopk; ++k) {
      if (k < K && slot_counts(row, k, E)) {
        const int e = row[k];
        atomicOr(&m.expert[e][tl >> 5], 1u << (tl & 31));
        atomicOr(&m.rank[e / Lx][tl >> 5], 1u << (tl & 31));
      }
    }
  }
  __syncthreads();
}

template <bool kProfile>
__global__ void __launch_bounds__(kNotifyThreads) ep_notify_kernel(const __grid_constant__ NotifyParams p) {
  cg::grid_group grid = cg::this_grid();
  const NotifyArgs& a = p.r[blockIdx.y];
  const WsLayout& lay = p.lay;
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, me = ctx.rank, K = a.K, E = a.E, Lx = E / P, Tmax = lay.max_tokens;
  const int NT = (Tmax + kChunkTokens - 1) / kChunkTokens;
  uint8_t* ws = ctx.ws[me];
  Control* ctl = control_of(ws);
  const unsigned long long epoch = ctl->epoch[kOpNotify] + 1;
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x, gstride = gridDim.x * blockDim.x;

  __shared__ TileMasks s_m;
  __shared__ int s_T[kMaxRanks];
  __shared__ int s_rank_base[kMaxRanks + 1];
  __shared__ int s_off[kMaxExperts];
  __shared__ int s_base[kMaxExperts];                   // scratch: totals, then per-task row bases
  __shared__ int s_rows;

  // profile instantiation only: phase stamps of block 0 (nanoseconds since kernel start) in Control::dbg[16..23]
  unsigned long long t_start = 0;
  if constexpr (kProfile) t_start = global_timer_ns();
  auto stamp = [&](int i) {
    if constexpr (kProfile)
      if (blockIdx.x == 0 && threadIdx.x == 0) ctl->dbg[16 + i] = global_timer_ns() - t_start;
  };

  // ---- A: publish my routing table into every peer (after they consumed the previous one)
  int ok = 1;
  if (threadIdx.x < P) ok = wait_flag_ge(&ctl->notify_ack[threadIdx.x], epoch - 1, ctx, kOpNotify, 0, threadIdx.x);
  int alive = __syncthreads_and(ok);
  if (alive) {
    const int n = a.T * K;
    for (int i = gtid; i < P * n; i += gstride) {
      int d = i / n, j = i - d * n;
      long long v = a.topk_idx[j];
      int e = (v < 0 || v >= E) ? -1 : (int)v;
      reinterpret_cast<int*>(ctx.ws[d] + lay.gather_idx)[(size_t)me * Tmax * K + j] = e;
      if (a.topk_w) reinterpret_cast<float*>(ctx.ws[d] + lay.gather_w)[(size_t)me * Tmax * K + j] = a.topk_w[j];
    }
    if (blockIdx.x == 0 && threadIdx.x < P) {
      int* hdr = reinterpret_cast<int*>(ctx.ws[threadIdx.x] + lay.gather_hdr) + me * 4;
      hdr[0] = a.T;
      hdr[1] = a.topk_w != nullptr;
    }
    __threadfence_system();
  }
  grid.sync();
  if (alive && blockIdx.x == 0 && threadIdx.x < P)
    st_release_sys(&control_of(ctx.ws[threadIdx.x])->notify_ready[me], epoch);

  stamp(0);
  // ---- B: wait for every rank's table
  ok = 1;
  if (alive && threadIdx.x < P) ok = wait_flag_ge(&ctl->notify_ready[threadIdx.x], epoch, ctx, kOpNotify, 1, threadIdx.x);
  alive = __syncthreads_and(ok) && alive;
  const int* ghdr = reinterpret_cast<const int*>(ws + lay.gather_hdr);
  const int* gidx = reinterpret_cast<const int*>(ws + lay.gather_idx);
  const float* gw = reinterpret_cast<const float*>(ws + lay.gather_w);
  if (threadIdx.x < kMaxRanks) s_T[threadIdx.x] = (alive && threadIdx.x < P) ? __ldcg(ghdr + threadIdx.x * 4) : 0;
  __syncthreads();
  const bool has_w = alive && __ldcg(ghdr + 1) != 0 && a.recv_w != nullptr;

  stamp(1);
  // ---- C: per-(source, tile) histograms
  for (int task = blockIdx.x; task < P * NT; task += gridDim.x) {
    int r = task / NT, tile = task - r * NT;
    if (tile * kChunkTokens >= s_T[r]) continue;
    build_masks(s_m, gidx + (size_t)r * Tmax * K, tile, s_T[r], K, E, Lx);
    for (int e = threadIdx.x; e < E; e += blockDim.x)
      a.hist[(size_t)task * E + e] = __popc(s_m.expert[e][0]) + __popc(s_m.expert[e][1]);
    if (threadIdx.x == 0) a.hits[task] = __popc(s_m.rank[me][0]) + __popc(s_m.rank[me][1]);
    if (a.rank_matrix && threadIdx.x < P)
      atomicAdd(&a.rank_matrix[r * P + threadIdx.x], __popc(s_m.rank[threadIdx.x][0]) + __popc(s_m.rank[threadIdx.x][1]));
    if (r == me && threadIdx.x < P)
      a.own_hits[tile * P + threadIdx.x] = __popc(s_m.rank[threadIdx.x][0]) + __popc(s_m.rank[threadIdx.x][1]);
    __syncthreads();
  }
  grid.sync();

  stamp(2);
  // ---- D1: exclusive scans over tiles
  {   // one warp per (source, expert): the lanes take 32 tiles at a time, exclusive prefix by a warp scan
    const int lane_ = threadIdx.x & 31;
    for (int i = gtid >> 5; i < P * E; i += gstride >> 5) {
      const int r = i / E, e = i - r * E, nt = (s_T[r] + kChunkTokens - 1) / kChunkTokens;
      int run = 0;
      for (int tile0 = 0; tile0 < nt; tile0 += 32) {
        const int tile = tile0 + lane_;
        int* cell = a.hist + ((size_t)r * NT + tile) * E + e;
        const int v = tile < nt ? *cell : 0;
        int incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int o = __shfl_up_sync(0xffffffffu, incl, d);
          if (lane_ >= d) incl += o;
        }
        if (tile < nt) *cell = run + incl - v;
        run += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane_ == 0) a.cnt[i] = run;
    }
  }
  {   // staged-row starts of every (source, chunk) and my own per-destination starts: one warp each, same warp scan
    const int w = gtid >> 5, lane_ = threadIdx.x & 31;
    if (w < 2 * P) {
      const bool own = w >= P;
      const int r = own ? me : w, d = w - P, nt = (s_T[r] + kChunkTokens - 1) / kChunkTokens;
      int run = 0;
      for (int tile0 = 0; tile0 < nt; tile0 += 32) {
        const int tile = tile0 + lane_;
        const int v = tile < nt ? (own ? a.own_hits[tile * P + d] : a.hits[r * NT + tile]) : 0;
        int incl = v;
#pragma unroll
        for (int q = 1; q < 32; q <<= 1) {
          const int o = __shfl_up_sync(0xffffffffu, incl, q);
          if (lane_ >= q) incl += o;
        }
        if (tile < nt) {
          if (own) a.own_hits[tile * P + d] = run + incl - v;
          else a.chunk_start[r * (NT + 1) + tile] = run + incl - v;
        }
        run += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (!own)
        for (int tile = nt + lane_; tile <= NT; tile += 32) a.chunk_start[r * (NT + 1) + tile] = run;
    }
  }
  grid.sync();

  stamp(3);
  // ---- D2: expert row offsets of every rank (each block keeps its own copy in shared memory)
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int tot = 0;
    for (int r = 0; r < P; ++r) tot += a.cnt[r * E + e];
    s_base[e] = tot;                                      // total rows of expert e (all sources)
  }
  __syncthreads();
  if ((threadIdx.x >> 5) < P) {    // warp d: aligned exclusive prefix over the local experts of rank d
    const int d = threadIdx.x >> 5, lane_ = threadIdx.x & 31;
    int run = 0;
    for (int l0 = 0; l0 < Lx; l0 += 32) {
      const int l = l0 + lane_, e = d * Lx + l;
      const int tot = l < Lx ? s_base[e] : 0;
      const int al = a.expand ? (tot + a.alignment - 1) / a.alignment * a.alignment : tot;
      int incl = al;
#pragma unroll
      for (int q = 1; q < 32; q <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, incl, q);
        if (lane_ >= q) incl += o;
      }
      if (l < Lx) {
        s_off[e] = run + incl - al;
        if (d == me && blockIdx.x == 0) { a.expert_counts[l] = tot; a.expert_offsets[l] = run + incl - al; }
      }
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (d == me && lane_ == 0) { s_rows = run; if (blockIdx.x == 0) a.expert_offsets[Lx] = run; }
  }
  if (threadIdx.x == 0) {
    int run = 0;
    for (int r = 0; r < P; ++r) { s_rank_base[r] = run; run += a.chunk_start[r * (NT + 1) + NT]; }
    s_rank_base[P] = run;
  }
  __syncthreads();
  if (!a.expand && threadIdx.x == 0) s_rows = s_rank_base[P];
  __syncthreads();
  if (blockIdx.x == 0) {
    if (threadIdx.x <= P) a.rank_rows[threadIdx.x] = s_rank_base[threadIdx.x];
    if (threadIdx.x < P) a.rank_tokens[threadIdx.x] = s_T[threadIdx.x];
    if (a.expand && a.alignment > 1) {  // padding rows carry no source
      for (int l = 0; l < Lx; ++l) {
        int e = me * Lx + l, tot = a.expert_counts[l];
        int end = (l + 1 < Lx) ? s_off[e + 1] : s_rows;
        for (int row = s_off[e] + tot + threadIdx.x; row < end && row < a.rcap; row += blockDim.x) {
          a.recv_row_src[row] = -1;
          if (a.recv_w) a.recv_w[row] = 0.f;
        }
      }
    }
  }

  stamp(4);
  // ---- E: per-token records
  for (int task = blockIdx.x; task < P * NT; task += gridDim.x) {
    int r = task / NT, tile = task - r * NT, T_r = s_T[r];
    if (tile * kChunkTokens >= T_r) continue;
    const int* gidx_r = gidx + (size_t)r * Tmax * K;
    build_masks(s_m, gidx_r, tile, T_r, K, E, Lx);
    {   // rows of expert e that precede this (source, tile): earlier sources + earlier tiles of this source
      const int* hist_task = a.hist + (size_t)task * E;
      for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int b = hist_task[e];
        for (int q = 0; q < r; ++q) b += a.cnt[q * E + e];
        s_base[e] = b;
      }
      __syncthreads();
    }
    int tl = threadIdx.x, t = tile * kChunkTokens + tl;
    if (tl < kChunkTokens && t < T_r) {
      int row[kMaxTopk];
#pragma unroll
      for (int k = 0; k < kMaxTopk; ++k) row[k] = k < K ? __ldcg(gidx_r + (size_t)t * K + k) : -1;
      const bool hit_me = (s_m.rank[me][tl >> 5] >> (tl & 31)) & 1u;
      if (hit_me) {
        int j = a.chunk_start[r * (NT + 1) + tile] + below(s_m.rank[me], tl);
        int* rec = a.stage_meta + ((size_t)r * Tmax + j) * a.meta_stride;
        rec[0] = t;
        int n = 0;
        if (a.expand) {
          for (int k = 0; k < K; ++k) {
            if (!slot_counts(row, k, E) || row[k] / Lx != me) continue;
            int e = row[k];
            int out_row = s_off[e] + s_base[e] + below(s_m.expert[e], tl);
            rec[2 + n++] = out_row | (k << kRowSlotShift);
            if (out_row < a.rcap) {
              a.recv_row_src[out_row] = (r * Tmax + t) * K + k;
              if (a.recv_w) a.recv_w[out_row] = has_w ? __ldcg(gw + ((size_t)r * Tmax + t) * K + k) : 0.f;
            }
          }
        } else {
          int out_row = s_rank_base[r] + j, slots_here = 0;
          for (int k = 0; k < K; ++k)
            if (slot_counts(row, k, E) && row[k] / Lx == me) slots_here |= 1 << k;
          rec[2] = out_row;
          rec[3] = slots_here;   // which slots of the token live on this rank
          n = 1;
          if (out_row < a.rcap) {
            a.recv_row_src[out_row] = (r * Tmax + t) * K;
            for (int k = 0; k < K; ++k) {
              bool mine = slot_counts(row, k, E) && row[k] / Lx == me;
              if (a.recv_idx) a.recv_idx[(size_t)out_row * K + k] = mine ? row[k] - me * Lx : -1;
              if (a.recv_w) a.recv_w[(size_t)out_row * K + k] = (mine && has_w) ? __ldcg(gw + ((size_t)r * Tmax + t) * K + k) : 0.f;
            }
          }
        }
        rec[1] = n;
      }
      if (r == me) {
        for (int d = 0; d < P; ++d) {
          bool hit = (s_m.rank[d][tl >> 5] >> (tl & 31)) & 1u;
          a.send_slot[(size_t)t * P + d] = hit ? a.own_hits[tile * P + d] + below(s_m.rank[d], tl) : -1;
        }
        for (int k = 0; k < K; ++k) {
          int v = -1;
          if (a.expand && slot_counts(row, k, E)) {
            int e = row[k];     // r == me here, so s_base already holds this rank's base
            v = s_off[e] + s_base[e] + below(s_m.expert[e], tl);
          }
          a.slot_row[(size_t)t * K + k] = v;
        }
      }
    }
    __syncthreads();
  }
  __threadfence();
  grid.sync();

  stamp(5);
  // ---- F: release the gathered table, publish counts to the host, advance the epoch
  if (blockIdx.x == 0) {
    if (threadIdx.x < P) st_release_sys(&control_of(ctx.ws[threadIdx.x])->notify_ack[me], epoch);
    if (a.mailbox) {
      for (int l = threadIdx.x; l < Lx; l += blockDim.x) a.mailbox[4 + l] = a.expert_counts[l];
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x == 0) {
        int maxT = 0;
        for (int r = 0; r < P; ++r) maxT = max(maxT, s_T[r]);
        a.mailbox[0] = alive ? s_rows : -1;
        a.mailbox[1] = s_rank_base[P];
        a.mailbox[2] = maxT;
        __threadfence_system();
        a.mailbox[3] = (int)(epoch & 0x7fffffff);
        __threadfence_system();
      }
    }
    if (threadIdx.x == 0) ctl->epoch[kOpNotify] = epoch;
  }
}

cudaError_t launch_notify(const NotifyParams& p, int nranks, int blocks, cudaStream_t stream) {
  dim3 grid(blocks, nranks), block(kNotifyThreads);
  void* args[] = {const_cast<NotifyParams*>(&p)};
  const void* fn = p.profile ? (const void*)ep_notify_kernel<true> : (const void*)ep_notify_kernel<false>;
  return cudaLaunchCooperativeKernel(fn, grid, block, args, 0, stream);
}

}  // namespace dep
