// ep_dispatch_ht: all-to-all-v token push with rank-level dedup and receive-side expansion.
//
// Every warp works on its own, there is no block-wide step inside the kernel.
//   Sender warps take groups of kGroupTokens source tokens.  A token row is read once into registers
//   (a quarter row per pass) and stored ONCE per destination GPU into that GPU's staging area through
//   the peer mapping (NVLink), optionally quantised to e4m3 with one fp32 scale per 128 values on the
//   way.  Rows whose destination is the sending rank itself are written straight into the output
//   tensor, one copy per local expert.  After a group the warp publishes one release flag per
//   destination: flags cover two tokens, so the receivers follow the senders closely, no sender ever
//   drains a pipeline at a chunk boundary, and there are several groups per sender warp, which keeps
//   the last wave of groups short.
//   Receiver warps take blocks of kRowBlock staged rows of one source, in the order the senders
//   produce them.  Each record names its source token; the warp waits for that token's flag and
//   materialises every output row of the staged row (one per local expert of the token), so a token
//   crosses NVLink once no matter how many experts of the destination it uses.
//   Groups and blocks are handed out by two shared counters; sender warps turn into receivers once
//   the last group is on its way.
//
// Between two GPUs 32 SMs of 16-byte register stores reach the same rate as bulk shared->global copies
// (about 0.69 TB/s per direction with both directions busy); the register form needs no staging in
// shared memory, no proxy fences and no barriers, and lets a block keep 16 rows in flight.
//
// The reference's dispatch (csrc/kernels/dispatch/dispatch.cpp:463-590) has the same three jobs (payload
// scatter, receiver expansion from a forward list, per-source completion flags) spread over 64
// role-specialised vector cores and WQE queues.
#include "api.h"

namespace dep {

constexpr int kCopyUnroll = 7;    // 16-byte pieces per lane and pass: 3.5 KB in flight per warp

__device__ __forceinline__ unsigned long long shfl_u64(unsigned long long v, int src) {
  return __shfl_sync(0xffffffffu, v, src);
}

// Copies `units` 16-byte pieces from `src` to every destination in `mask`: lane l of the mask holds its
// destination in `dst`.  All loads of a pass are issued before the first store.
template <bool kPeerWritten>
__device__ __forceinline__ void warp_fanout(const int4* src, int units, unsigned long long dst, unsigned mask, int lane) {
  for (int u0 = 0; u0 < units; u0 += 32 * kCopyUnroll) {
    int4 v[kCopyUnroll];
#pragma unroll
    for (int i = 0; i < kCopyUnroll; ++i) {
      const int u = u0 + i * 32 + lane;
      if (u < units) v[i] = kPeerWritten ? __ldcg(src + u) : __ldg(src + u);
    }
    for (unsigned m = mask; m; m &= m - 1) {
      int4* d = reinterpret_cast<int4*>(shfl_u64(dst, __ffs(m) - 1));
#pragma unroll
      for (int i = 0; i < kCopyUnroll; ++i) {
        const int u = u0 + i * 32 + lane;
        if (u < units) d[u] = v[i];
      }
    }
  }
}

// The same for a short run of floats (the scales of an fp8 row).
template <bool kPeerWritten>
__device__ __forceinline__ void warp_fanout_f32(const float* src, int n, unsigned long long dst, unsigned mask, int lane) {
  for (int b0 = 0; b0 < n; b0 += 32) {   // the trip count is the same for every lane: all of them take part in the shuffles
    const int b = b0 + lane;
    float v = 0.f;
    if (b < n) v = kPeerWritten ? __ldcg(src + b) : __ldg(src + b);
    for (unsigned m = mask; m; m &= m - 1) {
      float* d = reinterpret_cast<float*>(shfl_u64(dst, __ffs(m) - 1));
      if (b < n) d[b] = v;
    }
  }
}

// 16 bf16 values (two 16-byte pieces) -> their absolute maximum.
__device__ __forceinline__ float amax16(const int4& a, const int4& b, float v[16]) {
  const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __low2float(ha[i]); v[2 * i + 1] = __high2float(ha[i]);
    v[8 + 2 * i] = __low2float(hb[i]); v[8 + 2 * i + 1] = __high2float(hb[i]);
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(v[i]));
  return m;
}

// Fused quantiser: a bf16 row -> e4m3 bytes and one fp32 scale per 128 values, written to every destination.
// amax over 128 values clamped to 1e-4, scale = amax / 448, q = e4m3(x * ((1 / amax) * 448)): reciprocal, then
// multiply, which is how torch evaluates the recipe's `448.0 / amax` (deep_ep/utils/math.py:45-60 of the reference),
// so results equal the recipe bit for bit.
// Lane l of a pass owns 16 consecutive values; 8 consecutive lanes share a scale.
__device__ __forceinline__ void warp_quant_fanout(const int4* src, int H, unsigned long long dst, unsigned long long dst_sf,
                                                  unsigned mask, int lane) {
  const int units = H / 16, passes = (units + 31) / 32, nsf = H / 128;
  float sf_keep[2] = {0.f, 0.f};   // lane l ends up with the scales of blocks l and 32 + l
  for (int p0 = 0; p0 < passes; p0 += 2) {
    int4 raw[2][2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int u = (p0 + q) * 32 + lane;
      if (p0 + q < passes && u < units) { raw[q][0] = __ldg(src + 2 * u); raw[q][1] = __ldg(src + 2 * u + 1); }
      else { raw[q][0] = make_int4(0, 0, 0, 0); raw[q][1] = make_int4(0, 0, 0, 0); }
    }
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int p = p0 + q, u = p * 32 + lane;
      if (p >= passes) break;
      float v[16];
      float amax = amax16(raw[q][0], raw[q][1], v);
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      amax = fmaxf(amax, 1e-4f);
      const float inv = __frcp_rn(amax) * 448.0f;   // torch evaluates `448 / amax` (scalar / tensor) as reciprocal, then multiply
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        w[i] = (uint32_t)__nv_cvt_float_to_fp8(v[4 * i] * inv, __NV_SATFINITE, __NV_E4M3) |
               ((uint32_t)__nv_cvt_float_to_fp8(v[4 * i + 1] * inv, __NV_SATFINITE, __NV_E4M3) << 8) |
               ((uint32_t)__nv_cvt_float_to_fp8(v[4 * i + 2] * inv, __NV_SATFINITE, __NV_E4M3) << 16) |
               ((uint32_t)__nv_cvt_float_to_fp8(v[4 * i + 3] * inv, __NV_SATFINITE, __NV_E4M3) << 24);
      const int4 out = make_int4((int)w[0], (int)w[1], (int)w[2], (int)w[3]);
      // block p * 4 + g lives in lanes 8g..8g+7; lane l keeps the scale of block 32 * (p / 8) + l
      const float g = __shfl_sync(0xffffffffu, amax / 448.0f, (lane & 3) * 8);
      if ((lane >> 2) == (p & 7)) { if ((p >> 3) == 0) sf_keep[0] = g; else sf_keep[1] = g; }
      for (unsigned m = mask; m; m &= m - 1) {
        int4* d = reinterpret_cast<int4*>(shfl_u64(dst, __ffs(m) - 1));
        if (u < units) d[u] = out;
      }
    }
  }
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const int b = 32 * q + lane;
    for (unsigned m = mask; m; m &= m - 1) {
      float* d = reinterpret_cast<float*>(shfl_u64(dst_sf, __ffs(m) - 1));
      if (b < nsf) d[b] = sf_keep[q];
    }
  }
}

template <bool kProfile>
__global__ void __launch_bounds__(kDispatchThreads, 1) ep_dispatch_ht_kernel(const __grid_constant__ DispatchParams p) {
  const DispatchArgs& a = p.r[blockIdx.y];
  const WsLayout& lay = p.lay;
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, me = ctx.rank, Tmax = lay.max_tokens, H = lay.hidden, K = a.K;
  const int NG = (Tmax + kGroupTokens - 1) / kGroupTokens;
  const int lane = threadIdx.x & 31;
  const int q = lane >> 3, c = lane & 7;      // metadata of a group is fetched by lane = (token of the group) * 8 + field
  Control* ctl = control_of(ctx.ws[me]);
  const unsigned long long epoch = ctl->epoch[kOpDispatch] + 1;

  const bool fp8 = a.mode != kDispatchBf16;
  const int nsf = fp8 ? H / 128 : 0;
  const int row_bytes = fp8 ? H : H * 2;     // payload bytes of one output row
  const int units = row_bytes / 16;
  const bool sender = (int)blockIdx.x < p.send_blocks;
  PhaseClock<kProfile> clk;
  clk.start();

  if (sender) {
    // ================================================================ sender
    int ok = 1;
    if (lane < P) ok = wait_flag_ge(&ctl->disp_ack[lane], epoch - 1, ctx, kOpDispatch, 0, lane);
    bool alive = __all_sync(0xffffffffu, ok);
    clk.mark(kProfWait);
    const int Lx = a.E / P, ngroups = (a.T + kGroupTokens - 1) / kGroupTokens;
    const uint8_t* x = reinterpret_cast<const uint8_t*>(a.x);
    const int src_row_bytes = a.mode == kDispatchFp8Given ? H : H * 2;
    uint8_t* recv_x = reinterpret_cast<uint8_t*>(a.recv_x);
    const int my_first_row = (p.local_direct && !a.expand) ? a.rank_rows[me] : 0;
    // groups are handed out in order by a shared counter, so the warps stay busy whatever the groups' sizes
    for (int gi = next_ticket(&ctl->ticket[kOpDispatch][0], lane); gi < ngroups && alive;
         gi = next_ticket(&ctl->ticket[kOpDispatch][0], lane)) {
      const int t0 = gi * kGroupTokens, count = min(a.T - t0, kGroupTokens);
      // routing of the whole group in one round of loads: lane (q, c) holds send_slot[t0 + q][c] and the local output rows
      // of slots c and c + 8 of token t0 + q (-1: the slot's expert lives elsewhere)
      int ss = -1, sr0 = -1, sr1 = -1;
      if (q < count) {
        const int t = t0 + q;
        if (c < P) ss = a.send_slot[(size_t)t * P + c];
        if (p.local_direct && a.expand) {
          if (c < K) {
            const int r = a.slot_row[(size_t)t * K + c];
            const long long e = a.topk_idx[(size_t)t * K + c];
            if (r >= 0 && e >= 0 && e < a.E && (int)(e / Lx) == me) sr0 = r;
          }
          if (c + 8 < K) {
            const int r = a.slot_row[(size_t)t * K + c + 8];
            const long long e = a.topk_idx[(size_t)t * K + c + 8];
            if (r >= 0 && e >= 0 && e < a.E && (int)(e / Lx) == me) sr1 = r;
          }
        }
      }
      clk.mark(kProfMeta);
      for (int qq = 0; qq < count; ++qq) {
        const int t = t0 + qq;
        // lanes 0..P-1: the staged row on every destination rank; lanes P..P+K-1: the output rows on this rank
        const int j = __shfl_sync(0xffffffffu, ss, qq * 8 + (lane & 7));
        const int j_me = __shfl_sync(0xffffffffu, ss, qq * 8 + me);
        const int k = lane - P;
        const int r0 = __shfl_sync(0xffffffffu, sr0, qq * 8 + (k & 7)), r1 = __shfl_sync(0xffffffffu, sr1, qq * 8 + (k & 7));
        unsigned long long dst = 0, dst_sf = 0;
        if (lane < P) {
          if (j >= 0 && !(p.local_direct && lane == me) && DEP_INDEX_OK(ctx, j, Tmax, kOpDispatch, 0)) {
            dst = reinterpret_cast<unsigned long long>(ctx.ws[lane] + lay.stage + ((size_t)me * Tmax + j) * lay.stage_row_bytes);
            dst_sf = dst + H;
          }
        } else if (p.local_direct && k < K) {
          int row = -1;
          if (a.expand) row = k < 8 ? r0 : r1;
          else if (k == 0 && j_me >= 0) row = my_first_row + j_me;
          if (row >= 0 && (a.recv_rows <= 0 || DEP_INDEX_OK(ctx, row, a.recv_rows, kOpDispatch, 1))) {
            dst = reinterpret_cast<unsigned long long>(recv_x + (size_t)row * row_bytes);
            dst_sf = reinterpret_cast<unsigned long long>(a.recv_sf + (size_t)row * nsf);
          }
        }
        const unsigned mask = __ballot_sync(0xffffffffu, dst != 0);
        if (mask == 0) continue;
        const uint8_t* src = x + (size_t)t * src_row_bytes;
        if (a.mode == kDispatchFp8Fused) {
          warp_quant_fanout(reinterpret_cast<const int4*>(src), H, dst, dst_sf, mask, lane);
        } else {
          warp_fanout<false>(reinterpret_cast<const int4*>(src), units, dst, mask, lane);
          if (fp8) warp_fanout_f32<false>(a.x_sf + (size_t)t * nsf, nsf, dst_sf, mask, lane);
        }
        clk.add_rows(__popc(mask));
      }
      clk.mark(kProfData);
      // publish the group: every lane's stores are ordered before the flag by the warp barrier + release
      __syncwarp();
      if (lane < P && !(p.local_direct && lane == me))
        st_release_sys(reinterpret_cast<unsigned long long*>(ctx.ws[lane] + lay.disp_flag) + (size_t)me * NG + gi, epoch);
      clk.mark(kProfPublish);
    }
  }
  {
    // ================================================================ receiver (sender warps join once all groups are sent)
    uint8_t* recv_x = reinterpret_cast<uint8_t*>(a.recv_x);
    const uint8_t* stage = ctx.ws[me] + lay.stage;
    const unsigned long long* flags = reinterpret_cast<const unsigned long long*>(ctx.ws[me] + lay.disp_flag);
    // the sources whose rows pass through the staging area: all ranks, or all but this one
    const int S = p.local_direct ? P - 1 : P, first = p.local_direct ? 1 : 0;
    int max_nb = 0;
    for (int s = 0; s < S; ++s) {
      const int r = (me + first + s) % P;
      max_nb = max(max_nb, (a.rank_rows[r + 1] - a.rank_rows[r] + kRowBlock - 1) / kRowBlock);
    }
    // items are blocks of kRowBlock staged rows, block b of every source before block b + 1 of any: the order in which
    // the senders, which all walk their tokens front to back, complete them
    for (int item = next_ticket(&ctl->ticket[kOpDispatch][1], lane); item < max_nb * S;
         item = next_ticket(&ctl->ticket[kOpDispatch][1], lane)) {
      const int r = (me + first + item % S) % P, j0 = (item / S) * kRowBlock;
      const int rows_r = min(a.rank_rows[r + 1] - a.rank_rows[r], Tmax), T_r = a.rank_tokens[r];
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
      clk.mark(kProfMeta);
      int waited = -1;
      bool alive = true;
      for (int qq = 0; qq < cnt && alive; ++qq) {
        const int j = j0 + qq;
        const int t = __shfl_sync(0xffffffffu, f0, qq * 8);
        if (t < 0 || t >= T_r) {   // a record names the source token whose flag covers it: the plan is damaged
          if (lane == 0) report_failure(ctx, kStatusBadArgument, kOpDispatch, 3, r, T_r, (unsigned long long)(unsigned)t);
          alive = false;
          break;
        }
        if (t / kGroupTokens != waited) {
          waited = t / kGroupTokens;
          int ok = 1;
          if (lane == 0) ok = wait_flag_ge(flags + (size_t)r * NG + waited, epoch, ctx, kOpDispatch, 1, r);
          alive = __shfl_sync(0xffffffffu, ok, 0) != 0;
          clk.mark(kProfWait);
          if (!alive) break;
        }
        const int n = min(__shfl_sync(0xffffffffu, f0, qq * 8 + 1), kMaxTopk);
        const int fi = 2 + lane, from = qq * 8 + (fi & 7);
        const int e0 = __shfl_sync(0xffffffffu, f0, from), e1 = __shfl_sync(0xffffffffu, f1, from), e2 = __shfl_sync(0xffffffffu, f2, from);
        unsigned long long dst = 0, dst_sf = 0;
        if (lane < n) {
          const int row = ((fi >> 3) == 0 ? e0 : (fi >> 3) == 1 ? e1 : e2) & kRowMask;
          if (a.recv_rows <= 0 || DEP_INDEX_OK(ctx, row, a.recv_rows, kOpDispatch, 1)) {
            dst = reinterpret_cast<unsigned long long>(recv_x + (size_t)row * row_bytes);
            dst_sf = reinterpret_cast<unsigned long long>(a.recv_sf + (size_t)row * nsf);
          }
        }
        const unsigned mask = __ballot_sync(0xffffffffu, dst != 0);
        const uint8_t* src = stage + ((size_t)r * Tmax + j) * lay.stage_row_bytes;
        warp_fanout<true>(reinterpret_cast<const int4*>(src), units, dst, mask, lane);
        if (fp8) warp_fanout_f32<true>(reinterpret_cast<const float*>(src + H), nsf, dst_sf, mask, lane);
        clk.add_rows(__popc(mask));
        clk.mark(kProfData);
      }
      if (!alive) break;
    }
  }

  clk.finish(a.prof ? a.prof + (size_t)blockIdx.x * kDispatchProfWords : nullptr, sender ? 0 : 1);

  // ---- exit: the last block of this rank tells every source that its staged rows are consumed
  if (last_block_of_rank(ctl, kOpDispatch, gridDim.x)) {
    if (!ld_volatile_int(&ctl->abort) && threadIdx.x < P)
      st_release_sys(&control_of(ctx.ws[threadIdx.x])->disp_ack[me], epoch);
    if (threadIdx.x == 0) { ctl->ticket[kOpDispatch][0] = 0; ctl->ticket[kOpDispatch][1] = 0; ctl->epoch[kOpDispatch] = epoch; }
  }
}

cudaError_t launch_dispatch(const DispatchParams& p, int nranks, cudaStream_t stream) {
  if (p.lay.hidden > 8192) return cudaErrorInvalidValue;   // the fused quantiser keeps at most 64 scales per row in registers
  dim3 grid(p.send_blocks + p.recv_blocks, nranks), block(kDispatchThreads);
  void* args[] = {const_cast<DispatchParams*>(&p)};
  const void* fn = p.profile ? (const void*)ep_dispatch_ht_kernel<true> : (const void*)ep_dispatch_ht_kernel<false>;
  return cudaLaunchCooperativeKernel(fn, grid, block, args, 0, stream);
}

}  // namespace dep
