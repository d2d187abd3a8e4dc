// ep_dispatch_ht: all-to-all-v token push with rank-level dedup and receive-side expansion.
//
// Sender blocks read each token row once (bulk copy global -> shared), optionally quantise it
// to e4m3 with one fp32 scale per 128 values in registers, and push it ONCE per destination
// GPU into that GPU's staging area with bulk shared -> peer-global copies over NVLink.  After a
// 64-token chunk the block publishes one release flag per destination.  Receiver blocks wait
// for (source, chunk) flags and materialise every output row of a staged row (one row per
// local expert the token routes to) with bulk copies, so a token crosses NVLink once no
// matter how many experts of the destination it uses.
//
// The reference's dispatch (csrc/kernels/dispatch/dispatch.cpp:463-590) has the same
// three jobs (payload scatter, receiver expansion from a forward list, per-source completion
// flags) but spreads them over 64 role-specialised vector cores and WQE queues; here the
// copy engines of a few SMs do the moving and the roles are sender / receiver blocks.
#include "api.h"

namespace dep {

constexpr int kStages = 2;

__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

// bf16 row in `in` -> e4m3 bytes + fp32 scales in `out` ([H] bytes, then [H/128] floats).
// amax over 128 values clamped to 1e-4, scale = amax / 448, q = e4m3(x * ((1 / amax) * 448)).
__device__ __forceinline__ void quantize_row(const uint8_t* in, uint8_t* out, int H, int lane) {
  const int nblk = H / 128;
  float* sf = reinterpret_cast<float*>(out + H);
  for (int b = 0; b < nblk; ++b) {
    uint2 raw = *reinterpret_cast<const uint2*>(in + (size_t)(b * 128 + lane * 4) * 2);
    __nv_bfloat162 p0 = *reinterpret_cast<__nv_bfloat162*>(&raw.x), p1 = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
    float v0 = __low2float(p0), v1 = __high2float(p0), v2 = __low2float(p1), v3 = __high2float(p1);
    float amax = fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    amax = fmaxf(amax, 1e-4f);
    float inv = __frcp_rn(amax) * 448.0f;  // reciprocal then multiply: the rounding sequence of the published recipe
    uint32_t q = (uint32_t)__nv_cvt_float_to_fp8(v0 * inv, __NV_SATFINITE, __NV_E4M3) |
                 ((uint32_t)__nv_cvt_float_to_fp8(v1 * inv, __NV_SATFINITE, __NV_E4M3) << 8) |
                 ((uint32_t)__nv_cvt_float_to_fp8(v2 * inv, __NV_SATFINITE, __NV_E4M3) << 16) |
                 ((uint32_t)__nv_cvt_float_to_fp8(v3 * inv, __NV_SATFINITE, __NV_E4M3) << 24);
    *reinterpret_cast<uint32_t*>(out + b * 128 + lane * 4) = q;
    if (lane == 0) sf[b] = amax / 448.0f;
  }
}

__global__ void __launch_bounds__(256, 1) ep_dispatch_ht_kernel(const __grid_constant__ DispatchParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const DispatchArgs& a = p.r[blockIdx.y];
  const WsLayout& lay = p.lay;
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, me = ctx.rank, Tmax = lay.max_tokens, H = lay.hidden;
  const int NT = (Tmax + kChunkTokens - 1) / kChunkTokens;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  Control* ctl = control_of(ctx.ws[me]);
  const unsigned long long epoch = ctl->epoch[kOpDispatch] + 1;

  const bool fp8 = a.mode != kDispatchBf16;
  const int sf_bytes = fp8 ? (H / 128) * 4 : 0;
  const int row_bytes = fp8 ? H : H * 2;                        // payload bytes of one output row
  const int moved = fp8 ? ((H + sf_bytes + 15) & ~15) : H * 2;  // bytes of one staged row
  const bool sf_bulk = (sf_bytes % 16) == 0;
  const int in_bytes = a.mode == kDispatchFp8Fused ? H * 2 : moved;
  const int out_bytes = a.mode == kDispatchFp8Fused ? moved : 0;
  const int slot_bytes = (in_bytes + out_bytes + 127) & ~127;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem) + warp * kStages;
  uint8_t* slots = smem + 128 + (size_t)warp * kStages * slot_bytes;
  if (lane == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(&bars[s], 1);
    fence_barrier_init();
  }
  __syncthreads();
  uint32_t parity[kStages] = {0, 0};

  if ((int)blockIdx.x < p.send_blocks) {
    // ================================================================ sender
    int ok = 1;
    if (threadIdx.x < P) ok = wait_flag_ge(&ctl->disp_ack[threadIdx.x], epoch - 1, ctx, kOpDispatch, 0, threadIdx.x);
    int alive = __syncthreads_and(ok);
    const int nchunks = (a.T + kChunkTokens - 1) / kChunkTokens;
    const uint8_t* x = reinterpret_cast<const uint8_t*>(a.x);
    const int src_row_bytes = a.mode == kDispatchFp8Given ? H : H * 2;

    auto issue_load = [&](int t, int s) {  // lane 0 only
      uint8_t* dst = slots + (size_t)s * slot_bytes;
      uint32_t bytes = src_row_bytes + ((a.mode == kDispatchFp8Given && sf_bulk) ? sf_bytes : 0);
      mbar_expect_tx(&bars[s], bytes);
      bulk_g2s(dst, x + (size_t)t * src_row_bytes, src_row_bytes, &bars[s]);
      if (a.mode == kDispatchFp8Given && sf_bulk)
        bulk_g2s(dst + H, reinterpret_cast<const uint8_t*>(a.x_sf) + (size_t)t * sf_bytes, sf_bytes, &bars[s]);
    };

    for (int c = blockIdx.x; c < nchunks && alive; c += p.send_blocks) {
      const int t1 = min(a.T, (c + 1) * kChunkTokens);
      int t = c * kChunkTokens + warp;
      if (t < t1 && lane == 0) issue_load(t, 0);
      for (int it = 0; t < t1; t += nwarps, ++it) {
        const int s = it & 1, tn = t + nwarps;
        if (lane == 0) {
          bulk_wait_read<0>();  // the other slot's stores have left shared memory
          if (tn < t1) issue_load(tn, s ^ 1);
        }
        int j = lane < P ? a.send_slot[(size_t)t * P + lane] : -1;
        if (!mbar_wait(&bars[s], parity[s])) report_failure(ctx, kStatusTimeout, kOpDispatch, 10, me, 0, 0);
        parity[s] ^= 1;
        uint8_t* in = slots + (size_t)s * slot_bytes;
        uint8_t* src = in;
        if (a.mode == kDispatchFp8Fused) {
          src = in + in_bytes;
          quantize_row(in, src, H, lane);
          fence_proxy_async_smem();
        } else if (a.mode == kDispatchFp8Given && !sf_bulk) {
          const float* sf = a.x_sf + (size_t)t * (H / 128);
          for (int i = lane; i < H / 128; i += 32) reinterpret_cast<float*>(in + H)[i] = sf[i];
          fence_proxy_async_smem();
        }
        __syncwarp();
        for (int d = 0; d < P; ++d) {
          int jd = __shfl_sync(0xffffffffu, j, d);
          if (jd >= 0 && lane == 0 && DEP_INDEX_OK(ctx, jd, Tmax, kOpDispatch, 0))
            bulk_s2g(ctx.ws[d] + lay.stage + ((size_t)me * Tmax + jd) * lay.stage_row_bytes, src, moved);
        }
        if (lane == 0) bulk_commit();
      }
      if (lane == 0) { bulk_wait<0>(); fence_proxy_async(); }
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x < P) st_release_sys(&control_of(ctx.ws[threadIdx.x])->disp_chunk[me][c], epoch);
    }
  } else {
    // ================================================================ receiver
    const int rb = blockIdx.x - p.send_blocks;
    int max_nt = 0;
    for (int r = 0; r < P; ++r) max_nt = max(max_nt, (a.rank_tokens[r] + kChunkTokens - 1) / kChunkTokens);
    uint8_t* recv_x = reinterpret_cast<uint8_t*>(a.recv_x);
    const uint8_t* stage = ctx.ws[me] + lay.stage;
    const int nsf = H / 128;
    int alive = 1;
    // With few ranks there are fewer (source, chunk) pairs than receiver blocks: a chunk's rows are then cut into up
    // to 8 parts that different blocks expand (about two rounds of work items over the blocks).
    const int parts = max(1, min(8, (2 * p.recv_blocks + max_nt * P - 1) / max(1, max_nt * P)));
    for (int item = rb; item < max_nt * P * parts && alive; item += p.recv_blocks) {
      const int part = item % parts, pair = item / parts;
      const int c = pair / P, r = (me + pair % P) % P;
      if (c * kChunkTokens >= a.rank_tokens[r]) continue;
      const int c0 = a.chunk_start[r * (NT + 1) + c], cn = a.chunk_start[r * (NT + 1) + c + 1] - c0;
      const int j0 = c0 + cn * part / parts, j1 = c0 + cn * (part + 1) / parts;
      if (j0 == j1) continue;
      int ok = 1;
      if (threadIdx.x == 0) ok = wait_flag_ge(&ctl->disp_chunk[r][c], epoch, ctx, kOpDispatch, 1, r);
      alive = __syncthreads_and(ok);
      if (!alive) break;
      fence_proxy_async();

      auto issue_load = [&](int j, int s) {  // lane 0 only
        mbar_expect_tx(&bars[s], moved);
        bulk_g2s(slots + (size_t)s * slot_bytes, stage + ((size_t)r * Tmax + j) * lay.stage_row_bytes, moved, &bars[s]);
      };
      int j = j0 + warp;
      if (j < j1 && lane == 0) { bulk_wait_read<0>(); issue_load(j, 0); }
      for (int it = 0; j < j1; j += nwarps, ++it) {
        const int s = it & 1, jn = j + nwarps;
        if (lane == 0) {
          bulk_wait_read<0>();
          if (jn < j1) issue_load(jn, s ^ 1);
        }
        const int* rec = a.stage_meta + ((size_t)r * Tmax + j) * a.meta_stride;
        const int n = rec[1];
        if (!mbar_wait(&bars[s], parity[s])) report_failure(ctx, kStatusTimeout, kOpDispatch, 11, r, 0, 0);
        parity[s] ^= 1;
        const uint8_t* src = slots + (size_t)s * slot_bytes;
        for (int i = 0; i < n; ++i) {
          const int row = rec[2 + i] & kRowMask;
          if (a.recv_rows > 0 && !DEP_INDEX_OK(ctx, row, a.recv_rows, kOpDispatch, 1)) continue;
          if (lane == 0) {
            bulk_s2g(recv_x + (size_t)row * row_bytes, src, row_bytes);
            if (fp8 && sf_bulk) bulk_s2g(a.recv_sf + (size_t)row * nsf, src + H, sf_bytes);
          }
          if (fp8 && !sf_bulk)
            for (int q = lane; q < nsf; q += 32) a.recv_sf[(size_t)row * nsf + q] = reinterpret_cast<const float*>(src + H)[q];
        }
        __syncwarp();
        if (lane == 0) bulk_commit();
      }
    }
    if (lane == 0) bulk_wait<0>();
  }

  // ---- exit: the last block of this rank tells every source that its staged rows are consumed
  if (last_block_of_rank(ctl, kOpDispatch, gridDim.x)) {
    if (!ld_volatile_int(&ctl->abort) && threadIdx.x < P)
      st_release_sys(&control_of(ctx.ws[threadIdx.x])->disp_ack[me], epoch);
    if (threadIdx.x == 0) ctl->epoch[kOpDispatch] = epoch;
  }
}

static size_t dispatch_slot_bytes(const WsLayout& lay, int mode) {
  const int H = lay.hidden;
  const bool fp8 = mode != kDispatchBf16;
  const int moved = fp8 ? ((H + (H / 128) * 4 + 15) & ~15) : H * 2;
  const int in_bytes = mode == kDispatchFp8Fused ? H * 2 : moved;
  const int out_bytes = mode == kDispatchFp8Fused ? moved : 0;
  return (size_t)((in_bytes + out_bytes + 127) & ~127);
}

cudaError_t launch_dispatch(const DispatchParams& p, int nranks, cudaStream_t stream) {
  const size_t slot = dispatch_slot_bytes(p.lay, p.r[0].mode);
  const size_t budget = 220 << 10;
  int warps = (int)(budget / (kStages * slot));
  if (warps < 1) return cudaErrorInvalidValue;
  if (warps > 8) warps = 8;
  const size_t smem = 128 + (size_t)warps * kStages * slot;
  cudaError_t e = cudaFuncSetAttribute(ep_dispatch_ht_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  dim3 grid(p.send_blocks + p.recv_blocks, nranks), block(warps * 32);
  void* args[] = {const_cast<DispatchParams*>(&p)};
  return cudaLaunchCooperativeKernel((const void*)ep_dispatch_ht_kernel, grid, block, args, smem, stream);
}

}  // namespace dep
