// ep_combine_ht: all-to-all-v return of expert outputs fused with the top-k reduction.
//
// Expert-side blocks walk the same staged-row records that dispatch used: for one
// (source token, this rank) they sum the token's rows on this rank in slot order in fp32,
// round once to bf16 and push that single partial into the source rank's workspace over
// NVLink (a one-row group is a pure bulk copy).  A release flag per (source, 64-token chunk)
// follows.  Source-side blocks wait for the chunk flags of all ranks, sum the partials in
// rank order in fp32, add the optional biases and write bf16 into the caller's tensor.
// The optional fp32 value channel (used for dispatch-backward) is returned per slot and is
// never multiplied into the payload.
//
// Parity: csrc/kernels/combine/combine.cpp:2224-2917 of the reference in its EP8 form
// (rank-level dedup, no gateway stage): same numeric contract (fp32 sum -> bf16 partial ->
// fp32 sum -> bf16), but no entry/exit device barriers, no prepare kernel and no final
// device-to-device copy, because flags are epochs and the output is written in place.
#include "api.h"

namespace dep {

constexpr int kCombStages = 2;

__device__ __forceinline__ void fence_barrier_init2() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

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

__global__ void __launch_bounds__(256, 1) ep_combine_ht_kernel(const __grid_constant__ CombineParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const CombineArgs& a = p.r[blockIdx.y];
  const WsLayout& lay = p.lay;
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, me = ctx.rank, Tmax = lay.max_tokens, H = lay.hidden, K = a.K;
  const int NT = (Tmax + kChunkTokens - 1) / kChunkTokens;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int row_bytes = H * 2, units = H / 8;  // 16-byte units per row
  Control* ctl = control_of(ctx.ws[me]);
  const unsigned long long epoch = ctl->epoch[kOpCombine] + 1;

  if ((int)blockIdx.x < p.send_blocks) {
    // ================================================================ expert side: reduce + return
    const int slot_bytes = (row_bytes + 127) & ~127;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem) + warp * kCombStages;
    uint8_t* slots = smem + 128 + (size_t)warp * kCombStages * slot_bytes;
    if (lane == 0) {
      for (int s = 0; s < kCombStages; ++s) mbar_init(&bars[s], 1);
      fence_barrier_init2();
    }
    __syncthreads();
    uint32_t parity[kCombStages] = {0, 0};
    int ok = 1;
    if (threadIdx.x < P) ok = wait_flag_ge(&ctl->comb_ack[threadIdx.x], epoch - 1, ctx, kOpCombine, 0, threadIdx.x);
    int alive = __syncthreads_and(ok);
    int max_nt = 0;
    for (int r = 0; r < P; ++r) max_nt = max(max_nt, (a.rank_tokens[r] + kChunkTokens - 1) / kChunkTokens);
    const uint8_t* x = reinterpret_cast<const uint8_t*>(a.x);
    int it = 0;  // rows handled by this warp; picks the shared-memory slot
    for (int item = blockIdx.x; item < max_nt * P && alive; item += p.send_blocks) {
      const int c = item / P, s_rank = (me + item % P) % P;
      if (c * kChunkTokens >= a.rank_tokens[s_rank]) continue;
      const int j0 = a.chunk_start[s_rank * (NT + 1) + c], j1 = a.chunk_start[s_rank * (NT + 1) + c + 1];
      uint8_t* partial = ctx.ws[s_rank] + lay.partial;
      float* wret = reinterpret_cast<float*>(ctx.ws[s_rank] + lay.wret);
      for (int j = j0 + warp; j < j1; j += nwarps, ++it) {
        const int s = it & 1;
        const int* rec = a.stage_meta + ((size_t)s_rank * Tmax + j) * a.meta_stride;
        const int t = rec[0], n = rec[1];
        uint8_t* buf = slots + (size_t)s * slot_bytes;
        uint8_t* dst = partial + ((size_t)t * P + me) * row_bytes;
        if (lane == 0) bulk_wait_read<kCombStages - 1>();  // this slot's previous store has left shared memory
        __syncwarp();
        if (n == 1) {
          if (lane == 0) {
            mbar_expect_tx(&bars[s], row_bytes);
            bulk_g2s(buf, x + (size_t)(rec[2] & kRowMask) * row_bytes, row_bytes, &bars[s]);
          }
          if (!mbar_wait(&bars[s], parity[s])) report_failure(ctx, kStatusTimeout, kOpCombine, 10, me, 0, 0);
          parity[s] ^= 1;
        } else {
          for (int u = lane; u < units; u += 32) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int i = 0; i < n; ++i)
              add_bf16x8(acc, __ldg(reinterpret_cast<const int4*>(x + (size_t)(rec[2 + i] & kRowMask) * row_bytes) + u));
            reinterpret_cast<int4*>(buf)[u] = pack_bf16x8(acc);
          }
          fence_proxy_async_smem();
        }
        __syncwarp();
        if (lane == 0) { bulk_s2g(dst, buf, row_bytes); bulk_commit(); }
        if (a.w) {
          if (a.expand) {
            if (lane < n) wret[(size_t)t * K + (rec[2 + lane] >> kRowSlotShift)] = a.w[rec[2 + lane] & kRowMask];
          } else if (lane < K && ((rec[3] >> lane) & 1)) {
            wret[(size_t)t * K + lane] = a.w[(size_t)(rec[2] & kRowMask) * K + lane];
          }
        }
      }
      if (lane == 0) { bulk_wait<0>(); fence_proxy_async(); }
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x == 0) st_release_sys(&control_of(ctx.ws[s_rank])->comb_chunk[me][c], epoch);
    }
  } else {
    // ================================================================ source side: final reduction
    const int rb = blockIdx.x - p.send_blocks;
    const int nchunks = (a.T + kChunkTokens - 1) / kChunkTokens;
    const uint8_t* partial = ctx.ws[me] + lay.partial;
    const float* wret = reinterpret_cast<const float*>(ctx.ws[me] + lay.wret);
    int alive = 1;
    for (int c = rb; c < nchunks && alive; c += p.recv_blocks) {
      int ok = 1;
      if (threadIdx.x < P) ok = wait_flag_ge(&ctl->comb_chunk[threadIdx.x][c], epoch, ctx, kOpCombine, 1, threadIdx.x);
      alive = __syncthreads_and(ok);
      if (!alive) break;
      const int t1 = min(a.T, (c + 1) * kChunkTokens);
      for (int t = c * kChunkTokens + warp; t < t1; t += nwarps) {
        const int slot = lane < P ? a.send_slot[(size_t)t * P + lane] : -1;
        const unsigned mask = __ballot_sync(0xffffffffu, slot >= 0);
        const uint8_t* prow = partial + (size_t)t * P * row_bytes;
        int4* orow = reinterpret_cast<int4*>(reinterpret_cast<uint8_t*>(a.out) + (size_t)t * row_bytes);
        for (int u = lane; u < units; u += 32) {
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          for (unsigned m = mask; m; m &= m - 1)
            add_bf16x8(acc, ld_cg_int4(prow + (size_t)(__ffs(m) - 1) * row_bytes + (size_t)u * 16));
          if (a.bias0) add_bf16x8(acc, __ldg(reinterpret_cast<const int4*>(a.bias0 + (size_t)t * H) + u));
          if (a.bias1) add_bf16x8(acc, __ldg(reinterpret_cast<const int4*>(a.bias1 + (size_t)t * H) + u));
          orow[u] = pack_bf16x8(acc);
        }
        if (a.out_w && lane < K) {
          long long e = a.topk_idx[(size_t)t * K + lane];
          bool valid = e >= 0 && e < a.E;
          for (int q = 0; q < lane && valid; ++q) valid = a.topk_idx[(size_t)t * K + q] != e;
          a.out_w[(size_t)t * K + lane] = valid ? __ldcg(wret + (size_t)t * K + lane) : 0.f;
        }
      }
    }
  }

  if (last_block_of_rank(ctl, kOpCombine, gridDim.x)) {
    if (!ld_volatile_int(&ctl->abort) && threadIdx.x < P)
      st_release_sys(&control_of(ctx.ws[threadIdx.x])->comb_ack[me], epoch);
    if (threadIdx.x == 0) ctl->epoch[kOpCombine] = epoch;
  }
}

cudaError_t launch_combine(const CombineParams& p, int nranks, cudaStream_t stream) {
  const size_t slot = ((size_t)p.lay.hidden * 2 + 127) & ~(size_t)127;
  int warps = (int)((220 << 10) / (kCombStages * slot));
  if (warps < 1) return cudaErrorInvalidValue;
  if (warps > 8) warps = 8;
  const size_t smem = 128 + (size_t)warps * kCombStages * slot;
  cudaError_t e = cudaFuncSetAttribute(ep_combine_ht_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  dim3 grid(p.send_blocks + p.recv_blocks, nranks), block(warps * 32);
  void* args[] = {const_cast<CombineParams*>(&p)};
  return cudaLaunchCooperativeKernel((const void*)ep_combine_ht_kernel, grid, block, args, smem, stream);
}

}  // namespace dep
