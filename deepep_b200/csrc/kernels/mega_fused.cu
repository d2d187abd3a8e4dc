// mega_moe: the whole MoE layer of one rank in ONE persistent cooperative kernel.
//
//   phase 1  route_phase   handshake with the peers, routing tables read from peer memory, expert tiles,
//                          pull of the routed e4m3 rows + scales over NVLink          (grid barriers inside)
//   phase 2  gemm_phase    GEMM1 (+SwiGLU + MXFP8 requant) and GEMM2 (+ bf16 rows stored into the source
//                          ranks' combine slots over NVLink) as one tile list on tcgen05 / TMEM; a GEMM2
//                          tile starts as soon as the GEMM1 tiles of its row block are done
//   phase 3  finish_phase  handshake, y[t] = sum_k w[t, k] * row[t, k]
// One CTA per SM stays resident for all three phases; the phases are separated by grid barriers on this
// GPU and by flag words in peer memory across GPUs.
//
// Parity: mega_moe_kernel of the reference (experiments/megamoe/csrc/kernels/mega_moe/mega_moe.cpp:22-81,
// mega_moe_arch35.hpp:852-1006): input preparation / route / cross-rank sync, expert waves of
// dispatch + GMM1 + activation-quant + GMM2 + combine, cross-rank sync, unpermute.
#include <cooperative_groups.h>

#include "mega_gemm.cuh"
#include "mega_route.cuh"

namespace dep {

constexpr int kPullWarps = 2;                                    // warps beside the GEMM roles that pull tokens from peers
constexpr int kFusedThreads = kGemmThreads + kPullWarps * 32;

template <bool kPair>
__global__ void __launch_bounds__(kFusedThreads, 1) mega_moe_kernel(const __grid_constant__ MegaFusedParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ RouteShared sh;
  cg::grid_group grid = cg::this_grid();
  const MegaFusedArgs& a = p.r[blockIdx.y];
  if (blockIdx.x == 0)
  {
    for (int i = threadIdx.x; i < a.route.max_mtiles; i += blockDim.x) { a.ready[i] = 0; a.route.pulled[i] = 0; }
    if (threadIdx.x == 0 && a.tile_counter) *a.tile_counter = 0;
  }
  route_layout_phase(a.route, grid, sh);          // handshake, counts, tile layout (grid barriers inside)
  __threadfence();
  grid.sync();
  // The token pull overlaps the GEMMs: rows are pulled tile by tile, a GEMM1 tile starts once its rows have arrived.
  const int warp = threadIdx.x >> 5;
  if (warp < kGemmThreads / 32) {
    unsigned long long* stats = a.route.timer ? a.route.timer + (size_t)blockIdx.x * kMegaTimerWords + kTimMmaThread : nullptr;
    if constexpr (kPair) gemm_phase<true>(a.g1, &a.g2, a.ready, smem_raw, 4, blockIdx.x / 2, gridDim.x / 2, a.tile_counter, a.interleave, 1, stats);
    else gemm_phase<false>(a.g1, &a.g2, a.ready, smem_raw, 3, blockIdx.x, gridDim.x, a.tile_counter, a.interleave, 1, stats);
  } else {
    // the pull warps take part in the block (and, for CTA pairs, cluster) barriers of gemm_phase's set-up and tear-down
    if constexpr (kPair) { __syncthreads(); umma::cluster_sync_all(); }
    __syncthreads();
    route_pull_phase(a.route, sh, blockIdx.x * kPullWarps + (warp - kGemmThreads / 32), gridDim.x * kPullWarps);
    __syncthreads();
    if constexpr (kPair) umma::cluster_sync_all();
  }
  mega_stamp(a.route.timer, kTimGemm);             // this CTA ran out of tiles (or of rows to pull)
  __threadfence_system();
  grid.sync();
  finish_phase(a.finish, true);
}

cudaError_t launch_mega_fused(const MegaFusedParams& p, int nranks, int blocks, cudaStream_t stream) {
  const size_t smem = gemm_smem_bytes(3, true);
  bool pair = p.r[0].pair != 0;
  for (int i = 0; i < nranks; ++i)
    if ((p.r[i].pair != 0) != pair || (p.r[i].route.tile_pairs != 0) != pair) return cudaErrorInvalidValue;
  const void* fn = pair ? (const void*)mega_moe_kernel<true> : (const void*)mega_moe_kernel<false>;
  // the attribute belongs to the current device, so it is set on every launch (a process may drive several GPUs)
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  void* args[] = {const_cast<MegaFusedParams*>(&p)};
  if (!pair) return cudaLaunchCooperativeKernel(fn, dim3(blocks, nranks), dim3(kFusedThreads), args, smem, stream);
  // CTA pairs: a cooperative launch of clusters of two CTAs (an even number of CTAs per rank)
  if (blocks < 2) return cudaErrorInvalidValue;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks / 2 * 2, nranks); cfg.blockDim = dim3(kFusedThreads);
  cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeCooperative;
  attr[1].val.cooperative = 1;
  cfg.attrs = attr; cfg.numAttrs = 2;
  return cudaLaunchKernelExC(&cfg, fn, args);
}

}  // namespace dep
