// Stand-alone launches of the MegaMoE routing/pull and finishing phases (see mega_route.cuh).
#include "mega_route.cuh"

namespace dep {

constexpr int kRouteThreads = 256;

long long mega_input_bytes(int M, int H, int K) { return mega_input_layout(M, H, K).total; }
void mega_input_offsets(int M, int H, int K, long long* out) {
  MegaInput l = mega_input_layout(M, H, K);
  out[0] = l.hdr; out[1] = l.x; out[2] = l.x_sf; out[3] = l.idx; out[4] = l.w; out[5] = l.total;
}

__global__ void __launch_bounds__(kRouteThreads) mega_route_kernel(const __grid_constant__ MegaRouteParams p) {
  cg::grid_group grid = cg::this_grid();
  route_phase(p.r[blockIdx.y], grid);
}

cudaError_t launch_mega_route(const MegaRouteParams& p, int nranks, int blocks, cudaStream_t stream) {
  dim3 grid(blocks, nranks), block(kRouteThreads);
  void* args[] = {const_cast<MegaRouteParams*>(&p)};
  return cudaLaunchCooperativeKernel((const void*)mega_route_kernel, grid, block, args, 0, stream);
}

__global__ void __launch_bounds__(kRouteThreads) mega_finish_kernel(const __grid_constant__ MegaFinishParams p) {
  finish_phase(p.r[blockIdx.y], true);
}

cudaError_t launch_mega_finish(const MegaFinishParams& p, int nranks, int blocks, cudaStream_t stream) {
  dim3 grid(blocks, nranks), block(kRouteThreads);
  void* args[] = {const_cast<MegaFinishParams*>(&p)};
  return cudaLaunchCooperativeKernel((const void*)mega_finish_kernel, grid, block, args, 0, stream);
}

}  // namespace dep
