// ep_barrier: all-rank device barrier over flag words in peer memory, and a wait probe.
// Parity: csrc/kernels/instance_sync.cpp:4-18 and the notify_dispatch_barrier_kernel of
// csrc/kernels/notify/notify.cpp:1975-1982 in the reference.
#include "api.h"

namespace dep {

__global__ void ep_barrier_kernel(const __grid_constant__ BarrierParams p) {
  const RankCtx& ctx = p.r[blockIdx.x];
  Control* ctl = control_of(ctx.ws[ctx.rank]);
  const unsigned long long epoch = ctl->epoch[kOpBarrier] + 1;
  int ok = 1;
  if ((int)threadIdx.x < ctx.world) {
    __threadfence_system();
    st_release_sys(&control_of(ctx.ws[threadIdx.x])->barrier_flag[ctx.rank], epoch);
    ok = wait_flag_ge(&ctl->barrier_flag[threadIdx.x], epoch, ctx, kOpBarrier, 0, threadIdx.x);
  }
  __syncthreads_and(ok);
  if (threadIdx.x == 0) ctl->epoch[kOpBarrier] = epoch;
}

cudaError_t launch_barrier(const BarrierParams& p, int nranks, cudaStream_t stream) {
  void* args[] = {const_cast<BarrierParams*>(&p)};
  if (nranks > 1)  // virtual ranks wait on one another inside one launch: they must be co-resident
    return cudaLaunchCooperativeKernel((const void*)ep_barrier_kernel, dim3(nranks), dim3(32), args, 0, stream);
  return cudaLaunchKernel((const void*)ep_barrier_kernel, dim3(1), dim3(32), args, 0, stream);
}

// Waits (bounded by ctx.timeout_ns) for a flag word that no kernel ever writes.
__global__ void ep_wait_probe_kernel(const __grid_constant__ RankCtx ctx) {
  Control* ctl = control_of(ctx.ws[ctx.rank]);
  wait_flag_ge(&ctl->mega_flag[kMaxRanks - 1][3], ~0ull, ctx, kOpBarrier, 99, ctx.rank);
}

cudaError_t launch_wait_probe(const RankCtx& ctx, cudaStream_t stream) {
  void* args[] = {const_cast<RankCtx*>(&ctx)};
  return cudaLaunchKernel((const void*)ep_wait_probe_kernel, dim3(1), dim3(1), args, 0, stream);
}

}  // namespace dep
