// Shared device/host definitions of the expert-parallel kernels (sm_100a).
//
// Every rank owns one symmetric workspace that all peers of the NVLink domain
// map.  The first bytes of a workspace are a `Control` block: epochs owned by
// the rank itself and flag words that peers write with release stores.  All
// flags carry monotonically increasing epochs, so nothing is ever cleared
// between calls (the reference uses generation numbers the same way:
// csrc/runtime/session.hpp:86-91 of the reference).
//
// One launch can serve several *virtual ranks* that live on the same GPU
// (blockIdx.y selects the rank).  Production runs use one rank per launch;
// the virtual form exists so the cross-rank protocol can be tested on a
// single GPU inside one cooperative launch, where all blocks are co-resident.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dep {

constexpr int kMaxRanks = 8;          // one NVSwitch domain
constexpr int kChunkTokens = 64;      // tokens per routing tile of the layout pass
constexpr int kGroupTokens = 2;       // source tokens per completion flag of the high-throughput dispatch
constexpr int kRowBlock = 4;          // staged rows per work item of the local sides, and per completion flag of the combine
constexpr int kMaxChunks = 256;       // => at most 16384 tokens per rank
constexpr int kMaxTopk = 16;
constexpr int kMaxExperts = 1024;
constexpr int kRowSlotShift = 27;     // stage_meta entry = row | slot << 27
constexpr int kRowMask = (1 << kRowSlotShift) - 1;

enum Op : int {
  kOpBarrier = 0, kOpNotify = 1, kOpDispatch = 2, kOpCombine = 3, kOpLLDispatch = 4, kOpLLCombine = 5,
  kOpMega = 6, kOpA2avGmm = 7, kOpGmmA2av = 8, kNumOps = 12
};

enum Status : int { kStatusOk = 0, kStatusTimeout = 1, kStatusBadArgument = 2, kStatusAborted = 3 };

// Lives in mapped pinned host memory; the host reads it after a stream sync.
struct StatusBlock {
  int code;        // Status
  int op;          // Op
  int rank;
  int peer;
  int where;       // kernel-specific wait site
  int pad;
  unsigned long long expected;
  unsigned long long seen;
};

struct Control {
  // owned by this rank
  unsigned long long epoch[kNumOps];      // completed calls per op
  unsigned int blocks_done[kNumOps];      // exit counter used to find the last block
  unsigned int ticket[kNumOps][2];        // dynamic work counters: [0] items of the NVLink side, [1] items of the local side
  int abort;                              // set once a wait ran out; all later waits return at once
  int pad0[15];
  // written by peers (slot index = writer's rank)
  unsigned long long barrier_flag[kMaxRanks];
  unsigned long long notify_ready[kMaxRanks];
  unsigned long long notify_ack[kMaxRanks];
  unsigned long long disp_ack[kMaxRanks];
  unsigned long long comb_ack[kMaxRanks];
  unsigned long long ll_disp_ack[kMaxRanks];
  unsigned long long ll_comb_ack[kMaxRanks];
  unsigned long long mega_flag[kMaxRanks][4];
  unsigned long long gmm_flag[kMaxRanks][4];   // a2av_gmm: staged, pulled; gmm_a2av: ready, pushed
  // diagnostics: where a pipeline wait gave up (warp-indexed records of 4 words)
  unsigned long long dbg[256];
};
constexpr size_t kControlBytes = 64 << 10;
static_assert(sizeof(Control) <= kControlBytes, "control block overflows its reservation");

// Byte offsets of the regions inside a workspace; identical on every rank.
struct WsLayout {
  long long gather_hdr;    // int   [P][4]           (tokens, has_weights, -, -)
  long long gather_idx;    // int   [P][Tmax][K]
  long long gather_w;      // float [P][Tmax][K]
  long long stage;         // byte  [P][Tmax][stage_row_bytes]   dispatch staging, written by sources
  long long partial;       // bf16  [partial_tokens][P][H]        combine partials, written by expert ranks (a token window when smaller than Tmax)
  long long wret;          // float [Tmax][K]                     returned weights
  long long disp_flag;     // u64   [P][ceil(Tmax / kGroupTokens)] dispatch: the rows of (source, token group) have landed
  long long comb_flag;     // u64   [P][ceil(Tmax / kRowBlock)]    combine: the partials of (expert rank, block of its staged rows) have landed
  long long ll;            // low-latency region
  long long mega;          // fused-MoE region
  long long total;
  int max_tokens, hidden, topk, world;
  int stage_row_bytes, partial_tokens;   // partial_tokens: tokens per combine pass (Tmax unless the workspace was capped)
};

struct RankCtx {
  uint8_t* ws[kMaxRanks];     // every rank's workspace as mapped here
  StatusBlock* status;
  long long timeout_ns;
  int rank, world;
};

__host__ __device__ inline Control* control_of(uint8_t* ws) { return reinterpret_cast<Control*>(ws); }

#ifdef __CUDACC__
// ------------------------------------------------------------------ memory-model helpers
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(unsigned long long* p, unsigned long long v) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ int ld_volatile_int(const int* p) {
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void report_failure(const RankCtx& ctx, int code, int op, int where, int peer,
                                               unsigned long long expected, unsigned long long seen) {
  Control* c = control_of(ctx.ws[ctx.rank]);
  if (atomicExch(&c->abort, 1) == 0 && ctx.status != nullptr) {
    StatusBlock* s = ctx.status;
    s->op = op; s->rank = ctx.rank; s->peer = peer; s->where = where;
    s->expected = expected; s->seen = seen;
    __threadfence_system();
    s->code = code;
    __threadfence_system();
  }
}

// Optional index checking (build with DEEPEP_DEBUG_BOUNDS=1 in the environment of deepep_b200._build): an index outside its
// range is recorded in the status block (code kStatusBadArgument, wait site 100 + site, expected = limit, seen = index),
// the rank is aborted like after a time-out, and the access is skipped.  Without the flag the checks compile to nothing.
#ifdef DEEPEP_DEBUG_BOUNDS
__device__ __forceinline__ bool index_ok(const RankCtx& ctx, long long index, long long limit, int op, int site) {
  if (index >= 0 && index < limit) return true;
  report_failure(ctx, kStatusBadArgument, op, 100 + site, -1, (unsigned long long)limit, (unsigned long long)index);
  return false;
}
#define DEP_INDEX_OK(ctx, index, limit, op, site) index_ok(ctx, index, limit, op, site)
#else
#define DEP_INDEX_OK(ctx, index, limit, op, site) true
#endif

// One thread spins until *flag >= expect.  Returns false when the rank has been
// aborted or the time limit ran out (the failure is recorded for the host); the
// caller then skips its remaining work and leaves the kernel normally.
__device__ __forceinline__ bool wait_flag_ge(const unsigned long long* flag, unsigned long long expect,
                                             const RankCtx& ctx, int op, int where, int peer) {
  const Control* c = control_of(ctx.ws[ctx.rank]);
  unsigned long long t0 = 0;
  for (unsigned spins = 1;; ++spins) {
    unsigned long long v = ld_acquire_sys(flag);
    if (v >= expect) return true;
    if ((spins & 31u) == 0) {
      if (ld_volatile_int(&c->abort)) return false;
      unsigned long long now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if ((long long)(now - t0) > ctx.timeout_ns) {
        report_failure(ctx, kStatusTimeout, op, where, peer, expect, v);
        return false;
      }
      __nanosleep(64);
    }
  }
}

// Block-wide exit bookkeeping: returns true in exactly one block (the last to arrive) of
// the `nblocks` blocks of this rank.  Must be called by all threads of the block.
__device__ __forceinline__ bool last_block_of_rank(Control* c, int op, unsigned nblocks) {
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    unsigned prev = atomicAdd(&c->blocks_done[op], 1u);
    s_last = (prev == nblocks - 1);
    if (s_last) { c->blocks_done[op] = 0; __threadfence(); }
  }
  __syncthreads();
  return s_last != 0;
}

// Next work item of a shared counter (one atomic per warp); the last block of the launch sets the counters back to zero.
__device__ __forceinline__ int next_ticket(unsigned int* counter, int lane) {
  unsigned int v = 0;
  if (lane == 0) v = atomicAdd(counter, 1u);
  return (int)__shfl_sync(0xffffffffu, v, 0);
}

// ------------------------------------------------------------------ bulk-copy (TMA 1-D) helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// The hardware may park the thread for up to the hinted time before reporting "not yet",
// which keeps waiting warps from competing for issue slots with the warps that do the work.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(2000u) : "memory");
  return ok != 0;
}
// Bounded wait on a local mbarrier (completion of this CTA's own bulk loads).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (unsigned i = 0; i < (1u << 26); ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N> __device__ __forceinline__ void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// Phase clock of the profile instantiations (template <bool kProfile>): every warp charges the cycles between two
// marks to one of four phases; at the end of the kernel the block adds them up.  With kOn = false nothing is compiled in.
enum ProfPhase : int { kProfMeta = 0, kProfWait = 1, kProfData = 2, kProfPublish = 3, kProfPhases = 4 };
template <bool kOn>
struct PhaseClock {
  long long last = 0;
  long long sum[kProfPhases] = {0, 0, 0, 0};
  unsigned long long rows = 0, begin_ns = 0;
  __device__ __forceinline__ void start() { if (kOn) { last = clock64(); begin_ns = global_timer_ns(); } }
  __device__ __forceinline__ void mark(int phase) {
    if (kOn) { const long long now = clock64(); sum[phase] += now - last; last = now; }
  }
  __device__ __forceinline__ void add_rows(int n) { if (kOn) rows += n; }
  // all threads of the block; `out` = 8 words: role, start ns, end ns, 4 phase sums (cycles), rows
  __device__ __forceinline__ void finish(unsigned long long* out, int role) {
    if (!kOn) return;
    __shared__ unsigned long long s_acc[kProfPhases + 1];
    if (threadIdx.x <= kProfPhases) s_acc[threadIdx.x] = 0;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) {
      for (int i = 0; i < kProfPhases; ++i) atomicAdd(&s_acc[i], (unsigned long long)sum[i]);
      atomicAdd(&s_acc[kProfPhases], rows);
    }
    __syncthreads();
    if (threadIdx.x == 0 && out != nullptr) {
      out[0] = role; out[1] = begin_ns; out[2] = global_timer_ns();
      for (int i = 0; i <= kProfPhases; ++i) out[3 + i] = s_acc[i];
    }
  }
};

__device__ __forceinline__ int4 ld_cg_int4(const void* p) { return __ldcg(reinterpret_cast<const int4*>(p)); }

// Warp-wide copy of `units` 16-byte pieces from `src` to `ndst` destinations.  All loads of a batch of U pieces per
// lane are issued before the first store, so a row costs a few memory latencies instead of one per piece.
template <int U>
__device__ __forceinline__ void warp_copy_row(int4* const* dst, int ndst, const int4* src, int units, int lane) {
  for (int u0 = 0; u0 < units; u0 += 32 * U) {
    int4 v[U];
#pragma unroll
    for (int i = 0; i < U; ++i) {
      const int u = u0 + i * 32 + lane;
      if (u < units) v[i] = __ldcg(src + u);
    }
#pragma unroll
    for (int i = 0; i < U; ++i) {
      const int u = u0 + i * 32 + lane;
      if (u < units)
        for (int d = 0; d < ndst; ++d) dst[d][u] = v[i];
    }
  }
}
__device__ __forceinline__ void warp_copy_row1(int4* dst, const int4* src, int units, int lane) {
  int4* one[1] = {dst};
  warp_copy_row<8>(one, 1, src, units, lane);
}
#endif  // __CUDACC__

}  // namespace dep
