// ep_combine_ht: all-to-all-v return of expert outputs fused with the top-k reduction.
//
// Expert-side blocks walk the same staged-row records that dispatch used: for one
// (source token, this rank) they sum the token's rows on this rank in slot order in fp32,
// round once to bf16 and push that single partial into the source rank's workspace over
// NVLink (a one-row group is a pure bulk copy).  A release flag per (source, 64-token chunk)
// follows.  With few ranks there are fewer (source, chunk) pairs than SMs, so a chunk is cut into
// up to 8 parts that different blocks take; the block that finishes a chunk's last part publishes.  Source-side blocks wait for the chunk flags of all ranks, sum the partials in
// rank order in fp32, add the optional biases and write bf16 into the caller's tensor.
// The optional fp32 value channel (used for dispatch-backward) is returned per slot and is
// never multiplied into the payload.
//
// Both sides are the same shared-memory ring pipeline: warp 0 streams rows into a ring of row
// slots with bulk copies (up to ~220 KB in flight per SM; its lanes fill the slots of a batch of
// groups in parallel), warps 1..7 each take every
// 7th group, wait for the group's slots, reduce them in place from shared memory and hand the
// result to a bulk store.  Row movement never touches registers unless a sum is needed.
//
// Parity: csrc/kernels/combine/combine.cpp:2224-2917 of the reference in its EP8 form
// (rank-level dedup, no gateway stage): same numeric contract (fp32 sum -> bf16 partial ->
// fp32 sum -> bf16), but no entry/exit device barriers, no prepare kernel and no final
// device-to-device copy, because flags are epochs and the output is written in place.
#include "api.h"

namespace dep {

constexpr int kRingMaxSlots = 56;    // 2 x 56 barriers + the fill counter fit the 1 KB ring header
constexpr int kStreamUnits = 7;      // 16-byte pieces per lane of a quarter row (hidden <= 7168) in the streaming reduction
constexpr int kRingMaxRows = 8;      // larger groups are summed straight from global memory (see ring_rows)
constexpr int kCombineThreads = 256;
constexpr int kConsumerWarps = kCombineThreads / 32 - 1;

__device__ __forceinline__ void fence_barrier_init2() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory"); }

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

// Slots are filled strictly in ring order by one producer thread, but the uses of one slot are
// consumed by different warps.  An mbarrier wait only names a phase parity, so a warp waiting for
// use u of a slot could mistake the completed use u - 2 for its own.  `issued` (the number of fills
// the producer has started) removes the ambiguity: a consumer first waits until fill k was issued,
// after which the slot's barrier can only be in the phase of use k.
struct Ring {
  uint64_t* full;
  uint64_t* empty;
  volatile unsigned* issued;
  uint8_t* slots;
  int num_slots, slot_bytes;
  const Control* ctl;
  __device__ __forceinline__ uint8_t* slot(unsigned k) const { return slots + (size_t)(k % num_slots) * slot_bytes; }
  __device__ __forceinline__ uint32_t phase(unsigned k) const { return (k / num_slots) & 1u; }
  // Bounded; also gives up as soon as the rank is aborted.
  __device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity) const {
    for (unsigned i = 1; i < (1u << 28); ++i) {
      if (mbar_try_wait(bar, parity)) return true;
      if ((i & 255u) == 0 && ld_volatile_int(&ctl->abort)) break;
    }
    if ((threadIdx.x & 31) == 0) {  // leave a record of the wait that gave up
      unsigned long long* d = const_cast<unsigned long long*>(ctl->dbg) + ((blockIdx.x & 7) * 8 + (threadIdx.x >> 5)) * 4;
      d[0] = 0xdead0000ull | blockIdx.x;
      d[1] = (unsigned long long)(bar - full);   // < 32: full[slot]; >= 32: empty[slot - 32]
      d[2] = parity;
      d[3] += 1;
    }
    return false;
  }
  // producer (one thread)
  __device__ __forceinline__ bool push(unsigned k, const void* src, uint32_t bytes) const {
    if (!wait(&empty[k % num_slots], phase(k) ^ 1u)) return false;
    mbar_expect_tx(&full[k % num_slots], bytes);
    bulk_g2s(slot(k), src, bytes, &full[k % num_slots]);
    __threadfence_block();
    *issued = k + 1;
    return true;
  }
  // Lane-parallel variants: several lanes of the producer warp each fill one slot of a batch; the caller publishes the
  // batch afterwards with publish().  Issuing the copies from several lanes overlaps the waits and the issue latency
  // that a single producer thread pays one after the other (about 0.25 us per copy).
  __device__ __forceinline__ bool fill(unsigned k, const void* src, uint32_t bytes) const {
    if (!wait(&empty[k % num_slots], phase(k) ^ 1u)) return false;
    mbar_expect_tx(&full[k % num_slots], bytes);
    bulk_g2s(slot(k), src, bytes, &full[k % num_slots]);
    return true;
  }
  __device__ __forceinline__ bool fill_empty(unsigned k) const {
    if (!wait(&empty[k % num_slots], phase(k) ^ 1u)) return false;
    mbar_arrive(&full[k % num_slots]);
    return true;
  }
  __device__ __forceinline__ void publish(unsigned k_end) const {   // one lane, after __syncwarp()
    __threadfence_block();
    *issued = k_end;
  }
  __device__ __forceinline__ bool push_empty(unsigned k) const {
    if (!wait(&empty[k % num_slots], phase(k) ^ 1u)) return false;
    mbar_arrive(&full[k % num_slots]);
    __threadfence_block();
    *issued = k + 1;
    return true;
  }
  // warp-collective: lane 0 watches the fill counter, then every lane acquires the slot's barrier
  __device__ __forceinline__ bool wait_full(unsigned k) const {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) {
      for (unsigned i = 1; *issued <= k; ++i) {
        __nanosleep(100);
        if ((i & 63u) == 0 && (ld_volatile_int(&ctl->abort) || i > (1u << 24))) { ok = 0; break; }
      }
      __threadfence_block();
    }
    if (!__shfl_sync(0xffffffffu, ok, 0)) return false;
    return wait(&full[k % num_slots], phase(k));
  }
  __device__ __forceinline__ void release(unsigned k) const { mbar_arrive(&empty[k % num_slots]); }
};

// Sum `n` (<= kRingMaxRows) ring slots starting at k (fp32, slot order) into slot k; biases are added last.
__device__ __forceinline__ void reduce_slots(const Ring& ring, unsigned k, int n, int units, int lane,
                                             const int4* bias0, const int4* bias1) {
  const int4* rows[kRingMaxRows];
#pragma unroll
  for (int i = 0; i < kRingMaxRows; ++i) rows[i] = reinterpret_cast<const int4*>(ring.slot(k + (i < n ? i : 0)));
  int4* out = reinterpret_cast<int4*>(ring.slot(k));
  int u = lane;
  for (; u + 32 < units; u += 64) {   // two independent 16-byte columns per step
    float a0[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, a1[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < kRingMaxRows; ++i)
      if (i < n) { int4 v0 = rows[i][u], v1 = rows[i][u + 32]; add_bf16x8(a0, v0); add_bf16x8(a1, v1); }
    if (bias0) { add_bf16x8(a0, __ldg(bias0 + u)); add_bf16x8(a1, __ldg(bias0 + u + 32)); }
    if (bias1) { add_bf16x8(a0, __ldg(bias1 + u)); add_bf16x8(a1, __ldg(bias1 + u + 32)); }
    out[u] = pack_bf16x8(a0);
    out[u + 32] = pack_bf16x8(a1);
  }
  for (; u < units; u += 32) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < kRingMaxRows; ++i)
      if (i < n) add_bf16x8(acc, rows[i][u]);
    if (bias0) add_bf16x8(acc, __ldg(bias0 + u));
    if (bias1) add_bf16x8(acc, __ldg(bias1 + u));
    out[u] = pack_bf16x8(acc);
  }
}

// lane 0: store slot k to `dst`, then hand the slot back as soon as the copy engine has read it.
// (A slot is never kept across groups: the producer refills slots strictly in ring order, so a slot
// held until the warp's next group could block the producer from ever loading that group.)
__device__ __forceinline__ void store_and_release(const Ring& ring, unsigned k, void* dst, uint32_t bytes) {
  bulk_s2g(dst, ring.slot(k), bytes);
  bulk_commit();
  bulk_wait_read<0>();
  ring.release(k);
}

__global__ void __launch_bounds__(kCombineThreads, 1) ep_combine_ht_kernel(const __grid_constant__ CombineParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const CombineArgs& a = p.r[blockIdx.y];
  const WsLayout& lay = p.lay;
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, me = ctx.rank, Tmax = lay.max_tokens, H = lay.hidden, K = a.K;
  const int NT = (Tmax + kChunkTokens - 1) / kChunkTokens;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_bytes = H * 2, units = H / 8;  // 16-byte units per row
  Control* ctl = control_of(ctx.ws[me]);
  const unsigned long long epoch = ctl->epoch[kOpCombine] + 1;

  const bool expert_side = (int)blockIdx.x < p.send_blocks;
  // With one or two ranks a token has up to top-k rows on this rank, and a ring of ~15 whole rows cannot hold two such
  // groups: the expert side then works on quarter (or half) rows, so that later groups load while one is reduced.
  // Quarter rows also let a consumer keep a group's running sum in registers and hand every slot back as soon as it
  // has been added (`stream`), which turns the ring into a FIFO whose throughput is its size over the load latency.
  const int cparts = !(expert_side && P <= 2) ? 1 : (row_bytes / 4) % 128 == 0 ? 4 : (row_bytes / 2) % 128 == 0 ? 2 : 1;
  const bool stream = cparts == 4 && units / 4 <= 32 * kStreamUnits;
  const int seg_bytes = row_bytes / cparts, seg_units = units / cparts;
  Ring ring;
  ring.slot_bytes = (seg_bytes + 127) & ~127;
  // the launch sizes the ring for whole rows (see launch_combine): half rows must stay inside those bytes
  const int full_slot = (row_bytes + 127) & ~127;
  const int ring_bytes = min(kRingMaxSlots, (int)((220 << 10) / full_slot)) * full_slot;
  ring.num_slots = min(kRingMaxSlots, ring_bytes / ring.slot_bytes);
  ring.full = reinterpret_cast<uint64_t*>(smem);
  ring.empty = ring.full + kRingMaxSlots;
  ring.issued = reinterpret_cast<volatile unsigned*>(ring.empty + kRingMaxSlots);
  if (threadIdx.x == 0) *ring.issued = 0;
  ring.slots = smem + 1024;
  ring.ctl = ctl;
  const int ring_rows = min(kRingMaxRows, ring.num_slots);  // rows of one group that may sit in the ring
  if (threadIdx.x < ring.num_slots) {
    mbar_init(&ring.full[threadIdx.x], 1);
    mbar_init(&ring.empty[threadIdx.x], 1);
    fence_barrier_init2();
  }
  __syncthreads();

  int alive = 1;
  if (expert_side) {
    int ok = 1;
    if (threadIdx.x < P) ok = wait_flag_ge(&ctl->comb_ack[threadIdx.x], epoch - 1, ctx, kOpCombine, 0, threadIdx.x);
    alive = __syncthreads_and(ok);
  }

  if (alive && expert_side) {
    // ================================================================ expert side: reduce + return
    int max_nt = 0;
    for (int r = 0; r < P; ++r) max_nt = max(max_nt, (a.rank_tokens[r] + kChunkTokens - 1) / kChunkTokens);
    const uint8_t* x = reinterpret_cast<const uint8_t*>(a.x);
    // parts per (source, chunk): enough work items for about two rounds over the expert-side blocks
    const int parts = max(1, min(8, (2 * p.send_blocks + max_nt * P - 1) / max(1, max_nt * P)));
    const int num_items = max_nt * P * parts;
    unsigned k = 0;
    long long t_a = 0, t_b = 0, t_c = 0, t_d = 0, t0 = clock64(), tt;
    if (warp == 0) {
      // Producer: the whole warp.  A batch takes up to 8 consecutive records whose slots fit the ring; lane l fills
      // the l-th slot of the batch (record r, column part h, row i), then lane 0 publishes the batch.
      bool okp = true;
      for (int item = blockIdx.x; item < num_items && okp; item += p.send_blocks) {
        const int part = item % parts, pair = item / parts;
        const int c = pair / P, s_rank = (me + pair % P) % P;
        if (c * kChunkTokens >= a.rank_tokens[s_rank]) continue;
        const int c0 = a.chunk_start[s_rank * (NT + 1) + c], cn = a.chunk_start[s_rank * (NT + 1) + c + 1] - c0;
        const int j0 = c0 + cn * part / parts, j1 = c0 + cn * (part + 1) / parts;
        const int cap = min(32, ring.num_slots);
        if (stream) {
          // streaming consumers hand slots back one by one: publish every (record, column part) on its own so that
          // the consumers start on a group while the following ones are still being issued
          for (int j = j0; j < j1 && okp; ++j) {
            const int* rec = a.stage_meta + ((size_t)s_rank * Tmax + j) * a.meta_stride;
            const int n = rec[1], nn = n <= ring_rows ? n : 1;
            for (int h = 0; h < cparts && okp; ++h) {
              int ok = 1;
              if (lane < nn) {
                if (n <= ring_rows)
                  ok = (a.x_rows <= 0 || DEP_INDEX_OK(ctx, rec[2 + lane] & kRowMask, a.x_rows, kOpCombine, 0))
                           ? ring.fill(k + lane, x + (size_t)(rec[2 + lane] & kRowMask) * row_bytes + (size_t)h * seg_bytes, seg_bytes)
                           : ring.fill_empty(k + lane);
                else
                  ok = ring.fill_empty(k + lane);
              }
              okp = __all_sync(0xffffffffu, ok);
              __syncwarp();
              if (lane == 0 && okp) ring.publish(k + nn);
              k += nn;
            }
          }
          continue;
        }
        for (int jb = j0; jb < j1 && okp;) {
          // lanes 0..7: slots of record jb + lane
          int my_n = 0, my_slots = 0;
          if (lane < 8 && jb + lane < j1) {
            my_n = a.stage_meta[((size_t)s_rank * Tmax + jb + lane) * a.meta_stride + 1];
            my_slots = (my_n <= ring_rows ? my_n : 1) * cparts;
          }
          int incl = my_slots;
#pragma unroll
          for (int d = 1; d < 8; d <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += o;
          }
          // records taken: those whose slots end within the capacity (at least the first one)
          const unsigned fit = __ballot_sync(0xffffffffu, lane < 8 && jb + lane < j1 && (incl <= cap || lane == 0));
          const int count = __ffs(~fit) - 1;                       // fit is a run of ones from bit 0
          const int total = __shfl_sync(0xffffffffu, incl, count - 1);
          // lane l -> (record r, index inside the record)
          int r = 0, base = 0;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int e = __shfl_sync(0xffffffffu, incl, q);
            if (q < count && lane >= e) { r = q + 1; base = e; }
          }
          int ok = 1;
          if (lane < total) {
            const int* rec = a.stage_meta + ((size_t)s_rank * Tmax + jb + r) * a.meta_stride;
            const int n = rec[1], nn = n <= ring_rows ? n : 1;
            const int idx = lane - base, h = idx / nn, i = idx - h * nn;
            if (n <= ring_rows)
              ok = (a.x_rows <= 0 || DEP_INDEX_OK(ctx, rec[2 + i] & kRowMask, a.x_rows, kOpCombine, 0))
                       ? ring.fill(k + lane, x + (size_t)(rec[2 + i] & kRowMask) * row_bytes + (size_t)h * seg_bytes, seg_bytes)
                       : ring.fill_empty(k + lane);
            else
              ok = ring.fill_empty(k + lane);
          }
          okp = __all_sync(0xffffffffu, ok);
          __syncwarp();
          if (lane == 0 && okp) ring.publish(k + total);
          k += total;
          jb += count;
        }
      }
    } else {
      const int cw = warp - 1;
      unsigned q = 0;
      bool dead = false;
      for (int item = blockIdx.x; item < num_items; item += p.send_blocks) {
        const int part = item % parts, pair = item / parts;
        const int c = pair / P, s_rank = (me + pair % P) % P;
        if (c * kChunkTokens >= a.rank_tokens[s_rank]) continue;
        const int c0 = a.chunk_start[s_rank * (NT + 1) + c], cn = a.chunk_start[s_rank * (NT + 1) + c + 1] - c0;
        const int j0 = c0 + cn * part / parts, j1 = c0 + cn * (part + 1) / parts;
        uint8_t* partial = ctx.ws[s_rank] + lay.partial;
        float* wret = reinterpret_cast<float*>(ctx.ws[s_rank] + lay.wret);
        for (int j = j0; j < j1; ++j) {
          const int* rec = a.stage_meta + ((size_t)s_rank * Tmax + j) * a.meta_stride;
          const int t = rec[0], n = rec[1];
          const int nslots = n <= ring_rows ? n : 1;
          for (int h = 0; h < cparts; ++h, ++q, k += nslots) {
            if ((int)(q % kConsumerWarps) != cw || dead) continue;
            tt = clock64();
            if (stream && n > 1 && n <= ring_rows) {
              // running sum in registers (fp32, slot order); every slot but the last goes back as soon as it was added
              float acc[kStreamUnits][8];
#pragma unroll
              for (int v = 0; v < kStreamUnits; ++v)
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[v][e] = 0.f;
              for (int i = 0; i < n && !dead; ++i) {
                dead = !ring.wait_full(k + i);
                if (dead) break;
                const int4* row = reinterpret_cast<const int4*>(ring.slot(k + i));
#pragma unroll
                for (int v = 0; v < kStreamUnits; ++v)
                  if (lane + 32 * v < seg_units) add_bf16x8(acc[v], row[lane + 32 * v]);
                if (i + 1 < n) {
                  __syncwarp();
                  if (lane == 0) ring.release(k + i);
                }
              }
              if (dead) continue;
              int4* out = reinterpret_cast<int4*>(ring.slot(k + n - 1));
#pragma unroll
              for (int v = 0; v < kStreamUnits; ++v)
                if (lane + 32 * v < seg_units) out[lane + 32 * v] = pack_bf16x8(acc[v]);
              fence_proxy_async_smem();
              __syncwarp();
              t_b += clock64() - tt; tt = clock64();
              if (lane == 0) store_and_release(ring, k + n - 1, partial + ((size_t)t * P + me) * row_bytes + (size_t)h * seg_bytes, seg_bytes);
              t_c += clock64() - tt;
              if (a.w && h == 0) {
                if (a.expand) {
                  if (lane < n) wret[(size_t)t * K + (rec[2 + lane] >> kRowSlotShift)] = a.w[rec[2 + lane] & kRowMask];
                } else if (lane < K && ((rec[3] >> lane) & 1)) {
                  wret[(size_t)t * K + lane] = a.w[(size_t)(rec[2] & kRowMask) * K + lane];
                }
              }
              continue;
            }
            for (int i = 0; i < nslots && !dead; ++i) dead = !ring.wait_full(k + i);
            t_a += clock64() - tt; tt = clock64();
            if (dead) continue;
            if (n > ring_rows) {  // rare: more rows than a group may hold in the ring
              int4* out = reinterpret_cast<int4*>(ring.slot(k));
              for (int u = lane; u < seg_units; u += 32) {
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (int i = 0; i < n; ++i)
                  add_bf16x8(acc, __ldg(reinterpret_cast<const int4*>(x + (size_t)(rec[2 + i] & kRowMask) * row_bytes + (size_t)h * seg_bytes) + u));
                out[u] = pack_bf16x8(acc);
              }
              fence_proxy_async_smem();
            } else if (n > 1) {
              reduce_slots(ring, k, n, seg_units, lane, nullptr, nullptr);
              fence_proxy_async_smem();
            }
            __syncwarp();
            t_b += clock64() - tt; tt = clock64();
            if (lane == 0) {
              for (int i = 1; i < nslots; ++i) ring.release(k + i);
              store_and_release(ring, k, partial + ((size_t)t * P + me) * row_bytes + (size_t)h * seg_bytes, seg_bytes);
            }
            t_c += clock64() - tt;
            if (a.w && h == 0) {
              if (a.expand) {
                if (lane < n) wret[(size_t)t * K + (rec[2 + lane] >> kRowSlotShift)] = a.w[rec[2 + lane] & kRowMask];
              } else if (lane < K && ((rec[3] >> lane) & 1)) {
                wret[(size_t)t * K + lane] = a.w[(size_t)(rec[2] & kRowMask) * K + lane];
              }
            }
          }
        }
        // this part's partials are complete; whoever finishes the last part of the (source, chunk) publishes it
        tt = clock64();
        if (lane == 0) { bulk_wait<0>(); fence_proxy_async(); }
        __threadfence_system();
        consumer_barrier();
        t_d += clock64() - tt;
        if (warp == 1 && lane == 0) {
          bool last = true;
          if (parts > 1) {
            last = atomicAdd(&ctl->comb_parts[s_rank][c], 1u) + 1u == (unsigned)parts;
            if (last) ctl->comb_parts[s_rank][c] = 0u;     // ready for the next call
            __threadfence_system();
          }
          if (last && !ld_volatile_int(&ctl->abort)) st_release_sys(&control_of(ctx.ws[s_rank])->comb_chunk[me][c], epoch);
        }
      }
      if (blockIdx.x < 8 && lane == 0) { unsigned long long* d = ctl->dbg + (blockIdx.x * 8 + warp) * 4; d[0] = t_a; d[1] = t_b; d[2] = t_c; d[3] = t_d; }
    }
  } else if (alive) {
    // ================================================================ source side: final reduction
    const int rb = blockIdx.x - p.send_blocks;
    const int nchunks = (a.T + kChunkTokens - 1) / kChunkTokens;
    const uint8_t* partial = ctx.ws[me] + lay.partial;
    const float* wret = reinterpret_cast<const float*>(ctx.ws[me] + lay.wret);
    uint8_t* out = reinterpret_cast<uint8_t*>(a.out);
    unsigned k = 0;
    if (warp == 0) {
      bool okp = true;
      for (int c = rb; c < nchunks && okp; c += p.recv_blocks) {
        int ok = 1;
        if (lane < P) ok = wait_flag_ge(&ctl->comb_chunk[lane][c], epoch, ctx, kOpCombine, 1, lane);
        okp = __all_sync(0xffffffffu, ok);
        if (!okp) break;
        fence_proxy_async();
        const int t1 = min(a.T, (c + 1) * kChunkTokens);
        // four tokens per batch: lane = (token, rank); every partial of the batch is loaded by its own lane
        const int cap = min(32, ring.num_slots);
        for (int t = c * kChunkTokens; t < t1 && okp;) {
          const int tt = lane >> 3, d = lane & 7;
          const bool has = d < P && t + tt < t1 && a.send_slot[(size_t)(t + tt) * P + d] >= 0;
          const unsigned m32 = __ballot_sync(0xffffffffu, has);
          int off[5], take = 0;
          off[0] = 0;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int n = __popc((m32 >> (8 * q)) & 0xffu);
            const int ns = (n && n <= ring_rows) ? n : 1;
            off[q + 1] = off[q] + ns;
            if (t + q < t1 && (off[q + 1] <= cap || q == 0) && take == q) take = q + 1;
          }
          int ok = 1;
          if (tt < take) {
            const unsigned seg = (m32 >> (8 * tt)) & 0xffu;
            const int n = __popc(seg);
            if (n && n <= ring_rows) {
              if (has) ok = ring.fill(k + off[tt] + __popc(seg & ((1u << d) - 1u)), partial + ((size_t)(t + tt) * P + d) * row_bytes, row_bytes);
            } else if (d == 0) {
              ok = ring.fill_empty(k + off[tt]);
            }
          }
          okp = __all_sync(0xffffffffu, ok);
          __syncwarp();
          if (lane == 0 && okp) ring.publish(k + off[take]);
          k += off[take];
          t += take;
        }
      }
    } else {
      const int cw = warp - 1;
      unsigned q = 0;
      bool dead = false;
      for (int c = rb; c < nchunks; c += p.recv_blocks) {
        const int t1 = min(a.T, (c + 1) * kChunkTokens);
        for (int t = c * kChunkTokens; t < t1; ++t, ++q) {
          const int slot = lane < P ? a.send_slot[(size_t)t * P + lane] : -1;
          const unsigned dmask = __ballot_sync(0xffffffffu, slot >= 0);
          const int n = __popc(dmask);
          const int nslots = (n && n <= ring_rows) ? n : 1;
          if ((int)(q % kConsumerWarps) == cw && !dead) {
            for (int i = 0; i < nslots && !dead; ++i) dead = !ring.wait_full(k + i);
            if (!dead) {
              const int4* b0 = a.bias0 ? reinterpret_cast<const int4*>(a.bias0 + (size_t)t * H) : nullptr;
              const int4* b1 = a.bias1 ? reinterpret_cast<const int4*>(a.bias1 + (size_t)t * H) : nullptr;
              if (n > ring_rows) {  // more partials than a group may hold in the ring: read them directly
                int4* dst = reinterpret_cast<int4*>(ring.slot(k));
                for (int u = lane; u < units; u += 32) {
                  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                  for (unsigned m = dmask; m; m &= m - 1)
                    add_bf16x8(acc, ld_cg_int4(partial + ((size_t)t * P + (__ffs(m) - 1)) * row_bytes + (size_t)u * 16));
                  if (b0) add_bf16x8(acc, __ldg(b0 + u));
                  if (b1) add_bf16x8(acc, __ldg(b1 + u));
                  dst[u] = pack_bf16x8(acc);
                }
                fence_proxy_async_smem();
              } else if (n != 1 || b0 || b1) {
                reduce_slots(ring, k, n, units, lane, b0, b1);
                fence_proxy_async_smem();
              }
              __syncwarp();
              if (lane == 0) {
                for (int i = 1; i < nslots; ++i) ring.release(k + i);
                store_and_release(ring, k, out + (size_t)t * row_bytes, row_bytes);
              }
              if (a.out_w && lane < K) {
                long long e = a.topk_idx[(size_t)t * K + lane];
                bool valid = e >= 0 && e < a.E;
                for (int z = 0; z < lane && valid; ++z) valid = a.topk_idx[(size_t)t * K + z] != e;
                a.out_w[(size_t)t * K + lane] = valid ? __ldcg(wret + (size_t)t * K + lane) : 0.f;
              }
            }
          }
          k += nslots;
        }
      }
      if (lane == 0) bulk_wait<0>();
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
  size_t nslots = (220 << 10) / slot;
  if (nslots > kRingMaxSlots) nslots = kRingMaxSlots;
  if (nslots < 2) return cudaErrorInvalidValue;
  const size_t smem = 1024 + nslots * slot;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(ep_combine_ht_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    configured = smem;
  }
  dim3 grid(p.send_blocks + p.recv_blocks, nranks), block(kCombineThreads);
  void* args[] = {const_cast<CombineParams*>(&p)};
  return cudaLaunchCooperativeKernel((const void*)ep_combine_ht_kernel, grid, block, args, smem, stream);
}

}  // namespace dep
