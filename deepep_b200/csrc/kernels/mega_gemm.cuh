// Grouped block-scaled GEMM phase on the 5th-generation tensor cores (tcgen05 + tensor memory):
//   C[rows of expert e, n] = sum_k A[row, k] * B[e][n, k]
// A: e4m3 activations with one ue8m0 scale per 32 values of K; B: e2m1 weights (two per byte in
// global memory, widened to one byte per value by the copy engine) or e4m3 weights, with ue8m0
// scales per 32.
//
// `gemm_phase` is run by a whole CTA of kGemmThreads threads, one CTA per SM, warp-specialised:
//   warp 0     one lane issues the TMA tile loads (A, B) and bulk loads (scale chunks) of a stage
//   warp 1     allocates tensor memory; one lane copies the scales smem -> TMEM (tcgen05.cp) and
//              issues four tcgen05.mma (M=128, N=256, K=32) per stage; tcgen05.commit frees the stage
//   warps 2-9  epilogue (two warps per TMEM lane quadrant, each takes half of the columns):
//              tcgen05.ld of the fp32 accumulator (one tile row per thread), then
//              store fp32 | SwiGLU + MXFP8 requantisation | bf16 rows pushed into the source
//              rank's combine slots over NVLink.
// It walks one tile list that may hold two GEMMs back to back (GEMM1 tiles, then GEMM2 tiles whose
// A operand is GEMM1's output): a GEMM2 tile waits on a per-row-block counter that the GEMM1
// epilogues bump, so SMs that run out of GEMM1 tiles start on GEMM2 at once.  In the fused layer the
// tiles are handed out by an atomic counter (the producer warp takes the next tile and publishes its
// id to the MMA and epilogue warps through a ring of mbarriers), which balances the long GEMM1 tiles
// and the short GEMM2 tiles over the SMs; the stand-alone launch keeps the static round-robin.
//
// Tile shape: issuing one tcgen05 instruction costs the MMA thread about 50 cycles (measured), so a
// stage of four N=128 MMAs (256 tensor cycles) was issue-bound; N=256 doubles the work per instruction.
// A 128 x 256 fp32 accumulator takes 256 of the 512 TMEM columns and the scales need more, so there is
// one accumulator: the next tile's loads are prefetched during the epilogue, its MMAs start once the
// epilogue warps have drained the accumulator.  Both fused epilogues therefore park the bf16-rounded
// accumulator in shared memory first, hand tensor memory back, and only then do their arithmetic and
// their stores.  The stage time (about 0.6 us for 48 KB) is set by the rate at which shared memory
// is filled from L2, not by the tensor pipe (0.27 us).
// All waits are bounded; a wait that runs out sets an error flag, the CTA stops issuing work,
// frees its tensor memory and returns.
//
// Parity: the cube-core GMM1/GMM2 stages and their vector-core epilogues of the reference's MegaMoE
// (experiments/megamoe/csrc/kernels/mega_moe/mega_moe_wave_a8w4.hpp, catlass_gmm/block_mmad_a8w4.hpp,
// epilogue/block_epilogue_activation_mx_quant.hpp, stage/gmm2_combine.hpp).
#pragma once
#include "mega_api.h"
#include "umma.cuh"

namespace dep {

constexpr int kGemmThreads = 320;                    // TMA warp, MMA warp, 8 epilogue warps
constexpr int kEpiWarps = 8;
constexpr int kGemmMaxStages = kGemmMaxStagesHost;
constexpr int kTileABytes = kGemmBM * kGemmBK;       // 16 KB
constexpr int kTileBBytes = kGemmBN * kGemmBK;       // 32 KB in shared memory (one byte per value)
constexpr int kStageBytes = kTileABytes + kTileBBytes;
constexpr int kSfStageBytes = (1 + kGemmBN / 128) * kSfChunk;   // A scales + B scales of one stage
constexpr int kEpiWarpCols = kGemmBN / 2;            // columns handled by one epilogue warp
constexpr int kEpiStageBytes = kEpiWarps * 32 * kEpiWarpCols * 2;   // bf16 staging: each warp parks its 32 x 128 block
constexpr int kTmemCols = 512;
constexpr int kSfColBase = kGemmBN;                  // scale columns start after the accumulator
constexpr int kSfColsPerStage = 4 + 4 * (kGemmBN / 128);

__host__ __device__ constexpr size_t gemm_smem_bytes(int stages, bool staging) {
  return 1024 + (size_t)stages * (kStageBytes + kSfStageBytes) + (staging ? kEpiStageBytes : 0) + 256;
}

// The MMA thread releases pipeline stages in groups of `commit_every` (one tcgen05.commit per group); a stage is
// reloaded once the commit of its group has arrived, so with groups of two the pipeline must be deep enough that a
// whole group can be in flight while two others are consumed.
constexpr int kGroupRing = 8;   // group barriers in rotation; more than the groups a producer can be ahead of the MMAs
constexpr int kSchedRing = 8;   // tile ids in flight between the producer and the slowest consumer (< stages + 2)

struct GemmBarriers {
  uint64_t full[kGemmMaxStages], acc_full, acc_empty, epi_done;
  uint64_t peer_acc_empty;         // CTA pairs: the odd CTA's acc_empty, forwarded to the even CTA
  uint64_t released[kGroupRing];   // the MMAs of a group of kCommitEvery stages have completed
  uint64_t sched[kSchedRing];      // the producer has published tile_id[slot]
  int tile_id[kSchedRing];
  uint32_t tmem_base;
  int failed;
};

#ifdef __CUDACC__
__device__ __forceinline__ bool try_wait_now(uint64_t* bar, uint32_t parity) {   // no suspend hint: pipeline waits are short
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool try_wait_cluster(uint64_t* bar, uint32_t parity) {   // acquires what the peer CTA released
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Which wait ran out: the value a CTA leaves in its failure word (any nonzero value stops the CTA's other warps) and,
// through the kernel's error flag, what the host reports.
enum GemmWaitSite : int {
  kWaitAny = 1, kWaitTileTicket = 2, kWaitRowBlockDone = 3, kWaitRowsPulled = 4, kWaitGroupReleased = 5, kWaitAccEmpty = 6,
  kWaitPeerAccEmpty = 7, kWaitStageFull = 8, kWaitAccFull = 9, kWaitEpilogueDone = 10
};
__device__ __forceinline__ bool bounded_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* failed, int site = kWaitAny) {
  for (unsigned i = 0; i < (1u << 24); ++i) {
    if (try_wait_cluster(bar, parity)) return true;
    if ((i & 63u) == 63u && *failed) return false;
  }
  *failed = site;
  return false;
}
__device__ __forceinline__ bool bounded_wait(uint64_t* bar, uint32_t parity, volatile int* failed, int site = kWaitAny) {
  for (unsigned i = 0; i < (1u << 24); ++i) {
    if (try_wait_now(bar, parity)) return true;
    if ((i & 63u) == 63u && *failed) return false;
  }
  *failed = site;
  return false;
}
// Producer-side wait for "all `need` GEMM1 tiles of this row block have been written".
__device__ __forceinline__ bool wait_rows_ready(const int* counter, int need, volatile int* failed, int site = kWaitAny) {
  for (unsigned i = 0; i < (1u << 26); ++i) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
    if (v >= need) return true;
    if ((i & 63u) == 63u) { if (*failed) return false; __nanosleep(100); }
  }
  *failed = site;
  return false;
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// Position in the fused schedule -> tile id (ids below num_mtiles * n1 are GEMM1 tiles, the rest GEMM2 tiles).
// The schedule interleaves the two GEMMs in waves of `wave` row blocks: GEMM1 of wave 0, then for every later wave its
// GEMM1 tiles followed by the GEMM2 tiles of the wave before, and the last wave's GEMM2 tiles at the end.  GEMM2's
// rows leave for the source ranks over NVLink from early on instead of only after the last GEMM1 tile, and its A rows
// are still in L2.  A GEMM2 tile still comes after all GEMM1 tiles of its row block, so its wait always ends.
__device__ __forceinline__ int schedule_to_tile(int pos, int num_mtiles, int n1, int n2, int wave) {
  const int waves = (num_mtiles + wave - 1) / wave;
  for (int w = 0; w <= waves; ++w) {
    if (w < waves) {
      const int c1 = min(wave, num_mtiles - w * wave) * n1;
      if (pos < c1) return w * wave * n1 + pos;
      pos -= c1;
    }
    if (w >= 1) {
      const int c2 = min(wave, num_mtiles - (w - 1) * wave) * n2;
      if (pos < c2) return num_mtiles * n1 + (w - 1) * wave * n2 + pos;
      pos -= c2;
    }
  }
  return -1;
}

// Next tile of this CTA: the producer publishes it to the MMA and epilogue warps through a small ring.
__device__ __forceinline__ int fetch_tile(GemmBarriers* bars, uint32_t local_tile, volatile int* failed, bool from_peer = false) {
  const uint32_t slot = local_tile % kSchedRing;
  const bool ok = from_peer ? bounded_wait_cluster(&bars->sched[slot], (local_tile / kSchedRing) & 1u, failed, kWaitTileTicket)
                            : bounded_wait(&bars->sched[slot], (local_tile / kSchedRing) & 1u, failed, kWaitTileTicket);
  return ok ? *reinterpret_cast<volatile int*>(&bars->tile_id[slot]) : -1;
}

// g1: first GEMM of the list; g2: optional second GEMM (nullptr for a single GEMM).  `ready` (may be null):
// ready[mt] counts finished g1 tiles of row block mt; g2 tiles of mt wait until it reaches g1.n_tiles.
// `tile_counter` (may be null): tiles are handed out in list order by an atomic counter, whichever CTA is free takes
// the next one (it must be zero when the first CTA arrives); null: CTA c takes tiles c, c + num_ctas, ...
// Either way a tile is only ever taken after all tiles before it, so a GEMM2 tile's wait for its GEMM1 tiles ends.
// `smem_raw` must provide gemm_smem_bytes(stages, staging) bytes.
//
// kPair: the CTAs of a cluster of two work on one 256-row tile pair (row blocks 2j and 2j + 1, which the routing layout
// gives to the same expert).  Each CTA loads its own 128 rows of A and HALF of the 256 weight rows of B; the even CTA
// issues tcgen05.mma.cta_group::2 (M = 256), which reads both halves of B from the two CTAs' shared memory, so a stage
// fills 32 KB per CTA instead of 48 KB for the same tensor work.  Both CTAs' loads count their bytes on the even CTA's
// "stage full" barrier; the odd CTA's MMA warp forwards its "accumulator drained" barrier; the even CTA's commits arrive
// on both CTAs' barriers.  `cta` / `num_ctas` count pairs then, `stages` may be 4, and all threads of both CTAs must
// make this call (cluster barriers).
template <bool kPair>
__device__ __forceinline__ void gemm_phase(const MegaGemmParams& g1, const MegaGemmParams* g2, int* ready, uint8_t* smem_raw,
                                           int stages, int cta, int num_ctas, int* tile_counter = nullptr, int interleave = 0,
                                           int commit_every = 1, unsigned long long* mma_stats = nullptr) {
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);       // tiles need 1024-byte alignment
  uint8_t* tiles = smem;
  constexpr int kBBoxes = kPair ? 1 : kGemmBN / 128;                  // 128-row boxes of B this CTA loads per stage
  constexpr int kStage = kTileABytes + kBBoxes * 128 * kGemmBK;       // bytes of A and B per stage in this CTA
  const uint32_t crank = kPair ? umma::cluster_ctarank() : 0u;        // 0: issues the MMAs
  uint8_t* sf_smem = tiles + (size_t)stages * kStage;
  uint8_t* epi_smem = sf_smem + (size_t)stages * kSfStageBytes;
  const bool staging = g1.epi == kEpiCombine || (g2 && g2->epi == kEpiCombine);
  GemmBarriers* bars = reinterpret_cast<GemmBarriers*>(epi_smem + (staging ? kEpiStageBytes : 0));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kGemmMaxStages; ++s) mbar_init(&bars->full[s], 1);
    mbar_init(&bars->acc_full, 1);
    mbar_init(&bars->acc_empty, kEpiWarps);
    mbar_init(&bars->epi_done, kEpiWarps);
    for (int i = 0; i < kSchedRing; ++i) mbar_init(&bars->sched[i], 1);
    mbar_init(&bars->peer_acc_empty, 1);
    for (int i = 0; i < kGroupRing; ++i) mbar_init(&bars->released[i], 1);
    bars->failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    umma::prefetch_tensormap(&g1.tmap_a);
    umma::prefetch_tensormap(&g1.tmap_b);
    if (g2) { umma::prefetch_tensormap(&g2->tmap_a); umma::prefetch_tensormap(&g2->tmap_b); }
  }
  if constexpr (kPair) {      // the peer's barriers exist before anything arrives on them, and both CTAs allocate together
    __syncthreads();
    umma::cluster_sync_all();
  }
  if (warp == 1) {
    if constexpr (kPair) { umma::tmem_alloc_pair(&bars->tmem_base, kTmemCols); umma::tmem_relinquish_pair(); }
    else { umma::tmem_alloc(&bars->tmem_base, kTmemCols); umma::tmem_relinquish(); }
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = bars->tmem_base;
  volatile int* failed = &bars->failed;

  // row blocks in the tile list: 128-row tiles, or pairs of them (the routing layout keeps a pair inside one expert)
  const int num_mtiles = kPair ? (min(*g1.num_mtiles, g1.max_mtiles) + 1) / 2 : min(*g1.num_mtiles, g1.max_mtiles);
  const int tiles1 = num_mtiles * g1.n_tiles;
  const int total_tiles = tiles1 + (g2 ? num_mtiles * g2->n_tiles : 0);

  if (warp == 0) {
    // ============================================================ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      // The ticket of the NEXT tile is taken while the current tile is being loaded, so the round trip of the atomic is
      // off the path between two tiles.  A CTA still works through its tickets in increasing order, which is all the
      // argument for the end of every GEMM2 wait needs.
      const bool takes_tickets = tile_counter != nullptr && !(kPair && crank != 0);
      int ticket = takes_tickets ? atomicAdd(tile_counter, 1) : 0;
      for (uint32_t local_tile = 0;; ++local_tile) {
        int tile;
        if (kPair && crank != 0) {
          tile = fetch_tile(bars, local_tile, failed, true);      // the even CTA hands out the pair's tiles
        } else {
          tile = takes_tickets ? ticket : cta + (int)local_tile * num_ctas;
          if (takes_tickets && tile < total_tiles) ticket = atomicAdd(tile_counter, 1);
          if (tile >= total_tiles || *failed) tile = -1;
          else if (g2 && ready && interleave > 0)   // wave = row blocks whose GEMM1 tiles fill `2 * interleave` rounds of the CTAs
            tile = schedule_to_tile(tile, num_mtiles, g1.n_tiles, g2->n_tiles, (2 * interleave * num_ctas + g1.n_tiles - 1) / g1.n_tiles);
          const uint32_t slot = local_tile % kSchedRing;
          bars->tile_id[slot] = tile;
          mbar_arrive(&bars->sched[slot]);      // release: the id is visible to whoever passes the wait
          if constexpr (kPair) {
            umma::remote_store_u32(umma::map_to_cta(smem_u32(&bars->tile_id[slot]), 1), (uint32_t)tile);
            umma::remote_arrive(umma::map_to_cta(smem_u32(&bars->sched[slot]), 1));
          }
        }
        if (tile < 0) break;
        const bool second = tile >= tiles1;
        const MegaGemmParams& p = second ? *g2 : g1;
        const int local = second ? tile - tiles1 : tile;
        const int mt = kPair ? 2 * (local / p.n_tiles) + (int)crank : local / p.n_tiles, nb = local % p.n_tiles;
        const int brow = p.mtile_expert[mt] * p.n_total + nb * kGemmBN;        // first of the tile's 256 weight rows
        if (second && ready) {
          if (!wait_rows_ready(ready + mt, g1.n_tiles, failed, kWaitRowBlockDone)) break;
          fence_proxy_async();          // rows written by other SMs' stores are about to be read by the copy engine
        } else if (!second && p.a_ready) {
          if (!wait_rows_ready(p.a_ready + mt, kGemmBM, failed, kWaitRowsPulled)) break;
          fence_proxy_async();
        }
        for (int ks = 0; ks < p.k_steps; ++ks, ++it) {
          const int s = it % stages;
          if (it >= (uint32_t)stages) {     // the stage's previous contents have been consumed: their group was released
            const uint32_t grp = (it - (uint32_t)stages) / (uint32_t)commit_every;
            if (!bounded_wait(&bars->released[grp % kGroupRing], (grp / kGroupRing) & 1u, failed, kWaitGroupReleased)) break;
          }
          uint8_t* a_dst = tiles + (size_t)s * kStage;
          uint8_t* sf_dst = sf_smem + (size_t)s * kSfStageBytes;
          if constexpr (kPair) {
            // both CTAs' bytes are counted on the even CTA's barrier, which the MMA thread waits on
            const uint32_t bar = umma::map_to_cta(smem_u32(&bars->full[s]), 0);
            if (crank == 0) mbar_expect_tx(&bars->full[s], 2 * (kTileABytes + p.b_tx_bytes + kSfStageBytes));
            umma::tma_load_2d_pair(a_dst, &p.tmap_a, ks * kGemmBK, mt * kGemmBM, bar);
            umma::tma_load_2d_pair(sf_dst, &p.tmap_sfa, 0, mt * p.k_steps + ks, bar);
            // this CTA's half of the 256 weight rows, and the scales of all of them (each CTA of a pair needs them all)
            umma::tma_load_2d_pair(a_dst + kTileABytes, &p.tmap_b, 0, ((brow / 128 + (int)crank) * p.k_steps + ks) * 128, bar);
#pragma unroll
            for (int h = 0; h < kGemmBN / 128; ++h)
              umma::tma_load_2d_pair(sf_dst + (1 + h) * kSfChunk, &p.tmap_sfb, 0, (brow / 128 + h) * p.k_steps + ks, bar);
          } else {
            mbar_expect_tx(&bars->full[s], kTileABytes + kBBoxes * p.b_tx_bytes + kSfStageBytes);
            umma::tma_load_2d(a_dst, &p.tmap_a, ks * kGemmBK, mt * kGemmBM, &bars->full[s]);
            bulk_g2s(sf_dst, p.sfa + ((size_t)mt * p.k_steps + ks) * kSfChunk, kSfChunk, &bars->full[s]);
#pragma unroll
            for (int h = 0; h < kGemmBN / 128; ++h) {     // 128 weight rows per box; consecutive boxes continue the same swizzled tile
              umma::tma_load_2d(a_dst + kTileABytes + h * 128 * kGemmBK, &p.tmap_b, 0, ((brow / 128 + h) * p.k_steps + ks) * 128,
                                &bars->full[s]);
              bulk_g2s(sf_dst + (1 + h) * kSfChunk, p.sfb + ((size_t)(brow / 128 + h) * p.k_steps + ks) * kSfChunk, kSfChunk, &bars->full[s]);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ============================================================ MMA issuer
    if (lane == 0 && crank == 0) {
      // A is e4m3 (format 0); B is e2m1 (5) or e4m3 (0), per GEMM.  A pair issues M = 256: 128 rows in each CTA.
      constexpr int kInstrM = kPair ? 2 * kGemmBM : kGemmBM;
      const uint32_t idesc1 = umma::instr_desc_mxf8f6f4(kInstrM, kGemmBN, 0, g1.b_fp8 ? 0 : 5);
      const uint32_t idesc2 = g2 ? umma::instr_desc_mxf8f6f4(kInstrM, kGemmBN, 0, g2->b_fp8 ? 0 : 5) : idesc1;
      // commits of a pair arrive on the barrier of both CTAs
      auto commit_both = [&](uint64_t* bar) {
        if constexpr (kPair) {
          umma::commit_pair(smem_u32(bar));
          umma::commit_pair(umma::map_to_cta(smem_u32(bar), 1));
        } else {
          umma::commit(bar);
        }
      };
      uint32_t it = 0;
      long long waited = 0;                      // cycles spent waiting for operands (only counted when asked for)
      const long long loop_start = mma_stats ? clock64() : 0;
      for (uint32_t local_tile = 0;; ++local_tile) {
        const int tile = fetch_tile(bars, local_tile, failed);
        if (tile < 0) break;
        const int k_steps = tile >= tiles1 ? g2->k_steps : g1.k_steps;
        const uint32_t idesc = tile >= tiles1 ? idesc2 : idesc1;
        if (!bounded_wait(&bars->acc_empty, (local_tile & 1u) ^ 1u, failed, kWaitAccEmpty)) break;
        if constexpr (kPair)      // the odd CTA forwards one arrival per tile, the first as soon as it starts
          if (!bounded_wait_cluster(&bars->peer_acc_empty, local_tile & 1u, failed, kWaitPeerAccEmpty)) break;
        umma::fence_after_sync();
        for (int ks = 0; ks < k_steps; ++ks, ++it) {
          const int s = it % stages;
          const long long w0 = mma_stats ? clock64() : 0;
          if (!bounded_wait(&bars->full[s], (it / stages) & 1u, failed, kWaitStageFull)) break;
          if (mma_stats) waited += clock64() - w0;
          umma::fence_after_sync();
          const uint32_t a_addr = smem_u32(tiles + (size_t)s * kStage);
          const uint32_t sf_addr = smem_u32(sf_smem + (size_t)s * kSfStageBytes);
          const uint32_t tsfa = tmem + kSfColBase + s * kSfColsPerStage, tsfb = tsfa + 4;
          if constexpr (kPair) {
            umma::copy_sf_to_tmem_pair(tsfa, umma::smem_desc_sf(sf_addr));
#pragma unroll
            for (int h = 0; h < kGemmBN / 128; ++h)
              umma::copy_sf_to_tmem_pair(tsfb + 4 * h, umma::smem_desc_sf(sf_addr + (1 + h) * kSfChunk));
          } else {
            umma::copy_sf_to_tmem(tsfa, umma::smem_desc_sf(sf_addr));
#pragma unroll
            for (int h = 0; h < kGemmBN / 128; ++h)
              umma::copy_sf_to_tmem(tsfb + 4 * h, umma::smem_desc_sf(sf_addr + (1 + h) * kSfChunk));
          }
          const uint64_t da = umma::smem_desc_sw128(a_addr), db = umma::smem_desc_sw128(a_addr + kTileABytes);
#pragma unroll
          for (int k = 0; k < 4; ++k) {   // 32 K-values = 32 bytes = 2 descriptor units per step inside the swizzle row
            if constexpr (kPair)
              umma::mma_block_scaled_pair(tmem, da + 2 * k, db + 2 * k, umma::with_sf_ids(idesc, k, k), tsfa, tsfb, ks > 0 || k > 0);
            else
              umma::mma_block_scaled(tmem, da + 2 * k, db + 2 * k, umma::with_sf_ids(idesc, k, k), tsfa, tsfb, ks > 0 || k > 0);
          }
          if (it % (uint32_t)commit_every == (uint32_t)commit_every - 1)      // stages (tiles, scale columns) reusable once these MMAs finished
            commit_both(&bars->released[(it / (uint32_t)commit_every) % kGroupRing]);
        }
        commit_both(&bars->acc_full);              // accumulator complete
      }
      if (mma_stats)
        *mma_stats = ((unsigned long long)(waited >> 4) << 32) | (unsigned long long)(((clock64() - loop_start) >> 4) & 0xffffffffll);
    } else if (kPair && lane == 0) {
      // ---- odd CTA of a pair: no MMAs to issue; forward "accumulator drained" to the even CTA, once per tile
      const uint32_t acc_fwd = umma::map_to_cta(smem_u32(&bars->peer_acc_empty), 0);
      for (uint32_t local_tile = 0;; ++local_tile) {
        const int tile = fetch_tile(bars, local_tile, failed, true);
        if (tile < 0) break;
        if (!bounded_wait(&bars->acc_empty, (local_tile & 1u) ^ 1u, failed, kWaitAccEmpty)) break;
        umma::remote_arrive(acc_fwd);
      }
    }
  } else {
    // ============================================================ epilogue (warps 2..9)
    const int quad = warp & 3;                       // TMEM lanes [32 * quad, 32 * quad + 32)
    const int part = (warp - 2) >> 2;                // which half of the tile's columns this warp handles
    const int row_in_tile = quad * 32 + lane;
    uint8_t* stage = epi_smem + (size_t)(warp - 2) * 32 * kEpiWarpCols * 2;
    uint32_t first_done = 0;
    for (uint32_t local_tile = 0;; ++local_tile) {
      const int tile = fetch_tile(bars, local_tile, failed, kPair && crank != 0);
      if (tile < 0) break;
      const bool second = tile >= tiles1;
      const MegaGemmParams& p = second ? *g2 : g1;
      const int local = second ? tile - tiles1 : tile;
      const int mt = kPair ? 2 * (local / p.n_tiles) + (int)crank : local / p.n_tiles, nb = local % p.n_tiles;
      if (!bounded_wait(&bars->acc_full, local_tile & 1u, failed, kWaitAccFull)) break;
      umma::fence_after_sync();
      const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16);
      const long long row = (long long)mt * kGemmBM + row_in_tile;
      uint32_t v[32], u[32];
      if (p.epi == kEpiCombine) {
        // bf16 rows go to the source rank's combine slots.
        // 1) drain this warp's 32 x 128 block into shared memory as bf16 and hand the accumulator back at once
        const int code = p.row_src[row];
        uint8_t* dst_row = nullptr;
        if (code >= 0) {
          const int src = code / (p.max_tokens * p.topk), rem = code - src * p.max_tokens * p.topk;
          dst_row = p.ws[src] + p.comb_off + ((size_t)rem * p.hidden + (size_t)nb * kGemmBN) * 2;
        }
        uint4* mine = reinterpret_cast<uint4*>(stage + (size_t)lane * kEpiWarpCols * 2);   // 256 B per row = 16 pieces
        __syncwarp();                                     // the previous tile's block has been written out
        for (int c = 0; c < kEpiWarpCols; c += 32) {
          umma::tmem_ld32(taddr + part * kEpiWarpCols + c, v);
          umma::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t w0[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              __nv_bfloat162 b0 = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 2 * j]), __uint_as_float(v[8 * i + 2 * j + 1]));
              w0[j] = *reinterpret_cast<uint32_t*>(&b0);
            }
            mine[(c / 8 + i) ^ (lane & 15)] = make_uint4(w0[0], w0[1], w0[2], w0[3]);   // XOR swizzle against bank conflicts
          }
        }
        umma::fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->acc_empty);
        // 2) write the block out: 16 lanes x 16 B cover one row's 256-byte segment, 2 rows per instruction
#pragma unroll 4
        for (int r0 = 0; r0 < 32; r0 += 2) {
          const int rr = r0 + (lane >> 4), piece = lane & 15;
          uint8_t* drow = reinterpret_cast<uint8_t*>(__shfl_sync(0xffffffffu, (unsigned long long)dst_row, rr));
          const uint4 val = reinterpret_cast<const uint4*>(stage + (size_t)rr * kEpiWarpCols * 2)[piece ^ (rr & 15)];
          if (drow) reinterpret_cast<uint4*>(drow + (size_t)part * kEpiWarpCols * 2)[piece] = val;
        }
        continue;   // the accumulator was already released
      }
      if (p.epi == kEpiStoreF32) {
        for (int c = part * (kGemmBN / 2); c < (part + 1) * (kGemmBN / 2); c += 32) {
          umma::tmem_ld32(taddr + c, v);
          umma::tmem_ld_wait();
          float4* dst = reinterpret_cast<float4*>(p.c + row * p.ldc + nb * kGemmBN + c);
#pragma unroll
          for (int i = 0; i < 8; ++i) dst[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                                             __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
        }
      } else {
        // SwiGLU + requantisation: columns [0, 128) are gate rows of W1, [128, 256) the matching up rows.
        // With a staging area the bf16-rounded accumulator (the first step of the math anyway) is parked in shared
        // memory and tensor memory is handed back before the arithmetic, so the next tile's MMAs overlap it.
        uint4* mine = reinterpret_cast<uint4*>(stage + (size_t)lane * kEpiWarpCols * 2);   // 256 B per row = 16 pieces
        if (staging) {
          __syncwarp();
#pragma unroll
          for (int hh = 0; hh < kGemmBN / 128; ++hh) {
            const int half = part * (kGemmBN / 128) + hh;
            umma::tmem_ld32(taddr + half * 32, v);
            umma::tmem_ld32(taddr + kGemmBN / 2 + half * 32, u);
            umma::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint32_t wg[4], wu[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 bg = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 2 * j]), __uint_as_float(v[8 * i + 2 * j + 1]));
                __nv_bfloat162 bu = __floats2bfloat162_rn(__uint_as_float(u[8 * i + 2 * j]), __uint_as_float(u[8 * i + 2 * j + 1]));
                wg[j] = *reinterpret_cast<uint32_t*>(&bg);
                wu[j] = *reinterpret_cast<uint32_t*>(&bu);
              }
              mine[(hh * 8 + i) ^ (lane & 15)] = make_uint4(wg[0], wg[1], wg[2], wg[3]);
              mine[(hh * 8 + 4 + i) ^ (lane & 15)] = make_uint4(wu[0], wu[1], wu[2], wu[3]);
            }
          }
          umma::fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->acc_empty);
        }
        for (int half = part * (kGemmBN / 128); half < (part + 1) * (kGemmBN / 128); ++half) {
          float gv[32], uv[32];
          if (staging) {
            const int hh = half - part * (kGemmBN / 128);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint4 pg = mine[(hh * 8 + i) ^ (lane & 15)], pu = mine[(hh * 8 + 4 + i) ^ (lane & 15)];
              const __nv_bfloat162* bg = reinterpret_cast<const __nv_bfloat162*>(&pg);
              const __nv_bfloat162* bu = reinterpret_cast<const __nv_bfloat162*>(&pu);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                gv[8 * i + 2 * j] = __low2float(bg[j]); gv[8 * i + 2 * j + 1] = __high2float(bg[j]);
                uv[8 * i + 2 * j] = __low2float(bu[j]); uv[8 * i + 2 * j + 1] = __high2float(bu[j]);
              }
            }
          } else {
            umma::tmem_ld32(taddr + half * 32, v);
            umma::tmem_ld32(taddr + kGemmBN / 2 + half * 32, u);
            umma::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) { gv[i] = bf16_round(__uint_as_float(v[i])); uv[i] = bf16_round(__uint_as_float(u[i])); }
          }
          float h[32], amax = 0.f;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float g = gv[i], up = uv[i];
            // div.approx: the IEEE division has a slow path for huge / non-finite operands, which padding rows (whatever
            // the row buffer held) do contain; it made this epilogue, and with it the whole tile, measurably slower
            const float act = __fdividef(g, 1.0f + __expf(fminf(fmaxf(-g, -80.f), 80.f))) * up;
            h[i] = bf16_round(act);
            amax = fmaxf(amax, fabsf(h[i]));
          }
          // MX scale: 2^(floor(log2(amax)) - 8), at least 2^-127; values saturate at 448
          int e = (int)((__float_as_uint(fmaxf(amax, 1.1754944e-38f)) >> 23) & 0xff) - 127 - 8;
          e = max(e, -127);
          const float inv = __uint_as_float((uint32_t)(127 - e) << 23);   // 2^-e, exact (e in [-127, 120])
          uint32_t q[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            q[i] = (uint32_t)__nv_cvt_float_to_fp8(h[4 * i] * inv, __NV_SATFINITE, __NV_E4M3) |
                   ((uint32_t)__nv_cvt_float_to_fp8(h[4 * i + 1] * inv, __NV_SATFINITE, __NV_E4M3) << 8) |
                   ((uint32_t)__nv_cvt_float_to_fp8(h[4 * i + 2] * inv, __NV_SATFINITE, __NV_E4M3) << 16) |
                   ((uint32_t)__nv_cvt_float_to_fp8(h[4 * i + 3] * inv, __NV_SATFINITE, __NV_E4M3) << 24);
          }
          const long long col = (long long)nb * (kGemmBN / 2) + half * 32;
          uint4* dst = reinterpret_cast<uint4*>(p.a2 + row * p.inter + col);
          dst[0] = make_uint4(q[0], q[1], q[2], q[3]);
          dst[1] = make_uint4(q[4], q[5], q[6], q[7]);
          p.a2_sf[sf_offset(row, col, p.inter)] = (uint8_t)(e + 127);
        }
      }
      if (!(p.epi == kEpiSwigluQuant && staging)) {      // (that path released the accumulator before its arithmetic)
        umma::fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->acc_empty);
      }
      if (!second && g2 && ready) {
        // this tile's rows of the intermediate activations are in global memory: let GEMM2 producers know
        fence_proxy_async();
        __threadfence();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->epi_done);
        if (warp == 2 && lane == 0 && bounded_wait(&bars->epi_done, first_done & 1u, failed, kWaitEpilogueDone)) {
          __threadfence();
          atomicAdd(ready + mt, 1);
        }
        ++first_done;
      }
    }
    __threadfence_system();       // rows pushed to peers are visible before the kernel (or its next phase) signals them
  }

  umma::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *failed && g1.error_flag) *g1.error_flag = *failed;   // which wait ran out (GemmWaitSite)
  if constexpr (kPair) umma::cluster_sync_all();    // both CTAs are done with each other's shared and tensor memory
  if (warp == 1) {
    umma::fence_after_sync();
    if constexpr (kPair) umma::tmem_dealloc_pair(tmem, kTmemCols);
    else umma::tmem_dealloc(tmem, kTmemCols);
  }
}
#endif  // __CUDACC__

}  // namespace dep
