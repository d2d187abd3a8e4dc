// All-to-all-v fused with a bf16 grouped GEMM on tcgen05 / tensor memory, one persistent cooperative kernel per op.
//
//   a2av_gmm_kernel   x (sorted by global expert) is staged in this rank's symmetric workspace; every expert rank
//                     reads the peers' per-expert row tables, lays its rows out as (local expert, source rank) segments
//                     and two warps per CTA pull them over NVLink tile by tile while the other warps run the grouped
//                     GEMM; a tile's loads start as soon as its rows have arrived (per-tile counters).
//   gmm_a2av_kernel   grouped GEMM over the rows this rank holds; the epilogue stores each bf16 output row straight
//                     into the workspace of the rank the row came from, at its place in that rank's expert-sorted
//                     order; after a flag handshake every rank copies its returned rows into the output tensor.
//
// GEMM: 256 x 256 tiles, K in steps of 64, A K-major and B (weights [K, N], N contiguous) MN-major, both moved by
// TMA with the 128-byte swizzle; per stage two groups of four tcgen05.mma kind::f16 (M = 128, N = 256, K = 16), one
// group per 128-row half of the tile, each half with its own fp32 accumulator in tensor memory (2 x 256 columns).
// The two halves share every B stage: the kernel is bound by the rate at which one SM's shared memory is filled
// from L2 (measured about 100 KB/us), and the shared B cuts the bytes per FLOP by a third against 128-row tiles.
// Expert row blocks are not padded: a tile that reaches past its expert's rows computes rows that the epilogue drops.
// Every wait is bounded; a wait that runs out sets the error flag, the CTA stops issuing work, frees its tensor
// memory and returns.
//
// Parity: experiments/ep_gmm_fused/csrc/all_to_allv_grouped_mat_mul_udma/ascend950/*.cpp and
// grouped_mat_mul_all_to_allv_udma/ascend950/*.cpp of the reference (peer-serial all-to-all-v schedulers and
// remote-copy tiles around a grouped matmul).
#include <cooperative_groups.h>

#include "gmm_api.h"
#include "mega_gemm.cuh"   // bounded_wait, wait_rows_ready
#include "umma.cuh"

namespace cg = cooperative_groups;

namespace dep {

constexpr int kGmmGemmThreads = 320;                     // TMA warp, MMA warp, 8 epilogue warps
constexpr int kGmmPullWarps = 2;
constexpr int kGmmMaxStages = 4;
constexpr int kGmmTileA = kGmmBM * kGmmBK * 2;           // 16 KB
constexpr int kGmmBoxB = 64 * kGmmBK * 2;                // 8 KB: 64 K-rows of 64 N-values
constexpr int kGmmTileB = (kGmmBN / 64) * kGmmBoxB;      // 32 KB
constexpr int kGmmPullChunk = 8;
// Tiles are 256 rows x 256 columns: both 128-lane accumulators (all 512 tensor-memory columns) belong to one tile,
// the two row halves share every B stage, and a stage moves 64 KB for twice the work (the kernel is bound by the
// rate at which shared memory can be filled from L2, about 100 KB/us per SM, not by the tensor pipe).
__host__ __device__ constexpr int gmm_tile_rows(bool) { return 2 * kGmmBM; }
__host__ __device__ constexpr int gmm_stage_bytes(bool push) { return (gmm_tile_rows(push) / kGmmBM) * kGmmTileA + kGmmTileB; }
__host__ __device__ constexpr int gmm_stages(bool push) { return 3; }
__host__ __device__ constexpr size_t gmm_smem_bytes(bool push) {
  return 1024 + (size_t)gmm_stages(push) * gmm_stage_bytes(push) + 256;
}

struct GmmBarriers {
  uint64_t full[kGmmMaxStages], empty[kGmmMaxStages], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int failed;
};

struct GmmShared {
  int seg_src[kMaxExperts];        // [l * P + s] first row of the segment on its owner (staged x / returned output)
  int seg_dst[kMaxExperts + 1];    // [l * P + s] first row of the segment on this rank (exclusive prefix)
  int tile0[kMaxExperts + 1];      // [l] first tile of local expert l
  int alive, total_rows, num_tiles;
};

// Shared-memory descriptor of an MN-major operand: 64-value (128-byte) rows along N, 8 K-rows per 1024-byte swizzle
// atom; `lbo` = bytes between 64-value blocks along N, 1024 bytes between 8-row groups along K.
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// kind::f16 instruction descriptor: bf16 x bf16 -> fp32, A K-major, B MN-major.
__device__ __forceinline__ uint32_t instr_desc_bf16(int m, int n) {
  uint32_t d = 0;
  d |= 1u << 4;                       // D: fp32
  d |= 1u << 7;                       // A: bf16
  d |= 1u << 10;                      // B: bf16
  d |= 1u << 16;                      // B is MN-major
  d |= (uint32_t)(n >> 3) << 17;
  d |= (uint32_t)(m >> 4) << 24;
  return d;
}
__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
}

// ---------------------------------------------------------------- tables and layout
// Exclusive prefix of this rank's per-expert row counts into its table (one warp).
// table[0] = total rows, table[1] = `limit` (rows the owner's area really holds), table[4 + e] = first row of expert e.
__device__ __forceinline__ void publish_table(const GmmArgs& a, int* table, int limit, int lane) {
  int run = 0;
  for (int e0 = 0; e0 < a.E; e0 += 32) {
    const int e = e0 + lane;
    const int c = e < a.E ? max(a.counts[e], 0) : 0;
    int inc = c;
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, inc, d);
      if (lane >= d) inc += o;
    }
    if (e < a.E) table[4 + e] = run + inc - c;
    run += __shfl_sync(0xffffffffu, inc, 31);
  }
  if (lane == 0) { table[4 + a.E] = run; table[0] = run; table[1] = limit; }
}

// Segments (local expert, source rank) of this rank's gathered order, from every rank's table.  Run by all threads
// of every block (each block keeps its own copy in shared memory); block 0 also writes the tile list.
__device__ __forceinline__ void build_layout(const GmmArgs& a, GmmShared& sh, int alive, int gathered_cap, int tile_rows) {
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, me = ctx.rank, L = a.E / P;
  int bad = 0;
  for (int i = threadIdx.x; i < a.E; i += (int)blockDim.x) {
    const int l = i / P, s = i - l * P, e = me * L + l;
    const int* table = reinterpret_cast<const int*>(ctx.ws[s] + a.table_off);
    int first = 0, cnt = 0;
    if (alive) { first = __ldcg(table + 4 + e); cnt = __ldcg(table + 4 + e + 1) - first; }
    if (cnt < 0 || first < 0 || (alive && first + cnt > __ldcg(table + 1))) { bad = 1; cnt = 0; }   // the owner does not hold these rows
    sh.seg_src[i] = first;
    sh.seg_dst[i + 1] = cnt;
  }
  bad = __syncthreads_or(bad);
  if (threadIdx.x == 0) {
    int run = 0, tiles = 0;
    sh.seg_dst[0] = 0;
    for (int l = 0; l < L; ++l) {
      const int begin = run;
      for (int s = 0; s < P; ++s) { run += sh.seg_dst[l * P + s + 1]; sh.seg_dst[l * P + s + 1] = run; }
      sh.tile0[l] = tiles;
      tiles += (run - begin + tile_rows - 1) / tile_rows;
    }
    sh.tile0[L] = tiles;
    const bool fits = !bad && run <= gathered_cap && tiles <= a.max_tiles;
    if (!fits && a.error_flag) *a.error_flag = 2;
    sh.alive = alive && fits;
    sh.total_rows = sh.alive ? run : 0;
    sh.num_tiles = sh.alive ? tiles : 0;
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int l = threadIdx.x; l < L; l += (int)blockDim.x) {
      const int begin = sh.seg_dst[l * P], rows = sh.seg_dst[(l + 1) * P] - begin;
      for (int t = 0; sh.alive && t * tile_rows < rows; ++t)
        reinterpret_cast<int4*>(a.tile_info)[sh.tile0[l] + t] = make_int4(l, begin + t * tile_rows, min(tile_rows, rows - t * tile_rows), 0);
    }
    if (threadIdx.x == 0) { a.num_tiles[0] = sh.num_tiles; a.num_tiles[1] = sh.total_rows; }
  }
}

// Segment that holds gathered row r: the last i with seg_dst[i] <= r (empty segments share a start and are skipped).
__device__ __forceinline__ int find_segment(const GmmShared& sh, int n, int r) {
  int lo = 0, hi = n;            // invariant: seg_dst[lo] <= r < seg_dst[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (sh.seg_dst[mid] <= r) lo = mid; else hi = mid;
  }
  return lo;
}

// ---------------------------------------------------------------- the all-to-all-v pull (a2av_gmm)
__device__ __forceinline__ void pull_phase(const GmmArgs& a, const GmmShared& sh, int gw, int total_warps) {
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, lane = threadIdx.x & 31;
  const int units = a.K * 2 / 16;
  for (int row0 = gw * kGmmPullChunk; row0 < sh.total_rows; row0 += total_warps * kGmmPullChunk) {
    int src_rank = -1, src_row = 0, tile = 0;
    if (lane < kGmmPullChunk && row0 + lane < sh.total_rows) {
      const int r = row0 + lane, seg = find_segment(sh, a.E, r), l = seg / P;
      src_rank = seg - l * P;
      src_row = sh.seg_src[seg] + (r - sh.seg_dst[seg]);
      tile = sh.tile0[l] + (r - sh.seg_dst[l * P]) / gmm_tile_rows(false);
    }
#pragma unroll 1
    for (int c = 0; c < kGmmPullChunk; ++c) {
      const int s = __shfl_sync(0xffffffffu, src_rank, c);
      const int sr = __shfl_sync(0xffffffffu, src_row, c);
      if (s < 0) continue;
      const int4* from = reinterpret_cast<const int4*>(ctx.ws[s] + a.data_off + (size_t)sr * a.K * 2);
      int4* to = reinterpret_cast<int4*>(reinterpret_cast<uint8_t*>(a.gathered) + (size_t)(row0 + c) * a.K * 2);
      int4* one[1] = {to};
      warp_copy_row<14>(one, 1, from, units, lane);
    }
    __threadfence();
    __syncwarp();
    if (src_rank >= 0) atomicAdd(a.pulled + tile, 1);     // one arrival per row, lanes 0..7
  }
}

// ---------------------------------------------------------------- the grouped GEMM
// kPush = false: rows of the tile go to a.out on this rank.  kPush = true: each row goes to the rank it came from.
template <bool kPush>
__device__ __forceinline__ void gmm_phase(const GmmArgs& a, const GmmShared& sh, const int* a_ready, uint8_t* smem_raw,
                                          int cta, int num_ctas) {
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* tiles = smem_raw + (((raw + 1023u) & ~1023u) - raw);       // tiles need 1024-byte alignment
  constexpr int kGmmStages = gmm_stages(kPush);
  constexpr int kHalves = gmm_tile_rows(kPush) / kGmmBM;      // 128-row halves of a tile, one accumulator each
  constexpr int kGmmStageBytes = gmm_stage_bytes(kPush);
  constexpr int kOffB = kHalves * kGmmTileA;                  // B follows the A halves inside a stage
  uint8_t* epi_smem = tiles + (size_t)kGmmStages * kGmmStageBytes;
  GmmBarriers* bars = reinterpret_cast<GmmBarriers*>(epi_smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int P = a.ctx.world;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kGmmStages; ++s) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&bars->acc_full[b], 1); mbar_init(&bars->acc_empty[b], 8); }
    bars->failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    umma::prefetch_tensormap(&a.tmap_a);
    umma::prefetch_tensormap(&a.tmap_b);
  }
  if (warp == 1) {
    umma::tmem_alloc(&bars->tmem_base, 512);
    umma::tmem_relinquish();
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = bars->tmem_base;
  volatile int* failed = &bars->failed;
  const int n_tiles = (a.N + kGmmBN - 1) / kGmmBN, k_steps = a.K / kGmmBK;
  const int total_tiles = sh.num_tiles * n_tiles;
  const int4* tile_info = reinterpret_cast<const int4*>(a.tile_info);

  if (warp == 0) {
    // ============================================================ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = cta; tile < total_tiles && !*failed; tile += num_ctas) {
        const int mt = tile / n_tiles, nb = tile - mt * n_tiles;
        const int4 info = __ldcg(tile_info + mt);
        if (a_ready) {
          if (!wait_rows_ready(a_ready + mt, info.z, failed)) break;
          fence_proxy_async();            // rows written by this GPU's pull warps are about to be read by the copy engine
        }
        for (int ks = 0; ks < k_steps; ++ks, ++it) {
          const int s = it % kGmmStages;
          if (!bounded_wait(&bars->empty[s], ((it / kGmmStages) & 1u) ^ 1u, failed)) break;
          uint8_t* dst = tiles + (size_t)s * kGmmStageBytes;
          mbar_expect_tx(&bars->full[s], kGmmStageBytes);
#pragma unroll
          for (int m = 0; m < kHalves; ++m)       // rows past the end of the operand are filled with zeros
            umma::tma_load_2d(dst + m * kGmmTileA, &a.tmap_a, ks * kGmmBK, info.y + m * kGmmBM, &bars->full[s]);
#pragma unroll
          for (int j = 0; j < kGmmBN / 64; ++j)   // a box past the last column is filled with zeros
            umma::tma_load_2d(dst + kOffB + j * kGmmBoxB, &a.tmap_b, nb * kGmmBN + j * 64, info.x * a.K + ks * kGmmBK, &bars->full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ============================================================ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc_bf16(kGmmBM, kGmmBN);
      uint32_t it = 0, local_tile = 0;
      for (int tile = cta; tile < total_tiles && !*failed; tile += num_ctas, ++local_tile) {
        // one accumulator pair per tile (256-row tiles) or two alternating accumulators (128-row tiles)
        const uint32_t b = kHalves == 2 ? 0u : (local_tile & 1u);
        const uint32_t use = kHalves == 2 ? local_tile : (local_tile >> 1);
        if (!bounded_wait(&bars->acc_empty[b], (use & 1u) ^ 1u, failed)) break;
        umma::fence_after_sync();
        for (int ks = 0; ks < k_steps; ++ks, ++it) {
          const int s = it % kGmmStages;
          if (!bounded_wait(&bars->full[s], (it / kGmmStages) & 1u, failed)) break;
          umma::fence_after_sync();
          const uint32_t a_addr = smem_u32(tiles + (size_t)s * kGmmStageBytes);
          const uint64_t db = smem_desc_mn_sw128(a_addr + kOffB, kGmmBoxB);
#pragma unroll
          for (int m = 0; m < kHalves; ++m) {
            const uint64_t da = umma::smem_desc_sw128(a_addr + m * kGmmTileA);
#pragma unroll
            for (int k = 0; k < kGmmBK / 16; ++k)   // A: 16 values = 32 bytes inside the swizzle row; B: 16 K-rows = 2048 bytes
              mma_f16(tmem + (kHalves == 2 ? m : b) * kGmmBN, da + 2 * k, db + (uint64_t)(16 * 128 / 16) * k, idesc, ks > 0 || k > 0);
          }
          umma::commit(&bars->empty[s]);
        }
        umma::commit(&bars->acc_full[b]);
      }
    }
  } else {
    // ============================================================ epilogue (warps 2..9)
    const int quad = warp & 3;                       // TMEM lanes [32 * quad, 32 * quad + 32)
    const int part = (warp - 2) >> 2;                // which half of the tile's columns this warp handles
    const int row_in_tile = quad * 32 + lane;
    constexpr int kCols = kGmmBN / 2;
    uint32_t local_tile = 0;
    for (int tile = cta; tile < total_tiles && !*failed; tile += num_ctas, ++local_tile) {
      const int mt = tile / n_tiles, nb = tile - mt * n_tiles;
      const int4 info = __ldcg(tile_info + mt);
      const uint32_t b = kHalves == 2 ? 0u : (local_tile & 1u);
      const uint32_t use = kHalves == 2 ? local_tile : (local_tile >> 1);
      // This warp drains its 32 lanes of both accumulators (rows m * 128 + quad * 32 + lane); each thread stores its
      // row's columns straight from registers, 64 contiguous bytes per 32 columns, to this rank's output (a2av_gmm) or
      // into the receive area of the rank the row came from (gmm_a2av).
      if (!bounded_wait(&bars->acc_full[b], use & 1u, failed)) break;
      umma::fence_after_sync();
#pragma unroll
      for (int m = 0; m < kHalves; ++m) {
        const int r = m * kGmmBM + row_in_tile;
        uint8_t* dst_row = nullptr;
        if (r < info.z) {
          const int g = info.y + r;
          if (!kPush) {
            dst_row = reinterpret_cast<uint8_t*>(a.out) + ((size_t)g * a.N + (size_t)nb * kGmmBN) * 2;
          } else {
            int seg = info.x * P;
            while (seg + 1 < (info.x + 1) * P && sh.seg_dst[seg + 1] <= g) ++seg;
            const long long back = sh.seg_src[seg] + (g - sh.seg_dst[seg]);
            dst_row = a.ctx.ws[seg - info.x * P] + a.data_off + ((size_t)back * a.N + (size_t)nb * kGmmBN) * 2;
          }
        }
        const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16) + m * kGmmBN + part * kCols;
        uint32_t v[32];
        for (int c = 0; c < kCols; c += 32) {
          umma::tmem_ld32(taddr + c, v);
          umma::tmem_ld_wait();
          const int col = nb * kGmmBN + part * kCols + c;
          if (dst_row && col < a.N) {
            uint4* dst = reinterpret_cast<uint4*>(dst_row + (size_t)(part * kCols + c) * 2);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint32_t w0[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 b0 = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 2 * j]), __uint_as_float(v[8 * i + 2 * j + 1]));
                w0[j] = *reinterpret_cast<uint32_t*>(&b0);
              }
              dst[i] = make_uint4(w0[0], w0[1], w0[2], w0[3]);
            }
          }
        }
      }
      umma::fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_empty[b]);
    }
    if (kPush) __threadfence_system();   // rows pushed to peers are visible before this rank signals them
  }

  umma::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *failed && a.error_flag) *a.error_flag = 1;
  if (warp == 1) {
    umma::fence_after_sync();
    umma::tmem_dealloc(tmem, 512);
  }
}

// Grid-stride copy of `bytes` (a multiple of 16) with all threads of this rank's blocks.
__device__ __forceinline__ void rank_copy(void* dst, const void* src, size_t bytes) {
  const size_t n = bytes / 16, stride = (size_t)gridDim.x * blockDim.x;
  const int4* s = reinterpret_cast<const int4*>(src);
  int4* d = reinterpret_cast<int4*>(dst);
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n; i += 4 * stride) {
    const int4 v0 = __ldcs(s + i), v1 = __ldcs(s + i + stride), v2 = __ldcs(s + i + 2 * stride), v3 = __ldcs(s + i + 3 * stride);
    d[i] = v0; d[i + stride] = v1; d[i + 2 * stride] = v2; d[i + 3 * stride] = v3;
  }
  for (; i < n; i += stride) d[i] = __ldcs(s + i);
}

// ---------------------------------------------------------------- a2av_gmm
__global__ void __launch_bounds__(kGmmGemmThreads + kGmmPullWarps * 32, 1) a2av_gmm_kernel(const __grid_constant__ GmmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ GmmShared sh;
  cg::grid_group grid = cg::this_grid();
  const GmmArgs& a = p.r[blockIdx.y];
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, me = ctx.rank, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  Control* ctl = control_of(ctx.ws[me]);
  const unsigned long long epoch = ctl->epoch[kOpA2avGmm] + 1;

  // the peers have finished reading what the previous call staged here
  int ok = 1;
  if (threadIdx.x < P) ok = wait_flag_ge(&ctl->gmm_flag[threadIdx.x][1], epoch - 1, ctx, kOpA2avGmm, 0, threadIdx.x);
  int alive = __syncthreads_and(ok);
  // x that already lives in the stage area (a view handed out by the host API) needs no copy
  if (alive && reinterpret_cast<const uint8_t*>(a.x) != ctx.ws[me] + a.data_off)
    rank_copy(ctx.ws[me] + a.data_off, a.x, (size_t)a.rows_in * a.K * 2);
  if (blockIdx.x == 0) {
    if (warp == 0) publish_table(a, reinterpret_cast<int*>(ctx.ws[me] + a.table_off), a.rows_in, lane);
    for (int i = threadIdx.x; i < a.max_tiles; i += (int)blockDim.x) a.pulled[i] = 0;
  }
  __threadfence_system();
  grid.sync();
  if (blockIdx.x == 0 && threadIdx.x < P) st_release_sys(&control_of(ctx.ws[threadIdx.x])->gmm_flag[me][0], epoch);
  ok = 1;
  if (threadIdx.x < P) ok = wait_flag_ge(&ctl->gmm_flag[threadIdx.x][0], epoch, ctx, kOpA2avGmm, 1, threadIdx.x);
  alive = __syncthreads_and(ok) && alive;

  build_layout(a, sh, alive, min(a.gathered_cap, a.out_rows_cap), gmm_tile_rows(false));
  __threadfence();
  grid.sync();

  if (warp < kGmmGemmThreads / 32) {
    gmm_phase<false>(a, sh, a.pulled, smem_raw, blockIdx.x, gridDim.x);
  } else {
    __syncthreads();                               // pairs with the set-up barrier inside gmm_phase
    pull_phase(a, sh, blockIdx.x * kGmmPullWarps + (warp - kGmmGemmThreads / 32), gridDim.x * kGmmPullWarps);
    __syncthreads();                               // pairs with the tear-down barrier inside gmm_phase
  }
  grid.sync();
  if (blockIdx.x == 0) {
    if (threadIdx.x < P) st_release_sys(&control_of(ctx.ws[threadIdx.x])->gmm_flag[me][1], epoch);   // done reading your stage
    if (threadIdx.x == 0) ctl->epoch[kOpA2avGmm] = epoch;
  }
}

// ---------------------------------------------------------------- gmm_a2av
__global__ void __launch_bounds__(kGmmGemmThreads, 1) gmm_a2av_kernel(const __grid_constant__ GmmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ GmmShared sh;
  cg::grid_group grid = cg::this_grid();
  const GmmArgs& a = p.r[blockIdx.y];
  const RankCtx& ctx = a.ctx;
  const int P = ctx.world, me = ctx.rank, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  Control* ctl = control_of(ctx.ws[me]);
  const unsigned long long epoch = ctl->epoch[kOpGmmA2av] + 1;
  int* table = reinterpret_cast<int*>(ctx.ws[me] + a.table_off);

  // this rank's previous call has copied its returned rows out (stream order): the area may be written again
  if (blockIdx.x == 0 && warp == 0) publish_table(a, table, a.out_rows_cap, lane);
  __threadfence_system();
  grid.sync();
  if (blockIdx.x == 0 && threadIdx.x < P) st_release_sys(&control_of(ctx.ws[threadIdx.x])->gmm_flag[me][2], epoch);
  int ok = 1;
  if (threadIdx.x < P) ok = wait_flag_ge(&ctl->gmm_flag[threadIdx.x][2], epoch, ctx, kOpGmmA2av, 0, threadIdx.x);
  int alive = __syncthreads_and(ok);

  build_layout(a, sh, alive, a.rows_in, gmm_tile_rows(true));
  __threadfence();
  grid.sync();
  gmm_phase<true>(a, sh, nullptr, smem_raw, blockIdx.x, gridDim.x);
  __threadfence_system();
  grid.sync();

  if (blockIdx.x == 0 && threadIdx.x < P) st_release_sys(&control_of(ctx.ws[threadIdx.x])->gmm_flag[me][3], epoch);
  ok = 1;
  if (threadIdx.x < P) ok = wait_flag_ge(&ctl->gmm_flag[threadIdx.x][3], epoch, ctx, kOpGmmA2av, 1, threadIdx.x);
  alive = __syncthreads_and(ok) && alive;
  const int my_rows = min(__ldcg(table), a.out_rows_cap);
  // an output tensor that is a view of the receive area already holds the rows
  if (alive && reinterpret_cast<uint8_t*>(a.out) != ctx.ws[me] + a.data_off)
    rank_copy(a.out, ctx.ws[me] + a.data_off, (size_t)my_rows * a.N * 2);
  if (blockIdx.x == 0 && threadIdx.x == 0) ctl->epoch[kOpGmmA2av] = epoch;
}

static cudaError_t launch(const void* fn, int threads, size_t smem, const GmmParams& p, int nranks, int blocks, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  dim3 grid(blocks, nranks), block(threads);
  void* args[] = {const_cast<GmmParams*>(&p)};
  return cudaLaunchCooperativeKernel(fn, grid, block, args, smem, stream);
}
cudaError_t launch_a2av_gmm(const GmmParams& p, int nranks, int blocks, cudaStream_t stream) {
  return launch((const void*)a2av_gmm_kernel, kGmmGemmThreads + kGmmPullWarps * 32, gmm_smem_bytes(false), p, nranks, blocks, stream);
}
cudaError_t launch_gmm_a2av(const GmmParams& p, int nranks, int blocks, cudaStream_t stream) {
  return launch((const void*)gmm_a2av_kernel, kGmmGemmThreads, gmm_smem_bytes(true), p, nranks, blocks, stream);
}

bool encode_bf16_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows, const char** error) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) {
      *error = "cuTensorMapEncodeTiled is not available";
      return false;
    }
    encode = reinterpret_cast<EncodeFn>(fn);
  }
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    *error = "cuTensorMapEncodeTiled rejected the operand (base must be 16-byte aligned, the row pitch a multiple of 16 bytes)";
    return false;
  }
  return true;
}

}  // namespace dep
