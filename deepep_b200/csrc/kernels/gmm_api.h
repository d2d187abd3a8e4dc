// All-to-all-v fused with a bf16 grouped GEMM: argument blocks and launchers.
//
// Counterpart of the reference's experiments/ep_gmm_fused (csrc/all_to_allv_grouped_mat_mul_udma and
// csrc/grouped_mat_mul_all_to_allv_udma; python ops.py:182-369):
//   a2av_gmm   rows sorted by global expert travel to the expert's rank, which multiplies them by its experts' weights
//   gmm_a2av   the expert rank multiplies its gathered rows by its experts' weights and the results travel back
// Row order on the expert rank: local expert first, source rank second, source order inside a segment.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace dep {

constexpr int kGmmBM = 128;   // rows per accumulator (TMEM lanes); a2av_gmm tiles hold two of them
constexpr int kGmmBN = 256;   // output columns per tile
constexpr int kGmmBK = 64;    // K elements per pipeline stage (one 128-byte swizzle row of bf16)
constexpr int kGmmTableInts = 4 + kMaxExperts + 1;   // header (rows, -, -, -) + exclusive prefix of the per-expert row counts

// Byte offsets of the GMM areas inside a workspace (relative to WsLayout::mega); identical on every rank.
struct GmmRegion {
  long long table_a;   // int [kGmmTableInts]   a2av_gmm: where each expert's rows start in this rank's staged x
  long long table_b;   // int [kGmmTableInts]   gmm_a2av: where each expert's rows start in this rank's output
  long long stage;     // bf16 [max_rows][max_k] a2av_gmm: this rank's x, read by the expert ranks
  long long recv;      // bf16 [max_rows][max_n] gmm_a2av: rows returned to this rank, written by the expert ranks
  long long total;
};
__host__ __device__ inline GmmRegion gmm_region(long long max_rows, long long max_k, long long max_n) {
  GmmRegion g;
  long long at = 0;
  auto take = [&](long long b) { long long o = at; at = (at + b + 1023) / 1024 * 1024; return o; };
  g.table_a = take(kGmmTableInts * 4);
  g.table_b = take(kGmmTableInts * 4);
  g.stage = take(max_rows * max_k * 2);
  g.recv = take(max_rows * max_n * 2);
  g.total = at;
  return g;
}

struct GmmArgs {
  RankCtx ctx;
  long long table_off, data_off;   // absolute byte offsets in a workspace: this op's table, its stage / recv area
  const __nv_bfloat16* x;          // a2av_gmm: [rows_in, K] sorted by global expert; gmm_a2av: [rows_in, K] grouped by (local expert, source)
  const int* counts;               // [E] rows this rank sends to (a2av_gmm) / gets back from (gmm_a2av) every global expert
  __nv_bfloat16* out;              // a2av_gmm: [out_rows_cap, N] on the expert rank; gmm_a2av: [out_rows_cap, N] on the source rank
  __nv_bfloat16* gathered;         // a2av_gmm: [gathered_cap, K] the all-to-all-v result, A operand of the GEMM
  CUtensorMap tmap_a;              // A operand [rows, K] bf16: box 64 x 128, 128-byte swizzle
  CUtensorMap tmap_b;              // weights [L * K, N] bf16 (N contiguous): box 64 (N) x 64 (K), 128-byte swizzle
  int rows_in, E, K, N;
  int out_rows_cap, gathered_cap, max_tiles, pad;
  int* tile_info;                  // scratch [max_tiles][4]: local expert, first row, rows, -
  int* num_tiles;                  // [2]: tiles in use, rows on the expert side
  int* pulled;                     // scratch [max_tiles]: rows of each tile that have arrived (a2av_gmm)
  int* error_flag;                 // 1: a pipeline wait ran out; 2: the row counts exceed a capacity or disagree with x
};
struct GmmParams { WsLayout lay; GmmArgs r[kMaxRanks]; };
cudaError_t launch_a2av_gmm(const GmmParams& p, int nranks, int blocks, cudaStream_t stream);
cudaError_t launch_gmm_a2av(const GmmParams& p, int nranks, int blocks, cudaStream_t stream);

// 2-D bf16 tensor map, `cols` contiguous, 128-byte swizzle, box {64 columns, box_rows}.
bool encode_bf16_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows, const char** error);

}  // namespace dep
