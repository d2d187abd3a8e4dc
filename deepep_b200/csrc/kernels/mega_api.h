// Fused MoE (MegaMoE): argument blocks and launchers.
//
// Counterpart of the reference's experiments/megamoe (csrc/forward.cpp:237-478, kernels/mega_moe/*):
// dispatch -> grouped GEMM1 (fp8 activations x fp4 weights, block-scaled) -> SwiGLU + MXFP8 requant ->
// grouped GEMM2 -> combine into the source rank -> weighted unpermute.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace dep {

constexpr int kGemmBM = 128;   // token rows per tile (TMEM lanes)
constexpr int kGemmBN = 256;   // output columns per tile
constexpr int kGemmBK = 128;   // K elements per pipeline stage (one 128-byte swizzle row of fp8)
constexpr int kSfChunk = 512;  // bytes of block scales of 128 rows x 128 K-elements (ue8m0 per 32)

// Scale factors of a [rows, K] operand are stored as 512-byte chunks, one per (128-row block, 128-K block):
// byte (r % 32) * 16 + (r % 128) / 32 * 4 + (k / 32) % 4 of chunk (r / 128) * (K / 128) + k / 128.
// This is the image tcgen05.cp 32x128b.warpx4 moves into tensor memory without any shuffling.
__host__ __device__ inline long long sf_offset(long long row, long long k, long long K) {
  return ((row / 128) * (K / 128) + k / 128) * kSfChunk + (row % 32) * 16 + (row % 128) / 32 * 4 + (k / 32) % 4;
}

constexpr int kGemmMaxStagesHost = 6;   // deepest operand pipeline of the grouped GEMM

enum GemmEpilogue : int {
  kEpiStoreF32 = 0,        // C fp32 [rows, N] (tests)
  kEpiSwigluQuant = 1,     // tile = [128 gate | 128 up] columns -> silu(gate) * up -> e4m3 + ue8m0 per 32
  kEpiCombine = 2          // bf16 rows written into the source rank's combine slots over NVLink
};

struct MegaGemmParams {
  CUtensorMap tmap_a;        // activations [rows_pad, K] e4m3, box 128 x 128, 128-byte swizzle
  CUtensorMap tmap_b;        // weights, tiled as [(rows / 128) * (K / 128) * 128, 128 values]: e2m1 pairs that the copy engine widens
                             // to one byte per value, or e4m3 bytes (b_fp8)
  CUtensorMap tmap_sfa, tmap_sfb;   // the chunked scales as [chunks][512 B] (CTA pairs load them through the copy engine's tile path)
  const uint8_t* sfa;        // chunked scales of A
  const uint8_t* sfb;        // chunked scales of B
  const int* mtile_expert;   // [max_mtiles] local expert of each 128-row tile
  const int* a_ready;        // optional: rows of each tile of A in place so far; a tile's loads start at 128
  const int* num_mtiles;     // device scalar: tiles in use
  int max_mtiles, n_tiles, k_steps, n_total;
  int epi, b_tx_bytes;
  int pair, stages;          // stand-alone launch only: run as CTA pairs (the tile list must pair row blocks 2j, 2j + 1 of one expert);
                             // pipeline stages (0 = default)
  int commit_every, pad3;    // stand-alone launch only: stages released per tcgen05.commit (0 = 1)
  // kEpiStoreF32
  float* c;
  int ldc, b_fp8;            // b_fp8: the weights are e4m3 (A8W8) instead of e2m1 (A8W4)
  // kEpiSwigluQuant
  uint8_t* a2;               // [rows_pad, inter] e4m3
  uint8_t* a2_sf;            // chunked scales of a2
  int inter, pad1;
  // kEpiCombine
  const int* row_src;        // [rows_pad] (source * M + token) * topk + slot, -1 for padding rows
  uint8_t* ws[kMaxRanks];    // every rank's workspace
  long long comb_off;        // byte offset of the combine slots [M][topk][H] bf16 in a workspace
  int max_tokens, topk, hidden, pad2;
  int* error_flag;           // set when a pipeline wait ran out
  long long* debug;          // optional: cycle counters of block 0 (producer wait/issue/stages, MMA wait/issue/acc wait)
};
cudaError_t launch_mega_gemm(const MegaGemmParams& p, int blocks, cudaStream_t stream);

// Encodes a 2-D tensor map with a {128 (K), 128 (rows)} box and the 128-byte swizzle.
// fp4 = true: elements are packed e2m1 pairs that the copy engine widens to one byte each in shared memory.
bool encode_operand_map(CUtensorMap* map, const void* base, long long rows, long long k, bool fp4, const char** error);
// Encodes an array of 512-byte scale chunks as a 2-D map {128 x uint32, chunks} with a one-chunk box, no swizzle.
bool encode_sf_map(CUtensorMap* map, const void* base, long long chunks, const char** error);

// Phase stamps of the fused kernel, one record per CTA (globaltimer nanoseconds): kernel start, inputs quantised and
// handshake done, routing layout done, token pull done (pull warps), GEMM tile loop done, finish handshake done, end.
constexpr int kMegaTimerWords = 8;
enum MegaTimerSlot : int { kTimStart = 0, kTimHandshake = 1, kTimLayout = 2, kTimPull = 3, kTimGemm = 4, kTimFinishSync = 5, kTimEnd = 6,
                            kTimMmaThread = 7 };   // word 7: the MMA thread's cycles / 16, (waiting for operands) << 32 | (whole tile loop)

// ---------------------------------------------------------------- routing + token pull
struct MegaRouteArgs {
  RankCtx ctx;
  long long in_off;            // byte offset of the input block (x, x_sf, topk_idx, topk_w) in a workspace
  int T, E, K, H;              // tokens of this rank, experts, top-k, hidden
  int max_tokens, max_mtiles;
  int S, tile_pairs;           // tile_pairs: every expert's rows start at a multiple of 256 (pairs of 128-row tiles of one expert)
                               // S: shared experts of this rank: local experts E / world .. E / world + S - 1, fed with all of its own tokens
  const __nv_bfloat16* x_bf16; // optional [T, H]: quantised to MXFP8 into the input block at the start of the kernel
  unsigned long long* timer;   // optional [blocks][kMegaTimerWords] phase stamps in nanoseconds (see mega_tools.parse_timer)
  // outputs
  uint8_t* a1;                 // [rows_pad, H] e4m3
  uint8_t* a1_sf;              // chunked scales
  int* row_src;                // [rows_pad]
  int* mtile_expert;           // [max_mtiles]
  int* num_mtiles;             // [1]
  int* expert_rows;            // [L] rows per local expert
  int* expert_list;            // [L][world * max_tokens] scratch: routed slots of each local expert
  int* pulled;                 // optional [max_mtiles]: rows of each tile in place so far (zeroed by the caller)
};
struct MegaRouteParams { WsLayout lay; MegaRouteArgs r[kMaxRanks]; };
cudaError_t launch_mega_route(const MegaRouteParams& p, int nranks, int blocks, cudaStream_t stream);

// Byte size and region offsets {hdr, x, x_sf, topk_idx, topk_w, total} of the symmetric input block.
long long mega_input_bytes(int max_tokens, int hidden, int topk);
void mega_input_offsets(int max_tokens, int hidden, int topk, long long* out6);

struct MegaFinishArgs {
  RankCtx ctx;
  long long in_off, comb_off;
  int T, E, K, H, max_tokens, S;   // S shared experts: combine slots K .. K + S - 1 of a token carry their rows (weight 1)
  unsigned long long* timer;
  __nv_bfloat16* y;            // [T, H]
};
struct MegaFinishParams { WsLayout lay; MegaFinishArgs r[kMaxRanks]; };
cudaError_t launch_mega_finish(const MegaFinishParams& p, int nranks, int blocks, cudaStream_t stream);

// ---------------------------------------------------------------- the fused layer (one persistent kernel)
struct MegaFusedArgs {
  MegaGemmParams g1, g2;       // GEMM1 (SwiGLU + requant epilogue) and GEMM2 (combine epilogue)
  MegaRouteArgs route;
  MegaFinishArgs finish;
  int* ready;                  // [max_mtiles] finished GEMM1 tiles per row block (zeroed by the kernel)
  int* tile_counter;           // [1] next tile of the GEMM1 + GEMM2 tile list (zeroed by the kernel); null: static round-robin
  int interleave, pair;        // pair: CTA pairs share the weights tile (cluster of two; needs route.tile_pairs)
                               // interleave k > 0: GEMM2 tiles follow their GEMM1 wave (waves of 2k rounds of GEMM1 tiles); 0: all GEMM1 tiles first
};
struct MegaFusedParams { WsLayout lay; MegaFusedArgs r[kMaxRanks]; };
cudaError_t launch_mega_fused(const MegaFusedParams& p, int nranks, int blocks, cudaStream_t stream);

}  // namespace dep
