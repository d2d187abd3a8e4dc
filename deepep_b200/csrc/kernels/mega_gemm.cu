// Stand-alone launch of the grouped block-scaled GEMM phase (see mega_gemm.cuh) and the tensor-map encoder.
#include "mega_gemm.cuh"

namespace dep {

__global__ void __launch_bounds__(kGemmThreads, 1) mega_gemm_kernel(const __grid_constant__ MegaGemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  gemm_phase<false>(p, nullptr, nullptr, smem_raw, p.stages ? p.stages : (p.epi == kEpiCombine ? 3 : 4), blockIdx.x, gridDim.x, nullptr, 0,
                    p.commit_every ? p.commit_every : 1);
}
// The same as CTA pairs: launched as clusters of two CTAs.
__global__ void __launch_bounds__(kGemmThreads, 1) mega_gemm_pair_kernel(const __grid_constant__ MegaGemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  gemm_phase<true>(p, nullptr, nullptr, smem_raw, p.stages ? p.stages : 4, blockIdx.x / 2, gridDim.x / 2, nullptr, 0,
                   p.commit_every ? p.commit_every : 1);
}

cudaError_t launch_mega_gemm(const MegaGemmParams& p, int blocks, cudaStream_t stream) {
  // shared memory: the operand pipeline (a CTA of a pair holds half of the weights tile), the scale chunks, the epilogue's
  // staging area for the combine epilogue, barriers
  const bool staging = p.epi == kEpiCombine;
  const int stages = p.stages ? p.stages : (p.pair ? 4 : (staging ? 3 : 4));
  const size_t stage_bytes = (size_t)kTileABytes + (p.pair ? 128 : kGemmBN) * kGemmBK + kSfStageBytes;
  const size_t smem = 1024 + stages * stage_bytes + (staging ? kEpiStageBytes : 0) + 256;
  if (smem > 227 * 1024) return cudaErrorInvalidValue;
  const void* fn = p.pair ? (const void*)mega_gemm_pair_kernel : (const void*)mega_gemm_kernel;
  // the attribute belongs to the current device, so it is set on every launch (a process may drive several GPUs)
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  void* args[] = {const_cast<MegaGemmParams*>(&p)};
  if (p.pair) {
    if (blocks < 2) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks / 2 * 2); cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelExC(&cfg, fn, args);
  }
  return cudaLaunchKernel(fn, dim3(blocks), dim3(kGemmThreads), args, smem, stream);
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeFn tensor_map_encoder(const char** error) {
  static EncodeFn encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) {
      *error = "cuTensorMapEncodeTiled is not available";
      return nullptr;
    }
    encode = reinterpret_cast<EncodeFn>(fn);
  }
  return encode;
}

bool encode_sf_map(CUtensorMap* map, const void* base, long long chunks, const char** error) {
  EncodeFn encode = tensor_map_encoder(error);
  if (!encode) return false;
  cuuint64_t dims[2] = {kSfChunk / 4, (cuuint64_t)(chunks > 0 ? chunks : 1)};
  cuuint64_t strides[1] = {kSfChunk};
  cuuint32_t box[2] = {kSfChunk / 4, 1};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, elem,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    *error = "cuTensorMapEncodeTiled rejected the scale chunks (check the 16-byte alignment of the base)";
    return false;
  }
  return true;
}

bool encode_operand_map(CUtensorMap* map, const void* base, long long rows, long long k, bool fp4, const char** error) {
  EncodeFn encode = tensor_map_encoder(error);
  if (!encode) return false;
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(fp4 ? k / 2 : k)};
  cuuint32_t box[2] = {kGemmBK, 128};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = encode(map, fp4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base),
                      dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    *error = "cuTensorMapEncodeTiled rejected the operand (check 16/32-byte alignment of base and row stride)";
    return false;
  }
  return true;
}

}  // namespace dep
