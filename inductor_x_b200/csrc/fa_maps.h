// Tensor maps of the attention kernels (forward and backward): a [B, H, S, 128] view of
// 16-bit elements with arbitrary strides that are multiples of 16 bytes, copied in boxes of
// 64 columns x 128 rows with the 128-byte swizzle the tcgen05 shared-memory descriptors expect.
#pragma once
#include <cuda.h>

#include "host.h"

namespace ixb_host {

// cuTensorMapEncodeTiled, fetched through the runtime so the library does not link libcuda
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// dims (d, s, h, b); strides in elements; rows past S are zero-filled by the copy engine
inline int make_fa_map(CUtensorMap* map, const void* base, int is_bf16, int B, int H, int S, long long sb,
                       long long sh, long long ss) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return IXB_ERR_CUDA;
  const cuuint64_t dims[4] = {128, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  const cuuint64_t strides[3] = {(cuuint64_t)ss * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  const cuuint32_t box[4] = {64, 128, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                        4, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? IXB_OK : IXB_ERR_ARG;
}

}  // namespace ixb_host
