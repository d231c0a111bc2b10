// Host-side helper shared by the kernels that build TMA tensor maps.
#pragma once
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>

namespace vmoe {

inline PFN_cuTensorMapEncodeTiled tma_encode_fn() {
  static PFN_cuTensorMapEncodeTiled fn = nullptr;
  if (fn) return fn;
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || ptr == nullptr) return nullptr;
  fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(ptr);
  return fn;
}

// cuTensorMapEncodeTiled with one retry: a thread that has made no runtime call yet (e.g. an
// autograd worker thread) has no current driver context; cudaFree(0) binds the primary one.
inline CUresult tma_encode_tiled(CUtensorMap* map, CUtensorMapDataType dtype, cuuint32_t rank,
                                 void* addr, const cuuint64_t* dims, const cuuint64_t* strides,
                                 const cuuint32_t* box, const cuuint32_t* estr,
                                 CUtensorMapSwizzle swizzle) {
  PFN_cuTensorMapEncodeTiled enc = tma_encode_fn();
  if (!enc) return CUDA_ERROR_NOT_SUPPORTED;
  CUresult r = enc(map, dtype, rank, addr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT || r == CUDA_ERROR_NOT_INITIALIZED) {
    cudaFree(0);
    r = enc(map, dtype, rank, addr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  return r;
}

}  // namespace vmoe
