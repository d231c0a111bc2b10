// Mixup of a batch with rolled copies of itself in one pass:
//   out[l, b, :] = sum_i w[i, l, b] * x[l, (b + i) % B, :]      (i < size, fp32 accumulation)
// for inputs viewed as (lead, B, inner). The PyTorch formulation makes `size` rolled copies and
// as many multiply-adds over the whole batch; here every input element is read `size` times
// (the second read mostly from L2) and the output is written once.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "vmoe_api.h"

namespace vmoe {

void set_error(const char* fmt, const char* a, int code);

namespace {

constexpr int kMixThreads = 256;
constexpr int kMixMaxSize = 8;

__device__ __forceinline__ float mix_load(const float* p) { return *p; }
__device__ __forceinline__ float mix_load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void mix_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void mix_store(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

// One CTA walks one (l, b) row of `inner` elements; weights of the row sit in registers.
template <typename T>
__global__ void __launch_bounds__(kMixThreads)
mixup_kernel(const T* __restrict__ x, T* __restrict__ out, const float* __restrict__ w,
             long long lead_b, int batch, long long inner, int size) {
  for (long long row = blockIdx.x; row < lead_b; row += gridDim.x) {
    const long long l = row / batch;
    const int b = static_cast<int>(row - l * batch);
    float wi[kMixMaxSize];
    const T* src[kMixMaxSize];
#pragma unroll
    for (int i = 0; i < kMixMaxSize; ++i) {
      wi[i] = 0.f;
      src[i] = x;
      if (i < size) {
        wi[i] = w[static_cast<long long>(i) * lead_b + row];
        src[i] = x + (l * batch + (b + i) % batch) * inner;
      }
    }
    T* dst = out + row * inner;
    for (long long j = threadIdx.x; j < inner; j += kMixThreads) {
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < kMixMaxSize; ++i)
        if (i < size) acc += wi[i] * mix_load(src[i] + j);
      mix_store(dst + j, acc);
    }
  }
}

}  // namespace
}  // namespace vmoe

using namespace vmoe;

extern "C" int vmoe_mixup(const void* x, void* out, const float* weights, int32_t is_bf16,
                          int64_t lead, int64_t batch, int64_t inner, int32_t size,
                          vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (lead <= 0 || batch <= 0 || inner <= 0) return 0;
  if (size < 1 || size > kMixMaxSize || batch > 0x7fffffffLL) {
    set_error("%s (code %d)", "mixup: size must be in [1, 8]", size);
    return -1;
  }
  const long long rows = lead * batch;
  const int grid = static_cast<int>(rows < 148LL * 16 ? rows : 148LL * 16);
  if (is_bf16)
    mixup_kernel<__nv_bfloat16><<<grid, kMixThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), weights, rows,
        static_cast<int>(batch), inner, size);
  else
    mixup_kernel<float><<<grid, kMixThreads, 0, stream>>>(
        static_cast<const float*>(x), static_cast<float*>(out), weights, rows,
        static_cast<int>(batch), inner, size);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
    return -5;
  }
  return 0;
}
