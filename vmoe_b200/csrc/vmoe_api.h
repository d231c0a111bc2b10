// C ABI of libvmoe_b200.so. Every function takes raw device pointers and a CUDA stream and
// returns 0 on success or a negative error code (see vmoe_b200/ops/_lib.py for the ctypes
// mirror of these declarations). Nothing here depends on PyTorch.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* vmoe_stream_t;  // cudaStream_t
#define VMOE_API __attribute__((visibility("default")))

// ----------------------------------------------------------------------------- GEMM
// C[b] (M x N) = epilogue( A[b] (M x K) * B[b] (N x K)^T ), bf16 operands, fp32 accumulation
// on tcgen05 tensor cores with TMEM accumulators and TMA-fed shared memory.
//
// Operand storage ("major"):
//   a_mn_major = 0: A stored [M][lda] (K contiguous);  1: A stored [K][lda] (M contiguous)
//   b_mn_major = 0: B stored [N][ldb] (K contiguous);  1: B stored [K][ldb] (N contiguous)
// so that forward (x W^T), dgrad (dy W) and wgrad (dy^T x) all run without a transpose.
//
// Epilogue, in this order, per output element v = acc:
//   v += bias[col]                       (bias != NULL; fp32, length N per batch)
//   pre-activation copy to C2            (C2 != NULL; bf16, same layout as C)
//   v = gelu_tanh(v)                     (act == 1)
//   v *= gelu_tanh'(gelu_pre[row, col])  (gelu_pre != NULL; bf16, leading dim ldr2)
//   v += residual[row, col]              (residual != NULL; bf16, leading dim ldr)
//   colsum[col] += sum over rows of v    (colsum != NULL; fp32 atomics)
//   C[row, col] = v                      (bf16 or fp32 store, or fp32 atomic add)
typedef struct VmoeGemmArgs {
  const void* A;
  const void* B;
  void* C;
  void* C2;
  const float* bias;
  const void* residual;
  const void* gelu_pre;
  float* colsum;
  const unsigned* a_ready;  // optional per-(batch, m-tile) arrival counters for A rows
  unsigned* status;         // optional device status word (bits: see ptx_sm100.cuh)
  int64_t M, N, K, batch;
  int64_t lda, ldb, ldc, ldr, ldr2;
  int64_t a_batch_stride, b_batch_stride, c_batch_stride, bias_batch_stride, r_batch_stride;
  int32_t a_mn_major, b_mn_major;
  int32_t c_fp32;    // 0: C is bf16, 1: C is fp32
  int32_t c_atomic;  // 1: C += v with fp32 atomics (needs c_fp32)
  int32_t act;       // 0 none, 1 GELU(tanh)
  int32_t split_k;   // >1 splits the K range over CTAs (needs c_atomic)
  uint32_t a_ready_epoch;  // A tile (b, mt) may be loaded once a_ready[...] >= epoch * rows
  int32_t num_sms;   // CTAs to launch at most (0: all SMs of the device)
} VmoeGemmArgs;

VMOE_API int vmoe_gemm_bf16(const VmoeGemmArgs* args, vmoe_stream_t stream);

// Last error text of the calling thread ("" if none).
VMOE_API const char* vmoe_last_error(void);

#ifdef __cplusplus
}
#endif
