// Soft MoE routing weights: from the logits of one group (tokens x slots, fp32) to the dispatch
// weights (softmax over the tokens, per slot) and the combine weights (softmax over the slots,
// per token) in one pass, and the matching backward pass.
//
// One CTA owns one group. Forward keeps the group's logits in shared memory: rows (tokens) are
// reduced by one warp each, columns (slots) by one lane each, so both directions read shared
// memory without bank conflicts, and the two outputs are written with coalesced stores.
// Backward needs two dot products per element,
//   d_logits = D * (dD - sum_tokens(dD * D)) + C * (dC - sum_slots(dC * C)),
// which are accumulated in shared memory first (per slot, per token) and applied in a second
// sweep over the group.
#include <cuda_runtime.h>
#include <stdint.h>

#include "vmoe_api.h"

namespace vmoe {

void set_error(const char* fmt, const char* a, int code);

namespace {

constexpr int kSoftThreads = 256;
constexpr int kSoftWarps = kSoftThreads / 32;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// smem: tile[m * s] | row_max[m] | row_inv[m] | col_max[s] | col_inv[s]
__global__ void __launch_bounds__(kSoftThreads)
soft_router_fwd_kernel(const float* __restrict__ logits, float* __restrict__ dispatch,
                       float* __restrict__ combine, int m, int s) {
  extern __shared__ float soft_smem[];
  float* tile = soft_smem;
  float* row_max = tile + static_cast<size_t>(m) * s;
  float* row_inv = row_max + m;
  float* col_max = row_inv + m;
  float* col_inv = col_max + s;
  const long long base = static_cast<long long>(blockIdx.x) * m * s;
  const int total = m * s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  for (int i = threadIdx.x; i < total; i += kSoftThreads) tile[i] = logits[base + i];
  __syncthreads();

  // Rows: one warp per token, lanes stride over the slots.
  for (int r = warp; r < m; r += kSoftWarps) {
    const float* row = tile + static_cast<size_t>(r) * s;
    float mx = -INFINITY;
    for (int c = lane; c < s; c += 32) mx = fmaxf(mx, row[c]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int c = lane; c < s; c += 32) sum += __expf(row[c] - mx);
    sum = warp_sum(sum);
    if (lane == 0) {
      row_max[r] = mx;
      row_inv[r] = 1.f / sum;
    }
  }
  // Columns: one lane per slot (consecutive lanes read consecutive words), looping over tokens.
  for (int c = threadIdx.x; c < s; c += kSoftThreads) {
    float mx = -INFINITY;
    for (int r = 0; r < m; ++r) mx = fmaxf(mx, tile[static_cast<size_t>(r) * s + c]);
    float sum = 0.f;
    for (int r = 0; r < m; ++r) sum += __expf(tile[static_cast<size_t>(r) * s + c] - mx);
    col_max[c] = mx;
    col_inv[c] = 1.f / sum;
  }
  __syncthreads();

  for (int i = threadIdx.x; i < total; i += kSoftThreads) {
    const int r = i / s, c = i - r * s;
    const float x = tile[i];
    dispatch[base + i] = __expf(x - col_max[c]) * col_inv[c];
    combine[base + i] = __expf(x - row_max[r]) * row_inv[r];
  }
}

// smem: col_dot[s] | row_dot[m]
__global__ void __launch_bounds__(kSoftThreads)
soft_router_bwd_kernel(const float* __restrict__ dispatch, const float* __restrict__ combine,
                       const float* __restrict__ d_dispatch, const float* __restrict__ d_combine,
                       float* __restrict__ d_logits, int m, int s) {
  extern __shared__ float soft_smem[];
  float* col_dot = soft_smem;
  float* row_dot = col_dot + s;
  const long long base = static_cast<long long>(blockIdx.x) * m * s;
  const int total = m * s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  for (int c = threadIdx.x; c < s; c += kSoftThreads) {
    float acc = 0.f;
    if (d_dispatch)
      for (int r = 0; r < m; ++r) {
        const long long i = base + static_cast<long long>(r) * s + c;
        acc += d_dispatch[i] * dispatch[i];
      }
    col_dot[c] = acc;
  }
  for (int r = warp; r < m; r += kSoftWarps) {
    float acc = 0.f;
    if (d_combine)
      for (int c = lane; c < s; c += 32) {
        const long long i = base + static_cast<long long>(r) * s + c;
        acc += d_combine[i] * combine[i];
      }
    acc = warp_sum(acc);
    if (lane == 0) row_dot[r] = acc;
  }
  __syncthreads();

  for (int i = threadIdx.x; i < total; i += kSoftThreads) {
    const int r = i / s, c = i - r * s;
    float g = 0.f;
    if (d_dispatch) g += dispatch[base + i] * (d_dispatch[base + i] - col_dot[c]);
    if (d_combine) g += combine[base + i] * (d_combine[base + i] - row_dot[r]);
    d_logits[base + i] = g;
  }
}

int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
    return -5;
  }
  return 0;
}

size_t fwd_smem_bytes(int m, int s) {
  return (static_cast<size_t>(m) * s + 2 * static_cast<size_t>(m) + 2 * static_cast<size_t>(s)) *
         sizeof(float);
}

}  // namespace
}  // namespace vmoe

using namespace vmoe;

extern "C" int64_t vmoe_soft_router_max_group_elements(void) {
  // Largest tokens * slots of one group whose logits fit the forward kernel's shared memory
  // (leaving room for the row / column statistics of groups up to 4096 tokens or slots).
  return (227 * 1024 - 4 * 4096 * 4) / 4;
}

extern "C" int vmoe_soft_router_fwd(const float* logits, float* dispatch, float* combine,
                                    int64_t groups, int32_t m, int32_t s, vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (groups <= 0 || m <= 0 || s <= 0) return 0;
  const size_t smem = fwd_smem_bytes(m, s);
  if (smem > 227 * 1024 || groups > 0x7fffffffLL) {
    set_error("%s (code %d)", "soft router: a group does not fit in shared memory", m);
    return -1;
  }
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(soft_router_fwd_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) {
      set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
      return -5;
    }
    configured = smem;
  }
  soft_router_fwd_kernel<<<static_cast<unsigned>(groups), kSoftThreads, smem, stream>>>(
      logits, dispatch, combine, m, s);
  return check_launch();
}

extern "C" int vmoe_soft_router_bwd(const float* dispatch, const float* combine,
                                    const float* d_dispatch, const float* d_combine,
                                    float* d_logits, int64_t groups, int32_t m, int32_t s,
                                    vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (groups <= 0 || m <= 0 || s <= 0) return 0;
  const size_t smem = (static_cast<size_t>(m) + s) * sizeof(float);
  if (smem > 48 * 1024 || groups > 0x7fffffffLL) {
    set_error("%s (code %d)", "soft router backward: group too large", m);
    return -1;
  }
  soft_router_bwd_kernel<<<static_cast<unsigned>(groups), kSoftThreads, smem, stream>>>(
      dispatch, combine, d_dispatch, d_combine, d_logits, m, s);
  return check_launch();
}
