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
// VEC4: s is a multiple of 4 and all three arrays are 16-byte aligned, so the tile is moved with
// 16-byte accesses.
template <bool VEC4>
__global__ void __launch_bounds__(kSoftThreads)
soft_router_fwd_kernel(const float* __restrict__ logits, float* __restrict__ dispatch,
                       float* __restrict__ combine, int m, int s) {
  extern __shared__ __align__(16) float soft_smem[];
  float* tile = soft_smem;
  float* row_max = tile + static_cast<size_t>(m) * s;
  float* row_inv = row_max + m;
  float* col_max = row_inv + m;
  float* col_inv = col_max + s;
  const long long base = static_cast<long long>(blockIdx.x) * m * s;
  const int total = m * s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (VEC4) {
    const float4* src = reinterpret_cast<const float4*>(logits + base);
    float4* dst = reinterpret_cast<float4*>(tile);
    for (int i = threadIdx.x; i < total / 4; i += kSoftThreads) dst[i] = src[i];
  } else {
    for (int i = threadIdx.x; i < total; i += kSoftThreads) tile[i] = logits[base + i];
  }
  __syncthreads();

  // Rows: eight lanes per token, four tokens per warp at a time (the trip count is the same
  // for all lanes, so the shuffles below always run with a full warp).
  const int sub = lane >> 3, sl = lane & 7;
  for (int r0 = warp * 4; r0 < m; r0 += kSoftWarps * 4) {
    const int r = r0 + sub;
    const bool valid = r < m;
    const float* row = tile + static_cast<size_t>(valid ? r : 0) * s;
    // The four tokens of a warp start at different 8-column blocks, so that with a row
    // length that is a multiple of 32 words they read different shared-memory banks.
    const int nblk = s >> 3, tail = nblk << 3;
    float mx = -INFINITY;
    if (valid) {
      for (int k = 0, blk = sub % max(nblk, 1); k < nblk; ++k, blk = blk + 1 == nblk ? 0 : blk + 1)
        mx = fmaxf(mx, row[(blk << 3) + sl]);
      if (tail + sl < s) mx = fmaxf(mx, row[tail + sl]);
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    float sum = 0.f;
    if (valid) {
      for (int k = 0, blk = sub % max(nblk, 1); k < nblk; ++k, blk = blk + 1 == nblk ? 0 : blk + 1)
        sum += __expf(row[(blk << 3) + sl] - mx);
      if (tail + sl < s) sum += __expf(row[tail + sl] - mx);
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 4);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    if (valid && sl == 0) {
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

  // Outputs: one warp per token row, lanes across the slots.
  for (int r = warp; r < m; r += kSoftWarps) {
    const float rmx = row_max[r], rinv = row_inv[r];
    const long long rbase = base + static_cast<long long>(r) * s;
    const float* row = tile + static_cast<size_t>(r) * s;
    if (VEC4) {
      for (int c = lane * 4; c < s; c += 128) {
        const float4 x = *reinterpret_cast<const float4*>(row + c);
        float4 d, o;
        d.x = __expf(x.x - col_max[c + 0]) * col_inv[c + 0];
        d.y = __expf(x.y - col_max[c + 1]) * col_inv[c + 1];
        d.z = __expf(x.z - col_max[c + 2]) * col_inv[c + 2];
        d.w = __expf(x.w - col_max[c + 3]) * col_inv[c + 3];
        o.x = __expf(x.x - rmx) * rinv;
        o.y = __expf(x.y - rmx) * rinv;
        o.z = __expf(x.z - rmx) * rinv;
        o.w = __expf(x.w - rmx) * rinv;
        *reinterpret_cast<float4*>(dispatch + rbase + c) = d;
        *reinterpret_cast<float4*>(combine + rbase + c) = o;
      }
    } else {
      for (int c = lane; c < s; c += 32) {
        const float x = row[c];
        dispatch[rbase + c] = __expf(x - col_max[c]) * col_inv[c];
        combine[rbase + c] = __expf(x - rmx) * rinv;
      }
    }
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
  const auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool vec4 = s % 4 == 0 && aligned(logits) && aligned(dispatch) && aligned(combine);
  static size_t configured[2] = {0, 0};
  if (smem > 48 * 1024 && smem > configured[vec4]) {
    cudaError_t e = vec4 ? cudaFuncSetAttribute(soft_router_fwd_kernel<true>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                static_cast<int>(smem))
                         : cudaFuncSetAttribute(soft_router_fwd_kernel<false>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                static_cast<int>(smem));
    if (e != cudaSuccess) {
      set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
      return -5;
    }
    configured[vec4] = smem;
  }
  if (vec4)
    soft_router_fwd_kernel<true><<<static_cast<unsigned>(groups), kSoftThreads, smem, stream>>>(
        logits, dispatch, combine, m, s);
  else
    soft_router_fwd_kernel<false><<<static_cast<unsigned>(groups), kSoftThreads, smem, stream>>>(
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
