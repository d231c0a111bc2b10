// Router statistics for the noisy Top-K router: from gating logits (tokens x experts, fp32) to
// the softmax gates used for dispatch and the per-group sums behind the auxiliary losses
// (importance, load, GShard), plus the matching backward pass.
//
// One thread owns one token (E <= 64 values in registers). Group sums are reduced inside a warp
// when all of its tokens belong to one group (the common case) and added with one atomic per
// value; the losses themselves are computed by a one-thread-per-group kernel.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "vmoe_api.h"

namespace vmoe {

void set_error(const char* fmt, const char* a, int code);

namespace {

inline int launch_status(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
    return -5;
  }
  (void)what;
  return 0;
}

constexpr float kInvSqrt2 = 0.70710678118654752f;
constexpr float kInvSqrt2Pi = 0.39894228040143268f;

template <int MAXE>
struct TokenRoute {
  float gc[MAXE];  // clean softmax
  float go[MAXE];  // gates used for dispatch (noisy softmax when noise is on)
  float z[MAXE];   // (threshold - clean logit) / std  (noise only)
  int kth;         // index of the K-th largest noisy logit
  int top1;        // argmax of go
};

template <int MAXE>
__device__ __forceinline__ void softmax_e(const float (&l)[MAXE], int e_count, float (&out)[MAXE]) {
  float mx = -INFINITY;
#pragma unroll
  for (int e = 0; e < MAXE; ++e)
    if (e < e_count) mx = fmaxf(mx, l[e]);
  float s = 0.f;
#pragma unroll
  for (int e = 0; e < MAXE; ++e) {
    out[e] = e < e_count ? __expf(l[e] - mx) : 0.f;
    s += out[e];
  }
  const float inv = 1.f / s;
#pragma unroll
  for (int e = 0; e < MAXE; ++e) out[e] *= inv;
}

template <int MAXE>
__device__ __forceinline__ void route_token(const float* __restrict__ logits,
                                            const float* __restrict__ noise, long long m,
                                            int e_count, float noise_std, int k,
                                            TokenRoute<MAXE>& r) {
  float l[MAXE], ln[MAXE];
#pragma unroll
  for (int e = 0; e < MAXE; ++e) l[e] = e < e_count ? logits[m * e_count + e] : -INFINITY;
  softmax_e<MAXE>(l, e_count, r.gc);
  r.kth = 0;
  if (noise != nullptr) {
#pragma unroll
    for (int e = 0; e < MAXE; ++e)
      ln[e] = e < e_count ? l[e] + noise[m * e_count + e] * noise_std : -INFINITY;
    softmax_e<MAXE>(ln, e_count, r.go);
    // K-th largest noisy logit, ties to the lowest index.
    unsigned long long taken = 0ull;
    int sel = 0;
    for (int j = 0; j < k; ++j) {
      float best = -INFINITY;
      sel = 0;
      bool found = false;
#pragma unroll
      for (int e = 0; e < MAXE; ++e) {
        if (e < e_count && !((taken >> e) & 1ull) && (!found || ln[e] > best)) {
          best = ln[e];
          sel = e;
          found = true;
        }
      }
      taken |= 1ull << sel;
    }
    r.kth = sel;
    float thr = 0.f;
#pragma unroll
    for (int e = 0; e < MAXE; ++e)
      if (e == sel) thr = ln[e];
    const float inv_std = 1.f / noise_std;
#pragma unroll
    for (int e = 0; e < MAXE; ++e) r.z[e] = e < e_count ? (thr - l[e]) * inv_std : 0.f;
  } else {
#pragma unroll
    for (int e = 0; e < MAXE; ++e) {
      r.go[e] = r.gc[e];
      r.z[e] = 0.f;
    }
  }
  r.top1 = 0;
  float best = -INFINITY;
#pragma unroll
  for (int e = 0; e < MAXE; ++e) {
    if (e < e_count && r.go[e] > best) {
      best = r.go[e];
      r.top1 = e;
    }
  }
}

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// sums layout: [G][4][E] = importance (clean gates), load (p), top-1 counts, dispatch gates.
template <int MAXE>
__global__ void __launch_bounds__(128)
router_stats_fwd_kernel(const float* __restrict__ logits, const float* __restrict__ noise,
                        float* __restrict__ gates_out, float* __restrict__ sums, long long tokens,
                        int group_size, int e_count, float noise_std, int k) {
  const long long m = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool valid = m < tokens;
  const long long mm = valid ? m : tokens - 1;
  TokenRoute<MAXE> r;
  route_token<MAXE>(logits, noise, mm, e_count, noise_std, k, r);
  if (valid) {
#pragma unroll
    for (int e = 0; e < MAXE; ++e)
      if (e < e_count) gates_out[m * e_count + e] = r.go[e];
  }
  const int g = static_cast<int>(mm / group_size);
  const int g0 = __shfl_sync(0xffffffffu, g, 0);
  const bool uniform = __all_sync(0xffffffffu, g == g0);
  const int lane = threadIdx.x & 31;
  float* base = sums + static_cast<long long>(g) * 4 * e_count;
  const float w = valid ? 1.f : 0.f;
#pragma unroll
  for (int e = 0; e < MAXE; ++e) {
    if (e >= e_count) break;
    const float p = noise != nullptr ? 0.5f * erfcf(r.z[e] * kInvSqrt2) : 0.f;
    float v0 = w * r.gc[e], v1 = w * p, v2 = w * (r.top1 == e ? 1.f : 0.f), v3 = w * r.go[e];
    if (uniform) {
      v0 = warp_sum_f(v0);
      v1 = warp_sum_f(v1);
      v2 = warp_sum_f(v2);
      v3 = warp_sum_f(v3);
      if (lane == 0) {
        atomicAdd(base + e, v0);
        atomicAdd(base + e_count + e, v1);
        atomicAdd(base + 2 * e_count + e, v2);
        atomicAdd(base + 3 * e_count + e, v3);
      }
    } else if (valid) {
      atomicAdd(base + e, v0);
      atomicAdd(base + e_count + e, v1);
      atomicAdd(base + 2 * e_count + e, v2);
      atomicAdd(base + 3 * e_count + e, v3);
    }
  }
}

// losses: [G][3] = importance, load, gshard. coef: [G][3][E] = d loss / d sum.
__global__ void router_losses_kernel(const float* __restrict__ sums, float* __restrict__ losses,
                                     float* __restrict__ coef, int groups, int group_size,
                                     int e_count, int has_noise) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= groups) return;
  const float* s = sums + static_cast<long long>(g) * 4 * e_count;
  float* c = coef + static_cast<long long>(g) * 3 * e_count;
  const float inv_e = 1.f / e_count;
  for (int which = 0; which < 2; ++which) {  // squared coefficient of variation
    const float* v = s + which * e_count;
    float mean = 0.f;
    for (int e = 0; e < e_count; ++e) mean += v[e];
    mean *= inv_e;
    float var = 0.f;
    for (int e = 0; e < e_count; ++e) var += (v[e] - mean) * (v[e] - mean);
    var *= inv_e;
    const bool on = which == 0 || has_noise;
    losses[g * 3 + which] = on ? var / (mean * mean) : 0.f;
    for (int e = 0; e < e_count; ++e)
      c[which * e_count + e] =
          on ? 2.f * inv_e * (v[e] - mean) / (mean * mean) - 2.f * var * inv_e / (mean * mean * mean)
             : 0.f;
  }
  const float inv_s = 1.f / group_size;
  float acc = 0.f;
  for (int e = 0; e < e_count; ++e) {
    acc += s[2 * e_count + e] * s[3 * e_count + e];
    c[2 * e_count + e] = e_count * s[2 * e_count + e] * inv_s * inv_s;
  }
  losses[g * 3 + 2] = acc * e_count * inv_s * inv_s;
}

template <int MAXE>
__global__ void __launch_bounds__(128)
router_stats_bwd_kernel(const float* __restrict__ logits, const float* __restrict__ noise,
                        const float* __restrict__ d_gates, const float* __restrict__ d_losses,
                        const float* __restrict__ coef, float* __restrict__ d_logits,
                        __nv_bfloat16* __restrict__ d_logits_bf16, int ld_bf16, long long tokens,
                        int group_size, int e_count, float noise_std, int k) {
  const long long m = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (m >= tokens) return;
  TokenRoute<MAXE> r;
  route_token<MAXE>(logits, noise, m, e_count, noise_std, k, r);
  const int g = static_cast<int>(m / group_size);
  const float* c = coef + static_cast<long long>(g) * 3 * e_count;
  const float dl_imp = d_losses ? d_losses[g * 3 + 0] : 0.f;
  const float dl_load = d_losses ? d_losses[g * 3 + 1] : 0.f;
  const float dl_gsh = d_losses ? d_losses[g * 3 + 2] : 0.f;
  float dgc[MAXE], dgo[MAXE], dl[MAXE];
  float dot_c = 0.f, dot_o = 0.f;
#pragma unroll
  for (int e = 0; e < MAXE; ++e) {
    const bool in = e < e_count;
    dgc[e] = in ? dl_imp * c[e] : 0.f;
    dgo[e] = in ? (d_gates ? d_gates[m * e_count + e] : 0.f) + dl_gsh * c[2 * e_count + e] : 0.f;
    dot_c += r.gc[e] * dgc[e];
    dot_o += r.go[e] * dgo[e];
  }
  float dthr = 0.f;
#pragma unroll
  for (int e = 0; e < MAXE; ++e) {
    float v = r.gc[e] * (dgc[e] - dot_c) + r.go[e] * (dgo[e] - dot_o);
    if (noise != nullptr && e < e_count) {
      // p = 1 - Phi(z), z = (thr - l) / std: dp/dl = pdf(z) / std, dp/dthr = -pdf(z) / std.
      const float pdf = kInvSqrt2Pi * __expf(-0.5f * r.z[e] * r.z[e]) / noise_std;
      const float dp = dl_load * c[e_count + e];
      v += dp * pdf;
      dthr -= dp * pdf;
    }
    dl[e] = v;
  }
#pragma unroll
  for (int e = 0; e < MAXE; ++e) {
    if (e >= e_count) break;
    const float v = dl[e] + (noise != nullptr && e == r.kth ? dthr : 0.f);
    if (d_logits) d_logits[m * e_count + e] = v;
    if (d_logits_bf16) d_logits_bf16[m * ld_bf16 + e] = __float2bfloat16(v);
  }
}

}  // namespace

}  // namespace vmoe

using namespace vmoe;

#define VMOE_ROUTER_DISPATCH(E, CALL)                     \
  if ((E) <= 8) { CALL(8); }                              \
  else if ((E) <= 16) { CALL(16); }                       \
  else if ((E) <= 32) { CALL(32); }                       \
  else { CALL(64); }

extern "C" int vmoe_router_stats_fwd(const float* logits, const float* noise, float* gates_out,
                                     float* sums, float* losses, float* coef, int64_t tokens,
                                     int64_t group_size, int num_experts, float noise_std, int k,
                                     vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (tokens == 0) return 0;
  if (num_experts < 1 || num_experts > 64 || k < 1 || k > num_experts || group_size < 1 ||
      tokens % group_size) {
    set_error("%s (code %d)", "router_stats: need 1 <= k <= experts <= 64 and tokens % group == 0", 0);
    return -1;
  }
  const int groups = static_cast<int>(tokens / group_size);
  cudaMemsetAsync(sums, 0, sizeof(float) * groups * 4 * num_experts, stream);
  const int threads = 128;
  const unsigned grid = static_cast<unsigned>((tokens + threads - 1) / threads);
#define CALL(ME) router_stats_fwd_kernel<ME><<<grid, threads, 0, stream>>>(                    \
      logits, noise, gates_out, sums, tokens, static_cast<int>(group_size), num_experts,      \
      noise_std, k)
  VMOE_ROUTER_DISPATCH(num_experts, CALL)
#undef CALL
  router_losses_kernel<<<(groups + 127) / 128, 128, 0, stream>>>(
      sums, losses, coef, groups, static_cast<int>(group_size), num_experts, noise != nullptr);
  return launch_status("router_stats_fwd");
}

extern "C" int vmoe_router_stats_bwd(const float* logits, const float* noise, const float* d_gates,
                                     const float* d_losses, const float* coef, float* d_logits,
                                     void* d_logits_bf16, int64_t ld_bf16, int64_t tokens,
                                     int64_t group_size, int num_experts, float noise_std, int k,
                                     vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (tokens == 0) return 0;
  if (num_experts < 1 || num_experts > 64 || k < 1 || k > num_experts || group_size < 1) {
    set_error("%s (code %d)", "router_stats_bwd: need 1 <= k <= experts <= 64", 0);
    return -1;
  }
  const int threads = 128;
  const unsigned grid = static_cast<unsigned>((tokens + threads - 1) / threads);
#define CALL(ME) router_stats_bwd_kernel<ME><<<grid, threads, 0, stream>>>(                    \
      logits, noise, d_gates, d_losses, coef, d_logits,                                       \
      static_cast<__nv_bfloat16*>(d_logits_bf16), static_cast<int>(ld_bf16), tokens,          \
      static_cast<int>(group_size), num_experts, noise_std, k)
  VMOE_ROUTER_DISPATCH(num_experts, CALL)
#undef CALL
  return launch_status("router_stats_bwd");
}
