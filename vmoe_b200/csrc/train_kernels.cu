// Training-step kernels that are not matmuls: fused loss forward+backward (sigmoid and
// softmax cross-entropy over bf16 logits) and the multi-tensor optimizer update over flat
// fp32 parameter/gradient/moment buffers (Adam and SGD with momentum), including the
// global-norm reduction, clip factor, decoupled weight decay, per-tensor learning-rate
// multipliers (0 = frozen) and the refresh of the bf16 compute copies of the weights.
//
// Reference semantics: losses vmoe/train/trainer.py:441-477; optimizer chain
// vmoe/train/optimizer.py:102-139 (gradient scale -> clip -> adam|sgd -> decayed weights ->
// scale by -lr -> freeze), global norms vmoe/train/train_state.py:39-43.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx_sm100.cuh"
#include "vmoe_api.h"

namespace vmoe {

void set_error(const char* fmt, const char* a, int code);

static inline int launch_status2() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
    return -5;
  }
  return 0;
}

__device__ __forceinline__ float block_sum_256(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
  if (warp == 0) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  }
  return t;  // valid in warp 0
}

// ----------------------------------------------------------------------------- losses
// One CTA per example. loss[row] = sum_c bce(logit, label); dlogits = (sigmoid - label)*scale.
// Columns >= n (padding up to ld) get zero gradient.
template <typename LabelT>
__global__ void __launch_bounds__(256)
sigmoid_xent_kernel(const __nv_bfloat16* __restrict__ logits, const LabelT* __restrict__ labels,
                    float* __restrict__ loss, __nv_bfloat16* __restrict__ dlogits, int n,
                    long long ld, long long ld_labels, float grad_scale) {
  __shared__ float red[8];
  const long long row = blockIdx.x;
  const __nv_bfloat16* x = logits + row * ld;
  const LabelT* z = labels + row * ld_labels;
  __nv_bfloat16* dx = dlogits ? dlogits + row * ld : nullptr;
  float acc = 0.f;
  for (int c = threadIdx.x; c < ld; c += blockDim.x) {
    if (c < n) {
      const float v = __bfloat162float(x[c]);
      const float t = static_cast<float>(z[c]);
      const float ea = __expf(-fabsf(v));
      acc += fmaxf(v, 0.f) - v * t + log1pf(ea);
      if (dx) {
        const float sig = v >= 0.f ? 1.f / (1.f + ea) : ea / (1.f + ea);
        dx[c] = __float2bfloat16((sig - t) * grad_scale);
      }
    } else if (dx) {
      dx[c] = __float2bfloat16(0.f);
    }
  }
  const float total = block_sum_256(acc, red);
  if (threadIdx.x == 0) loss[row] = total;
}

// loss[row] = -sum_c label_c * log_softmax(logits)_c; dlogits = (softmax*sum(label) - label)*scale
template <typename LabelT>
__global__ void __launch_bounds__(256)
softmax_xent_kernel(const __nv_bfloat16* __restrict__ logits, const LabelT* __restrict__ labels,
                    float* __restrict__ loss, __nv_bfloat16* __restrict__ dlogits, int n,
                    long long ld, long long ld_labels, float grad_scale) {
  __shared__ float red[8];
  __shared__ float bcast[3];
  const long long row = blockIdx.x;
  const __nv_bfloat16* x = logits + row * ld;
  const LabelT* z = labels + row * ld_labels;
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < n; c += blockDim.x) mx = fmaxf(mx, __bfloat162float(x[c]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = red[0];
    for (int i = 1; i < (blockDim.x >> 5); ++i) m = fmaxf(m, red[i]);
    bcast[0] = m;
  }
  __syncthreads();
  mx = bcast[0];
  float se = 0.f, sl = 0.f, slx = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float v = __bfloat162float(x[c]) - mx;
    const float t = static_cast<float>(z[c]);
    se += __expf(v);
    sl += t;
    slx += t * v;
  }
  se = block_sum_256(se, red);
  if (threadIdx.x == 0) bcast[1] = se;
  sl = block_sum_256(sl, red);
  if (threadIdx.x == 0) bcast[2] = sl;
  slx = block_sum_256(slx, red);
  __syncthreads();
  const float sum_exp = bcast[1], sum_lab = bcast[2];
  const float lse = __logf(sum_exp);
  if (threadIdx.x == 0) loss[row] = sum_lab * lse - slx;
  if (dlogits) {
    __nv_bfloat16* dx = dlogits + row * ld;
    for (int c = threadIdx.x; c < ld; c += blockDim.x) {
      float gval = 0.f;
      if (c < n) {
        const float v = __bfloat162float(x[c]) - mx;
        gval = (__expf(v) / sum_exp * sum_lab - static_cast<float>(z[c])) * grad_scale;
      }
      dx[c] = __float2bfloat16(gval);
    }
  }
}

// ----------------------------------------------------------------------------- optimizer
constexpr int OPT_CHUNK = 1024;  // elements per metadata entry; tensors are padded to this

struct ChunkMeta {  // one per OPT_CHUNK elements of the flat buffers
  float weight_decay;
  float lr_mult;     // 0 freezes the tensor
  float grad_scale;  // per-tensor gradient multiplier applied before clipping
  float pad;
};

// sums[0] += sum((g * grad_scale)^2)   (double accumulation)
__global__ void __launch_bounds__(256)
grad_sumsq_kernel(const float* __restrict__ g, const ChunkMeta* __restrict__ meta, long long n,
                  double* __restrict__ sums) {
  __shared__ float red[8];
  float acc = 0.f;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(g + i);
    const float sc = meta ? meta[i / OPT_CHUNK].grad_scale : 1.f;
    acc += sc * sc * (v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
  }
  const float t = block_sum_256(acc, red);
  if (threadIdx.x == 0) atomicAdd(sums, static_cast<double>(t));
}

// mode 0: Adam (bias-corrected), mode 1: SGD with momentum trace (m = g + momentum * m).
// update = -lr * lr_mult * (direction + wd * p); sums[1] += update^2, sums[2] += p_new^2.
// clip: if clip_norm > 0, g *= clip_norm / max(sqrt(sums[0]), clip_norm)   (global-norm clip);
//       if clip_value > 0, g = clamp(g, -clip_value, clip_value).
// grad_div divides every gradient first (number of ranks / microsteps already summed).
__global__ void __launch_bounds__(256)
optimizer_step_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                      float* __restrict__ v, __nv_bfloat16* __restrict__ shadow,
                      const ChunkMeta* __restrict__ meta, long long n, int mode, float lr,
                      float b1, float b2, float eps, float bc1, float bc2, float momentum,
                      float clip_norm, float clip_value, float grad_div, double* __restrict__ sums) {
  __shared__ float red[8];
  float gfac = 1.f / grad_div;
  if (clip_norm > 0.f) {
    const float norm = static_cast<float>(sqrt(sums[0])) / grad_div;
    gfac *= clip_norm / fmaxf(norm, clip_norm);
  }
  float upd2 = 0.f, par2 = 0.f;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
    const ChunkMeta cm = meta[i / OPT_CHUNK];
    float4 pv = *reinterpret_cast<float4*>(p + i);
    const float4 gv4 = *reinterpret_cast<const float4*>(g + i);
    float4 mv = *reinterpret_cast<float4*>(m + i);
    float4 vv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (mode == 0) vv = *reinterpret_cast<float4*>(v + i);
    float pa[4] = {pv.x, pv.y, pv.z, pv.w};
    const float ga[4] = {gv4.x, gv4.y, gv4.z, gv4.w};
    float ma[4] = {mv.x, mv.y, mv.z, mv.w};
    float va[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float gg = ga[j] * cm.grad_scale * gfac;
      if (clip_value > 0.f) gg = fminf(fmaxf(gg, -clip_value), clip_value);
      float dir;
      if (mode == 0) {
        ma[j] = b1 * ma[j] + (1.f - b1) * gg;
        va[j] = b2 * va[j] + (1.f - b2) * gg * gg;
        dir = (ma[j] / bc1) / (sqrtf(va[j] / bc2) + eps);
      } else {
        ma[j] = gg + momentum * ma[j];
        dir = ma[j];
      }
      const float upd = -lr * cm.lr_mult * (dir + cm.weight_decay * pa[j]);
      pa[j] += upd;
      upd2 += upd * upd;
      par2 += pa[j] * pa[j];
    }
    *reinterpret_cast<float4*>(p + i) = make_float4(pa[0], pa[1], pa[2], pa[3]);
    *reinterpret_cast<float4*>(m + i) = make_float4(ma[0], ma[1], ma[2], ma[3]);
    if (mode == 0) *reinterpret_cast<float4*>(v + i) = make_float4(va[0], va[1], va[2], va[3]);
    if (shadow) {
      uint2 q;
      q.x = pack_bf16x2(pa[0], pa[1]);
      q.y = pack_bf16x2(pa[2], pa[3]);
      *reinterpret_cast<uint2*>(shadow + i) = q;
    }
  }
  if (sums) {
    const float t1 = block_sum_256(upd2, red);
    if (threadIdx.x == 0) atomicAdd(sums + 1, static_cast<double>(t1));
    const float t2 = block_sum_256(par2, red);
    if (threadIdx.x == 0) atomicAdd(sums + 2, static_cast<double>(t2));
  }
}

}  // namespace vmoe

using namespace vmoe;

extern "C" int vmoe_xent(int32_t kind, const void* logits, const void* labels,
                         int32_t labels_dtype, float* loss, void* dlogits, int64_t rows, int64_t n,
                         int64_t ld, int64_t ld_labels, float grad_scale, vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (rows == 0) return 0;
  auto x = static_cast<const __nv_bfloat16*>(logits);
  auto dx = static_cast<__nv_bfloat16*>(dlogits);
  const unsigned grid = static_cast<unsigned>(rows);
  const int nn = static_cast<int>(n);
#define VMOE_XENT(KERNEL, T)                                                              \
  KERNEL<T><<<grid, 256, 0, stream>>>(x, static_cast<const T*>(labels), loss, dx, nn, ld, \
                                      ld_labels, grad_scale)
  if (kind == 0) {
    if (labels_dtype == 0) VMOE_XENT(sigmoid_xent_kernel, float);
    else if (labels_dtype == 1) VMOE_XENT(sigmoid_xent_kernel, __nv_bfloat16);
    else VMOE_XENT(sigmoid_xent_kernel, uint8_t);
  } else {
    if (labels_dtype == 0) VMOE_XENT(softmax_xent_kernel, float);
    else if (labels_dtype == 1) VMOE_XENT(softmax_xent_kernel, __nv_bfloat16);
    else VMOE_XENT(softmax_xent_kernel, uint8_t);
  }
#undef VMOE_XENT
  return launch_status2();
}

extern "C" int vmoe_grad_sumsq(const float* g, const void* meta, int64_t n, double* sums,
                               vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (n == 0) return 0;
  if (n % 4) {
    set_error("%s (code %d)", "optimizer buffers must be padded to a multiple of 4", 0);
    return -1;
  }
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  grad_sumsq_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
      g, static_cast<const ChunkMeta*>(meta), n, sums);
  return launch_status2();
}

extern "C" int vmoe_optimizer_step(float* p, const float* g, float* m, float* v, void* shadow,
                                   const void* meta, int64_t n, int32_t mode, float lr, float b1,
                                   float b2, float eps, float bc1, float bc2, float momentum,
                                   float clip_norm, float clip_value, float grad_div, double* sums,
                                   vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (n == 0) return 0;
  if (n % OPT_CHUNK) {
    set_error("%s (code %d)", "optimizer buffers must be padded to the chunk size", 0);
    return -1;
  }
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  optimizer_step_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
      p, g, m, v, static_cast<__nv_bfloat16*>(shadow), static_cast<const ChunkMeta*>(meta), n, mode,
      lr, b1, b2, eps, bc1, bc2, momentum, clip_norm, clip_value, grad_div, sums);
  return launch_status2();
}
