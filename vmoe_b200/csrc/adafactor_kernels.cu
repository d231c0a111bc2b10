// big_vision Adafactor as three table-driven kernels over ALL parameter tensors of a bucket
// (vmoe/train/optimizer.py:238-286 wraps optax's scale_by_factored_rms + momentum):
//
//   stats    per tile of 16 rows: g = grad * scale (clipped), row sums of g^2 + eps go straight
//            into the row accumulator's moving average, column partial sums are added to a
//            scratch vector with one atomic per column and tile;
//   finish   per (tensor, batch entry): column moving average from the scratch sums, mean of the
//            row vector (the normaliser of optax's factored preconditioner);
//   update   per 1024-element chunk: u = g * rsqrt(row / mean) * rsqrt(col)  (or g * rsqrt(v) for
//            small / 1-D tensors, whose full second moment is updated here), momentum, weight
//            decay, parameter and bf16-shadow write, sums of squares of update and parameter.
//
// A tensor is (batch, R, C) row-major: the factored axes are the last two (the two largest; the
// host checks). `rows_are_d1` says which accumulator plays optax's "v_row" (the mean over the
// LARGEST axis): the row vector when C is the largest axis, else the column vector.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx_sm100.cuh"
#include "vmoe_api.h"

namespace vmoe {

void set_error(const char* fmt, const char* a, int code);

struct AfTensor {  // mirrors VmoeAdafactorTensor
  float* p;
  const float* g;
  float* mu;
  __nv_bfloat16* shadow;
  float* vr;       // (batch, R)  mean of g^2 over columns   (factored)
  float* vc;       // (batch, C)  mean of g^2 over rows      (factored)
  float* v;        // (numel)     full second moment         (not factored)
  float* col_acc;  // (batch, C)  scratch, zero on entry, zero on exit
  float* norm;     // (batch)     scratch: mean of the normalising vector
  long long batch, rows, cols;
  float weight_decay, lr_mult, grad_scale;
  int factored, c_is_largest;
  long long chunk0;  // first 1024-element chunk of this tensor in the update kernel's work list
};

constexpr int AF_TILE_ROWS = 16;
constexpr int AF_CHUNK = 1024;

__device__ __forceinline__ float af_gfac(float clip_norm, float grad_div, const double* sums) {
  float gfac = 1.f / grad_div;
  if (clip_norm > 0.f) {
    const float norm = static_cast<float>(sqrt(sums[0])) / grad_div;
    gfac *= clip_norm / fmaxf(norm, clip_norm);
  }
  return gfac;
}

__device__ __forceinline__ float af_block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
  if (warp == 0) {
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

// grid.x: row tiles (strided), grid.y: tensor. One warp per row of the tile, lanes over columns.
__global__ void __launch_bounds__(256)
adafactor_stats_kernel(const AfTensor* __restrict__ table, float decay, float eps, float clip_norm,
                       float clip_value, float grad_div, const double* __restrict__ sums) {
  const AfTensor t = table[blockIdx.y];
  if (!t.factored) return;
  const float gfac = af_gfac(clip_norm, grad_div, sums) * t.grad_scale;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long tiles_per_b = (t.rows + AF_TILE_ROWS - 1) / AF_TILE_ROWS;
  const long long tiles = t.batch * tiles_per_b;
  __shared__ float col_part[8][32];
  for (long long tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const long long b = tile / tiles_per_b;
    const long long r0 = (tile % tiles_per_b) * AF_TILE_ROWS;
    const float* gb = t.g + (b * t.rows) * t.cols;
    // columns in slabs of 32: every warp sums its two rows of the tile for the slab's columns
    for (long long c0 = 0; c0 < t.cols; c0 += 32) {
      const long long c = c0 + lane;
      float cs = 0.f;
#pragma unroll
      for (int rr = 0; rr < AF_TILE_ROWS / 8; ++rr) {
        const long long r = r0 + warp + 8 * rr;
        if (r < t.rows && c < t.cols) {
          float gg = gb[r * t.cols + c] * gfac;
          if (clip_value > 0.f) gg = fminf(fmaxf(gg, -clip_value), clip_value);
          cs += gg * gg + eps;
        }
      }
      col_part[warp][lane] = cs;
      __syncthreads();
      if (warp == 0 && c < t.cols) {
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) tot += col_part[w][lane];
        atomicAdd(t.col_acc + b * t.cols + c, tot);
      }
      __syncthreads();
    }
    // row sums: one warp per row, lanes stride over the columns
#pragma unroll
    for (int rr = 0; rr < AF_TILE_ROWS / 8; ++rr) {
      const long long r = r0 + warp + 8 * rr;
      if (r >= t.rows) continue;
      float rs = 0.f;
      for (long long c = lane; c < t.cols; c += 32) {
        float gg = gb[r * t.cols + c] * gfac;
        if (clip_value > 0.f) gg = fminf(fmaxf(gg, -clip_value), clip_value);
        rs += gg * gg + eps;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) rs += __shfl_xor_sync(0xffffffffu, rs, o);
      if (lane == 0) {
        float* vr = t.vr + b * t.rows + r;
        *vr = decay * *vr + (1.f - decay) * rs / static_cast<float>(t.cols);
      }
    }
  }
}

// One CTA per (tensor, batch entry).
__global__ void __launch_bounds__(256)
adafactor_finish_kernel(const AfTensor* __restrict__ table, const long long* __restrict__ first,
                        int num_tensors, float decay) {
  __shared__ float red[8];
  // which tensor does this block belong to: `first[i]` = first block of tensor i
  int ti = 0;
  while (ti + 1 < num_tensors && first[ti + 1] <= static_cast<long long>(blockIdx.x)) ++ti;
  const AfTensor t = table[ti];
  if (!t.factored) return;
  const long long b = blockIdx.x - first[ti];
  if (b >= t.batch) return;
  float* vc = t.vc + b * t.cols;
  float* acc = t.col_acc + b * t.cols;
  float part = 0.f;
  for (long long c = threadIdx.x; c < t.cols; c += blockDim.x) {
    const float nv = decay * vc[c] + (1.f - decay) * acc[c] / static_cast<float>(t.rows);
    vc[c] = nv;
    acc[c] = 0.f;
    if (!t.c_is_largest) part += nv;  // columns are optax's v_row: they carry the normaliser
  }
  if (t.c_is_largest) {
    const float* vr = t.vr + b * t.rows;
    for (long long r = threadIdx.x; r < t.rows; r += blockDim.x) part += vr[r];
  }
  const float tot = af_block_sum(part, red);
  if (threadIdx.x == 0)
    t.norm[b] = tot / static_cast<float>(t.c_is_largest ? t.rows : t.cols);
}

// One CTA per 1024-element chunk of the work list (4 elements per thread).
__global__ void __launch_bounds__(256)
adafactor_update_kernel(const AfTensor* __restrict__ table, int num_tensors, float decay, float eps,
                        float momentum, float lr, float clip_norm, float clip_value,
                        float grad_div, double* __restrict__ sums_in, double* __restrict__ sums_out) {
  __shared__ float red[8];
  int lo = 0, hi = num_tensors - 1;
  while (lo < hi) {  // last tensor whose first chunk is <= this block
    const int mid = (lo + hi + 1) >> 1;
    if (table[mid].chunk0 <= static_cast<long long>(blockIdx.x)) lo = mid; else hi = mid - 1;
  }
  const AfTensor t = table[lo];
  const float gfac = af_gfac(clip_norm, grad_div, sums_in) * t.grad_scale;
  const long long numel = t.batch * t.rows * t.cols;
  const long long base = (static_cast<long long>(blockIdx.x) - t.chunk0) * AF_CHUNK;
  float upd2 = 0.f, par2 = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const long long i = base + threadIdx.x + 256 * j;
    if (i >= numel) continue;
    float gg = t.g[i] * gfac;
    if (clip_value > 0.f) gg = fminf(fmaxf(gg, -clip_value), clip_value);
    float u;
    if (t.factored) {
      const long long rc = t.rows * t.cols;
      const long long b = i / rc, rem = i - b * rc;
      const long long r = rem / t.cols, c = rem - r * t.cols;
      const float vr = t.vr[b * t.rows + r], vc = t.vc[b * t.cols + c], nm = t.norm[b];
      u = t.c_is_largest ? gg * rsqrtf(vr / nm) * rsqrtf(vc) : gg * rsqrtf(vc / nm) * rsqrtf(vr);
    } else {
      const float nv = decay * t.v[i] + (1.f - decay) * (gg * gg + eps);
      t.v[i] = nv;
      u = gg * rsqrtf(nv);
    }
    if (momentum > 0.f) {
      const float m = momentum * t.mu[i] + (1.f - momentum) * u;
      t.mu[i] = m;
      u = m;
    }
    const float pv = t.p[i];
    const float upd = -lr * t.lr_mult * (u + t.weight_decay * pv);
    const float np = pv + upd;
    t.p[i] = np;
    if (t.shadow) t.shadow[i] = __float2bfloat16(np);
    upd2 += upd * upd;
    par2 += np * np;
  }
  const float t1 = af_block_sum(upd2, red);
  if (threadIdx.x == 0) atomicAdd(sums_out + 1, static_cast<double>(t1));
  const float t2 = af_block_sum(par2, red);
  if (threadIdx.x == 0) atomicAdd(sums_out + 2, static_cast<double>(t2));
}

}  // namespace vmoe

using namespace vmoe;

static_assert(sizeof(AfTensor) == sizeof(VmoeAdafactorTensor), "table layouts must agree");

extern "C" int vmoe_adafactor_step(const VmoeAdafactorTensor* table, const int64_t* finish_first,
                                   int32_t num_tensors, int64_t finish_blocks,
                                   int64_t update_chunks, int64_t max_tiles, float decay, float eps,
                                   float momentum, float lr, float clip_norm, float clip_value,
                                   float grad_div, double* sums, vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (num_tensors <= 0) return 0;
  const AfTensor* tb = reinterpret_cast<const AfTensor*>(table);
  if (max_tiles > 0) {
    long long gx = max_tiles < 148 * 4 ? max_tiles : 148 * 4;
    dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(num_tensors));
    adafactor_stats_kernel<<<grid, 256, 0, stream>>>(tb, decay, eps, clip_norm, clip_value,
                                                     grad_div, sums);
  }
  if (finish_blocks > 0)
    adafactor_finish_kernel<<<static_cast<unsigned>(finish_blocks), 256, 0, stream>>>(
        tb, reinterpret_cast<const long long*>(finish_first), num_tensors, decay);
  adafactor_update_kernel<<<static_cast<unsigned>(update_chunks), 256, 0, stream>>>(
      tb, num_tensors, decay, eps, momentum, lr, clip_norm, clip_value, grad_div, sums, sums);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
    return -5;
  }
  return 0;
}
