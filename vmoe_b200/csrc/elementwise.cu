// Memory-bound kernels of the transformer block: LayerNorm forward/backward, column sums
// (bias gradients), NHWC image -> bf16 patch matrix. All use 16-byte vector accesses on
// bf16 rows and fp32 arithmetic; each is one pass over its inputs.
//
// They replace what the reference leaves to XLA fusions (vmoe/nn/vit_moe.py:164,177,260
// LayerNorm; :337-339 patch-embedding conv input).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdlib.h>
#include <atomic>
#include <stdint.h>

#include "ptx_sm100.cuh"
#include "vmoe_api.h"

namespace vmoe {

void set_error(const char* fmt, const char* a, int code);

static inline int launch_status(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
    return -5;
  }
  (void)what;
  return 0;
}

__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z),
         d = unpack_bf16x2(q.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 q;
  q.x = pack_bf16x2(f[0], f[1]);
  q.y = pack_bf16x2(f[2], f[3]);
  q.z = pack_bf16x2(f[4], f[5]);
  q.w = pack_bf16x2(f[6], f[7]);
  return q;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ----------------------------------------------------------------------------- LayerNorm
// One warp per row; lane l owns the 8-element chunks l, l+32, ... (MAXC of them at most), so
// its gamma/beta values never change and live in registers. The next row's data is fetched
// (as packed bf16) while the current row is reduced, which keeps two rows per warp in flight.
template <int MAXC>
__device__ __forceinline__ void ln_load_row(const __nv_bfloat16* base, long long row, int h,
                                            int lane, int chunks, uint4 (&q)[MAXC]) {
  const uint4* r = reinterpret_cast<const uint4*>(base + row * h);
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int ch = lane + 32 * c;
    q[c] = ch < chunks ? __ldg(r + ch) : make_uint4(0, 0, 0, 0);
  }
}

template <int MAXC>
__device__ __forceinline__ void ln_load_affine(const float* p, int lane, int chunks, float fill,
                                               float (&v)[MAXC][8]) {
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int ch = lane + 32 * c;
#pragma unroll
    for (int i = 0; i < 8; ++i) v[c][i] = fill;
    if (p != nullptr && ch < chunks) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(p + ch * 8));
      const float4 b = __ldg(reinterpret_cast<const float4*>(p + ch * 8) + 1);
      v[c][0] = a.x; v[c][1] = a.y; v[c][2] = a.z; v[c][3] = a.w;
      v[c][4] = b.x; v[c][5] = b.y; v[c][6] = b.z; v[c][7] = b.w;
    }
  }
}

template <int MAXC>
__global__ void __launch_bounds__(256)
layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma,
                     const float* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                     float* __restrict__ mean_out, float* __restrict__ rstd_out, long long rows,
                     int h, float eps) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int chunks = h >> 3;
  float gm[MAXC][8], bt[MAXC][8];
  ln_load_affine<MAXC>(gamma, lane, chunks, 1.0f, gm);
  ln_load_affine<MAXC>(beta, lane, chunks, 0.0f, bt);
  uint4 cur[MAXC], nxt[MAXC];
  if (warp < rows) ln_load_row<MAXC>(x, warp, h, lane, chunks, cur);
  for (long long row = warp; row < rows; row += nwarps) {
    if (row + nwarps < rows) ln_load_row<MAXC>(x, row + nwarps, h, lane, chunks, nxt);
    float v[MAXC][8];
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      unpack8(cur[c], v[c]);
#pragma unroll
      for (int i = 0; i < 8; ++i) s += v[c][i];  // chunks past the row end hold zeros
    }
    const float mean = warp_sum(s) / h;
    float sq = 0.f;
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      if (lane + 32 * c < chunks) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float d = v[c][i] - mean;
          sq += d * d;
        }
      }
    }
    const float rstd = rsqrtf(warp_sum(sq) / h + eps);
    uint4* yr = reinterpret_cast<uint4*>(y + row * h);
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      const int ch = lane + 32 * c;
      if (ch < chunks) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = (v[c][i] - mean) * rstd * gm[c][i] + bt[c][i];
        yr[ch] = pack8(o);
      }
    }
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
#pragma unroll
    for (int c = 0; c < MAXC; ++c) cur[c] = nxt[c];
  }
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)) with g = dy * gamma (+ dres if given).
// Every warp keeps partial sums of dgamma = sum_rows dy * xhat and dbeta = sum_rows dy for its
// own columns in registers; at the end the CTA adds them up in shared memory and writes one
// row of partials to `partial` ([gridDim.x][2*h], scratch memory). A second kernel
// (ln_reduce_partials_kernel) sums the rows of `partial` into dgamma / dbeta, so the result
// does not depend on the order in which CTAs finish.
template <int MAXC>
__global__ void __launch_bounds__(128, MAXC <= 3 ? 3 : 1)
layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                     const float* __restrict__ gamma, const float* __restrict__ mean_in,
                     const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                     __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, long long rows,
                     int h) {
  extern __shared__ float red[];  // [4 warps][2][h]
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int chunks = h >> 3;
  // All per-element arithmetic works on fp32 pairs (one instruction per two values).
  f32x2 gm[MAXC][4], ag[MAXC][4], ab[MAXC][4];
  {
    float g1[MAXC][8];
    ln_load_affine<MAXC>(gamma, lane, chunks, 1.0f, g1);
#pragma unroll
    for (int c = 0; c < MAXC; ++c)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        gm[c][j] = f2_pack(g1[c][2 * j], g1[c][2 * j + 1]);
        ag[c][j] = ab[c][j] = f2_pack(0.f, 0.f);
      }
  }
  uint4 xc[MAXC], dc[MAXC], xn[MAXC], dn[MAXC], rc[MAXC];
  if (warp < rows) {
    ln_load_row<MAXC>(x, warp, h, lane, chunks, xc);
    ln_load_row<MAXC>(dy, warp, h, lane, chunks, dc);
  }
  auto pair_of = [](uint32_t u) {
    const float2 f = unpack_bf16x2(u);
    return f2_pack(f.x, f.y);
  };
  for (long long row = warp; row < rows; row += nwarps) {
    // The residual gradient of this row is requested first, then the next row's x / dy: all
    // of it is in flight while the sums below are formed.
    if (dres) ln_load_row<MAXC>(dres, row, h, lane, chunks, rc);
    if (row + nwarps < rows) {
      ln_load_row<MAXC>(x, row + nwarps, h, lane, chunks, xn);
      ln_load_row<MAXC>(dy, row + nwarps, h, lane, chunks, dn);
    }
    const float mean = __ldg(mean_in + row), rstd = __ldg(rstd_in + row);
    const f32x2 rstd2 = f2_pack(rstd, rstd), nmr2 = f2_pack(-mean * rstd, -mean * rstd);
    f32x2 s1 = f2_pack(0.f, 0.f), s2 = f2_pack(0.f, 0.f);
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      if (lane + 32 * c < chunks) {
        const uint32_t xw[4] = {xc[c].x, xc[c].y, xc[c].z, xc[c].w};
        const uint32_t dw[4] = {dc[c].x, dc[c].y, dc[c].z, dc[c].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const f32x2 xh = f2_fma(pair_of(xw[j]), rstd2, nmr2);  // (x - mean) * rstd
          const f32x2 d = pair_of(dw[j]);
          const f32x2 g = f2_mul(d, gm[c][j]);
          ag[c][j] = f2_fma(d, xh, ag[c][j]);
          ab[c][j] = f2_add(ab[c][j], d);
          s1 = f2_add(s1, g);
          s2 = f2_fma(g, xh, s2);
        }
      }
    }
    float s1a, s1b, s2a, s2b;
    f2_unpack(s1, s1a, s1b);
    f2_unpack(s2, s2a, s2b);
    const float m1 = warp_sum(s1a + s1b) / h, m2 = warp_sum(s2a + s2b) / h;
    const f32x2 nm1 = f2_pack(-m1, -m1), nm2 = f2_pack(-m2, -m2);
    uint4* dxr = reinterpret_cast<uint4*>(dx + row * h);
    const bool rr = dres != nullptr;
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      const int ch = lane + 32 * c;
      if (ch < chunks) {
        const uint32_t xw[4] = {xc[c].x, xc[c].y, xc[c].z, xc[c].w};
        const uint32_t dw[4] = {dc[c].x, dc[c].y, dc[c].z, dc[c].w};
        const uint32_t rw[4] = {rc[c].x, rc[c].y, rc[c].z, rc[c].w};
        uint32_t ow[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const f32x2 xh = f2_fma(pair_of(xw[j]), rstd2, nmr2);
          const f32x2 g = f2_mul(pair_of(dw[j]), gm[c][j]);
          // rstd * (g - m1 - xh * m2) (+ residual gradient)
          f32x2 o = f2_mul(f2_add(f2_fma(xh, nm2, g), nm1), rstd2);
          if (rr) o = f2_add(o, pair_of(rw[j]));
          float oa, ob;
          f2_unpack(o, oa, ob);
          ow[j] = pack_bf16x2(oa, ob);
        }
        dxr[ch] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      }
    }
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      xc[c] = xn[c];
      dc[c] = dn[c];
    }
  }
  if (partial != nullptr) {
    // Each warp stores its sums in its own slice; the four slices are then added in a fixed
    // order, so the result does not depend on warp scheduling.
    float* mine = red + (threadIdx.x >> 5) * 2 * h;
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      const int ch = lane + 32 * c;
      if (ch < chunks) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float a0, a1, b0, b1;
          f2_unpack(ag[c][j], a0, a1);
          f2_unpack(ab[c][j], b0, b1);
          mine[ch * 8 + 2 * j] = a0;
          mine[ch * 8 + 2 * j + 1] = a1;
          mine[h + ch * 8 + 2 * j] = b0;
          mine[h + ch * 8 + 2 * j + 1] = b1;
        }
      }
    }
    __syncthreads();
    float* out = partial + static_cast<long long>(blockIdx.x) * 2 * h;
    for (int i = threadIdx.x; i < 2 * h; i += blockDim.x)
      out[i] = (red[i] + red[2 * h + i]) + (red[4 * h + i] + red[6 * h + i]);
  }
}

// Row r of a tensor whose rows come in blocks of `inner` consecutive rows (stride h) with the
// blocks `outer` elements apart; (inner, outer) = (1, h) is a plain contiguous matrix. Lets the
// short-row kernels read / write the q or k slice of a packed (B, T, 3, H, D) tensor in place.
struct RowMap {
  long long inner, outer;
  int h;
  __device__ __forceinline__ long long at(long long r) const {
    return (r / inner) * outer + (r % inner) * h;
  }
};

// ---- short rows (h = 16, 32, 64 or 128: head-dimension LayerNorm of QK-norm attention)
// LPR = h / 8 lanes hold one row (8 elements each), so a warp normalises 32 / LPR rows at a
// time and the reductions stay inside the LPR-lane group.
template <int LPR>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int LPR>
__global__ void __launch_bounds__(256)
layernorm_fwd_small_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma,
                           const float* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                           float* __restrict__ mean_out, float* __restrict__ rstd_out,
                           long long rows, float eps, RowMap xm, RowMap ym) {
  constexpr int H = LPR * 8, RPW = 32 / LPR;
  const int lane = threadIdx.x & 31, sub = lane / LPR, l = lane % LPR;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  float gm[8], bt[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    gm[i] = gamma ? __ldg(gamma + l * 8 + i) : 1.f;
    bt[i] = beta ? __ldg(beta + l * 8 + i) : 0.f;
  }
  // All groups of a warp run the same number of iterations (rows past the end are masked out),
  // so the shuffles always see a full warp.
  const long long iters = (rows + nwarps * RPW - 1) / (nwarps * RPW);
  for (long long it = 0; it < iters; ++it) {
    const long long row = (it * nwarps + warp) * RPW + sub;
    const bool ok = row < rows;
    float v[8];
    if (ok) {
      unpack8(__ldg(reinterpret_cast<const uint4*>(x + xm.at(row)) + l), v);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += v[i];
    const float mean = group_sum<LPR>(s) / H;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) sq += (v[i] - mean) * (v[i] - mean);
    const float rstd = rsqrtf(group_sum<LPR>(sq) / H + eps);
    if (ok) {
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = (v[i] - mean) * rstd * gm[i] + bt[i];
      reinterpret_cast<uint4*>(y + ym.at(row))[l] = pack8(o);
      if (l == 0) {
        if (mean_out) mean_out[row] = mean;
        if (rstd_out) rstd_out[row] = rstd;
      }
    }
  }
}

template <int LPR>
__global__ void __launch_bounds__(128)
layernorm_bwd_small_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                           const float* __restrict__ gamma, const float* __restrict__ mean_in,
                           const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                           __nv_bfloat16* __restrict__ dx, float* __restrict__ partial,
                           long long rows, RowMap dym, RowMap xm, RowMap dxm) {
  constexpr int H = LPR * 8, RPW = 32 / LPR;
  extern __shared__ float red[];  // [4 warps][2][H]
  const int lane = threadIdx.x & 31, sub = lane / LPR, l = lane % LPR;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  float gm[8], ag[8], ab[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    gm[i] = gamma ? __ldg(gamma + l * 8 + i) : 1.f;
    ag[i] = ab[i] = 0.f;
  }
  // All groups of a warp run the same number of iterations (rows past the end are masked
  // out), so the shuffles always see a full warp.
  const long long iters = (rows + nwarps * RPW - 1) / (nwarps * RPW);
  for (long long it = 0; it < iters; ++it) {
    const long long row = (it * nwarps + warp) * RPW + sub;
    const bool ok = row < rows;
    float xv[8], dv[8];
    if (ok) {
      unpack8(__ldg(reinterpret_cast<const uint4*>(x + xm.at(row)) + l), xv);
      unpack8(__ldg(reinterpret_cast<const uint4*>(dy + dym.at(row)) + l), dv);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) xv[i] = dv[i] = 0.f;
    }
    const float mean = ok ? __ldg(mean_in + row) : 0.f, rstd = ok ? __ldg(rstd_in + row) : 0.f;
    float s1 = 0.f, s2 = 0.f, xh[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      xh[i] = (xv[i] - mean) * rstd;
      const float g = dv[i] * gm[i];
      ag[i] += dv[i] * xh[i];
      ab[i] += dv[i];
      s1 += g;
      s2 += g * xh[i];
    }
    const float m1 = group_sum<LPR>(s1) / H, m2 = group_sum<LPR>(s2) / H;
    if (ok) {
      float o[8], rv[8];
      if (dres) unpack8(__ldg(reinterpret_cast<const uint4*>(dres + row * H) + l), rv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        o[i] = rstd * (dv[i] * gm[i] - m1 - xh[i] * m2);
        if (dres) o[i] += rv[i];
      }
      reinterpret_cast<uint4*>(dx + dxm.at(row))[l] = pack8(o);
    }
  }
  if (partial != nullptr) {
    // Add the groups of the warp (lanes with equal l), then the four warps in a fixed order.
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
      for (int o = LPR; o < 32; o <<= 1) {
        ag[i] += __shfl_xor_sync(0xffffffffu, ag[i], o);
        ab[i] += __shfl_xor_sync(0xffffffffu, ab[i], o);
      }
    }
    float* mine = red + (threadIdx.x >> 5) * 2 * H;
    if (sub == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        mine[l * 8 + i] = ag[i];
        mine[H + l * 8 + i] = ab[i];
      }
    }
    __syncthreads();
    float* out = partial + static_cast<long long>(blockIdx.x) * 2 * H;
    for (int i = threadIdx.x; i < 2 * H; i += blockDim.x)
      out[i] = (red[i] + red[2 * H + i]) + (red[4 * H + i] + red[6 * H + i]);
  }
}

// dgamma[j] += sum_b partial[b][j], dbeta[j] += sum_b partial[b][h + j]. Block = 32 columns x
// 8 row groups; every thread adds a strided subset of the rows in a fixed order and the eight
// partial results are combined through shared memory, also in a fixed order.
__global__ void __launch_bounds__(256)
ln_reduce_partials_kernel(const float* __restrict__ partial, int nblocks, int h,
                          float* __restrict__ dgamma, float* __restrict__ dbeta) {
  __shared__ float part[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int j = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (j < 2 * h)
    for (int b = ty; b < nblocks; b += 8) s += partial[static_cast<long long>(b) * 2 * h + j];
  part[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && j < 2 * h) {
    float t = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) t += part[r][tx];
    if (j < h) {
      if (dgamma) dgamma[j] += t;
    } else if (dbeta) {
      dbeta[j - h] += t;
    }
  }
}

// ----------------------------------------------------------------------------- column sum
// out[b][n] += sum_r x[b][r][n]; CTA = 32 row-lanes x 32 column-chunks of 8.
__global__ void __launch_bounds__(256)
colsum_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, long long rows,
              long long n, int rows_per_cta) {
  const int b = blockIdx.z;
  const long long chunk = static_cast<long long>(blockIdx.x) * 32 + (threadIdx.x & 31);
  const int rlane = threadIdx.x >> 5;  // 0..7
  const long long r0 = static_cast<long long>(blockIdx.y) * rows_per_cta;
  const long long r1 = min(rows, r0 + rows_per_cta);
  __shared__ float red[8][32][8 + 1];
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const bool ok = chunk * 8 < n;
  if (ok) {
    const __nv_bfloat16* base = x + (static_cast<long long>(b) * rows) * n + chunk * 8;
    // Four independent 16-byte loads per thread and trip keep enough bytes in flight per SM.
    long long r = r0 + rlane;
    for (; r + 24 < r1; r += 32) {
      uint4 q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) q[u] = __ldg(reinterpret_cast<const uint4*>(base + (r + 8 * u) * n));
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float f[8];
        unpack8(q[u], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
    }
    for (; r < r1; r += 8) {
      float f[8];
      unpack8(__ldg(reinterpret_cast<const uint4*>(base + r * n)), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[rlane][threadIdx.x & 31][i] = acc[i];
  __syncthreads();
  if (rlane == 0 && ok) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) s += red[j][threadIdx.x & 31][i];
      atomicAdd(out + static_cast<long long>(b) * n + chunk * 8 + i, s);
    }
  }
}

// ----------------------------------------------------------------------------- patchify
// images fp32/bf16 NHWC (B, H, W, C) -> bf16 (B*gh*gw, ph*pw*C); one thread per output pair.
template <typename T>
__global__ void __launch_bounds__(256)
patchify_kernel(const T* __restrict__ img, __nv_bfloat16* __restrict__ out, long long total_pairs,
                int hh, int ww, int c, int ph, int pw, int gh, int gw) {
  const int pd = ph * pw * c;  // patch dim (even whenever pw*c is even)
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
       i < total_pairs; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = i * 2;
    const int col = static_cast<int>(e % pd);
    const long long prow = e / pd;
    const int gx = static_cast<int>(prow % gw);
    const int gy = static_cast<int>((prow / gw) % gh);
    const long long b = prow / (static_cast<long long>(gw) * gh);
    const int py = col / (pw * c);
    const int rem = col % (pw * c);  // (px, ch) contiguous in the image row
    const T* src = img + ((b * hh + (gy * ph + py)) * ww + gx * pw) * c + rem;
    const float a = static_cast<float>(src[0]), bb = static_cast<float>(src[1]);
    reinterpret_cast<uint32_t*>(out)[i] = pack_bf16x2(a, bb);
  }
}

}  // namespace vmoe

using namespace vmoe;

extern "C" int vmoe_layernorm_fwd(const void* x, const float* gamma, const float* beta, void* y,
                                  float* mean, float* rstd, int64_t rows, int64_t h, float eps,
                                  vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (rows == 0) return 0;
  if (h % 8 || h > 2048) {
    set_error("%s (code %d)", "layernorm: hidden size must be a multiple of 8 and <= 2048", 0);
    return -1;
  }
  const int threads = 256;
  auto xx = static_cast<const __nv_bfloat16*>(x);
  auto yy = static_cast<__nv_bfloat16*>(y);
  const int chunks = static_cast<int>(h / 8);
  if (chunks == 2 || chunks == 4 || chunks == 8 || chunks == 16) {
    // Short rows: several rows per warp.
    const long long warps = (rows * chunks + 31) / 32;
    const long long want = (warps * 32 + threads - 1) / threads;
    const int g = static_cast<int>(want < 148 * 8 ? want : 148 * 8);
    const RowMap cm{1, h, static_cast<int>(h)};
#define VMOE_LN_FWD_SMALL(L) layernorm_fwd_small_kernel<L><<<g, threads, 0, stream>>>( \
      xx, gamma, beta, yy, mean, rstd, rows, eps, cm, cm)
    if (chunks == 2) VMOE_LN_FWD_SMALL(2);
    else if (chunks == 4) VMOE_LN_FWD_SMALL(4);
    else if (chunks == 8) VMOE_LN_FWD_SMALL(8);
    else VMOE_LN_FWD_SMALL(16);
#undef VMOE_LN_FWD_SMALL
    return launch_status("layernorm_fwd");
  }
  const long long blocks = (rows * 32 + threads - 1) / threads;
  const int grid = static_cast<int>(blocks < 148 * 2 ? blocks : 148 * 2);
#define VMOE_LN_FWD(C) layernorm_fwd_kernel<C><<<grid, threads, 0, stream>>>( \
      xx, gamma, beta, yy, mean, rstd, rows, static_cast<int>(h), eps)
  if (chunks <= 32 * 3) VMOE_LN_FWD(3);
  else if (chunks <= 32 * 4) VMOE_LN_FWD(4);
  else if (chunks <= 32 * 5) VMOE_LN_FWD(5);
  else VMOE_LN_FWD(8);
#undef VMOE_LN_FWD
  return launch_status("layernorm_fwd");
}

// Number of CTAs the backward kernel uses for `rows` rows (callers size the scratch with it).
static bool ln_small(long long h) {
  const long long chunks = h / 8;
  return h % 8 == 0 && (chunks == 2 || chunks == 4 || chunks == 8 || chunks == 16);
}

static int ln_bwd_grid(long long rows, long long h = 768) {
  // Short rows pack 32 / (h / 8) rows into a warp.
  const long long warps = ln_small(h) ? (rows * (h / 8) + 31) / 32 : rows;
  const long long blocks = (warps * 32 + 127) / 128;
  const long long cap = 148 * 3;
  return static_cast<int>(blocks < cap ? blocks : cap);
}

extern "C" int64_t vmoe_layernorm_bwd_scratch_bytes(int64_t rows, int64_t h) {
  return static_cast<int64_t>(ln_bwd_grid(rows, h)) * 2 * h * sizeof(float);
}

namespace vmoe {
int layernorm_bwd_launch(const void* dy, const void* x, const float* gamma, const float* mean,
                         const float* rstd, const void* dres, void* dx, float* dgamma,
                         float* dbeta, float* scratch, int64_t rows, int64_t h,
                         cudaStream_t stream) {
  if (rows == 0) return 0;
  if (h % 8 || h > 2048) {
    set_error("%s (code %d)", "layernorm: hidden size must be a multiple of 8 and <= 2048", 0);
    return -1;
  }
  const bool want = dgamma != nullptr || dbeta != nullptr;
  if (want && scratch == nullptr) {
    set_error("%s (code %d)", "layernorm_bwd: scratch buffer required for dgamma/dbeta", 0);
    return -1;
  }
  const int threads = 128;
  const int grid = ln_bwd_grid(rows, h);
  const size_t smem = 4 * 2 * h * sizeof(float);  // one slice per warp (threads / 32 = 4)
  auto a = static_cast<const __nv_bfloat16*>(dy);
  auto b = static_cast<const __nv_bfloat16*>(x);
  auto r = static_cast<const __nv_bfloat16*>(dres);
  auto o = static_cast<__nv_bfloat16*>(dx);
  float* part = want ? scratch : nullptr;
  const int chunks = static_cast<int>(h / 8);
  if (ln_small(h)) {
    const RowMap cm{1, h, static_cast<int>(h)};
#define VMOE_LN_BWD_SMALL(L) layernorm_bwd_small_kernel<L><<<grid, threads, smem, stream>>>( \
      a, b, gamma, mean, rstd, r, o, part, rows, cm, cm, cm)
    if (chunks == 2) VMOE_LN_BWD_SMALL(2);
    else if (chunks == 4) VMOE_LN_BWD_SMALL(4);
    else if (chunks == 8) VMOE_LN_BWD_SMALL(8);
    else VMOE_LN_BWD_SMALL(16);
#undef VMOE_LN_BWD_SMALL
    if (want) {
      const int n = static_cast<int>(2 * h);
      ln_reduce_partials_kernel<<<(n + 31) / 32, 256, 0, stream>>>(part, grid, static_cast<int>(h),
                                                                    dgamma, dbeta);
    }
    return launch_status("layernorm_bwd");
  }
#define VMOE_LN_BWD(C) layernorm_bwd_kernel<C><<<grid, threads, smem, stream>>>( \
      a, b, gamma, mean, rstd, r, o, part, rows, static_cast<int>(h))
  if (chunks <= 32 * 3) VMOE_LN_BWD(3);
  else if (chunks <= 32 * 4) VMOE_LN_BWD(4);
  else if (chunks <= 32 * 5) VMOE_LN_BWD(5);
  else {
    cudaFuncSetAttribute(layernorm_bwd_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         4 * 2 * 2048 * static_cast<int>(sizeof(float)));
    VMOE_LN_BWD(8);
  }
#undef VMOE_LN_BWD
  if (want) {
    const int n = static_cast<int>(2 * h);
    ln_reduce_partials_kernel<<<(n + 31) / 32, 256, 0, stream>>>(part, grid, static_cast<int>(h),
                                                                  dgamma, dbeta);
  }
  return launch_status("layernorm_bwd");
}
}  // namespace vmoe

extern "C" int vmoe_layernorm_bwd(const void* dy, const void* x, const float* gamma,
                                  const float* mean, const float* rstd, const void* dres, void* dx,
                                  float* dgamma, float* dbeta, float* scratch, int64_t rows,
                                  int64_t h, vmoe_stream_t stream_) {
  return layernorm_bwd_launch(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, scratch, rows, h,
                              static_cast<cudaStream_t>(stream_));
}

extern "C" int vmoe_colsum_bf16(const void* x, float* out, int64_t batch, int64_t rows, int64_t n,
                                vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (rows == 0 || n == 0 || batch == 0) return 0;
  if (n % 8) {
    set_error("%s (code %d)", "colsum: n must be a multiple of 8", 0);
    return -1;
  }
  const long long chunks = n / 8;
  const unsigned gx = static_cast<unsigned>((chunks + 31) / 32);
  // Enough row slices to fill the machine, at least 64 rows each.
  // Measured on 100 864 rows: 4 CTAs per SM are best for 768 columns (45 us against 57 us with 8),
  // 6 for 2304 and 3072 columns (75 / 95 us against 88 / 112 us).
  static const int forced = [] {
    const char* e = getenv("VMOE_B200_COLSUM_CTAS_PER_SM");
    const int v = e ? atoi(e) : 0;
    return v >= 1 && v <= 16 ? v : 0;
  }();
  const int per_sm = forced ? forced : (n <= 1024 ? 4 : 6);
  long long slices = (148 * per_sm) / (static_cast<long long>(gx) * batch);
  if (slices < 1) slices = 1;
  long long rpc = (rows + slices - 1) / slices;
  if (rpc < 64) rpc = 64;
  const unsigned gy = static_cast<unsigned>((rows + rpc - 1) / rpc);
  dim3 grid(gx, gy, static_cast<unsigned>(batch));
  colsum_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), out, rows, n,
                                          static_cast<int>(rpc));
  return launch_status("colsum");
}

extern "C" int vmoe_patchify(const void* img, int32_t img_is_bf16, void* out, int64_t b, int64_t hh,
                             int64_t ww, int64_t c, int64_t ph, int64_t pw, vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long gh = hh / ph, gw = ww / pw;
  if ((pw * c) % 2) {
    set_error("%s (code %d)", "patchify: patch_width * channels must be even", 0);
    return -1;
  }
  const long long pairs = b * gh * gw * ph * pw * c / 2;
  if (pairs == 0) return 0;
  const int threads = 256;
  long long blocks = (pairs + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (img_is_bf16)
    patchify_kernel<__nv_bfloat16><<<static_cast<int>(blocks), threads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(img), static_cast<__nv_bfloat16*>(out), pairs,
        static_cast<int>(hh), static_cast<int>(ww), static_cast<int>(c), static_cast<int>(ph),
        static_cast<int>(pw), static_cast<int>(gh), static_cast<int>(gw));
  else
    patchify_kernel<float><<<static_cast<int>(blocks), threads, 0, stream>>>(
        static_cast<const float*>(img), static_cast<__nv_bfloat16*>(out), pairs,
        static_cast<int>(hh), static_cast<int>(ww), static_cast<int>(c), static_cast<int>(ph),
        static_cast<int>(pw), static_cast<int>(gh), static_cast<int>(gw));
  return launch_status("patchify");
}

// ------------------------------------------------------------------ embedding finalisation
// out[b, 0, :] = cls + pos[0] (if a class token is used) and out[b, c + t, :] = emb[b, t, :] +
// pos[c + t]: the class-token concatenation and the position-embedding add in one pass over
// the patch embeddings. One warp per output row.
__global__ void __launch_bounds__(256)
embed_finalize_kernel(const __nv_bfloat16* __restrict__ emb, const float* __restrict__ cls,
                      const float* __restrict__ pos, __nv_bfloat16* __restrict__ out,
                      long long batch, int tokens, int h, int has_cls) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int out_tokens = tokens + has_cls;
  const int chunks = h >> 3;
  for (long long row = warp; row < batch * out_tokens; row += nwarps) {
    const long long b = row / out_tokens;
    const int t = static_cast<int>(row - b * out_tokens);
    const bool is_cls = has_cls && t == 0;
    const uint4* src = is_cls ? nullptr
                              : reinterpret_cast<const uint4*>(
                                    emb + (b * tokens + (t - has_cls)) * static_cast<long long>(h));
    uint4* dst = reinterpret_cast<uint4*>(out + row * h);
    for (int ch = lane; ch < chunks; ch += 32) {
      float v[8];
      if (is_cls) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = cls ? __ldg(cls + ch * 8 + i) : 0.f;
      } else {
        unpack8(__ldg(src + ch), v);
      }
      if (pos != nullptr) {
        const float4 p0 = __ldg(reinterpret_cast<const float4*>(pos + static_cast<long long>(t) * h + ch * 8));
        const float4 p1 = __ldg(reinterpret_cast<const float4*>(pos + static_cast<long long>(t) * h + ch * 8) + 1);
        v[0] += p0.x; v[1] += p0.y; v[2] += p0.z; v[3] += p0.w;
        v[4] += p1.x; v[5] += p1.y; v[6] += p1.z; v[7] += p1.w;
      }
      dst[ch] = pack8(v);
    }
  }
}

extern "C" int vmoe_embed_finalize(const void* emb, const float* cls, const float* pos, void* out,
                                   int64_t batch, int64_t tokens, int64_t h, int has_cls,
                                   vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (batch * (tokens + (has_cls ? 1 : 0)) == 0) return 0;
  if (h % 8) {
    set_error("%s (code %d)", "embed_finalize: hidden size must be a multiple of 8", 0);
    return -1;
  }
  const long long rows = batch * (tokens + (has_cls ? 1 : 0));
  const long long blocks = (rows * 32 + 255) / 256;
  const int grid = static_cast<int>(blocks < 148 * 8 ? blocks : 148 * 8);
  embed_finalize_kernel<<<grid, 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(emb), cls, pos, static_cast<__nv_bfloat16*>(out), batch,
      static_cast<int>(tokens), static_cast<int>(h), has_cls ? 1 : 0);
  return launch_status("embed_finalize");
}

// ------------------------------------------------------------------ short rows inside packed tensors
// LayerNorm over rows of h = 16 / 32 / 64 / 128 elements that are laid out as blocks of `inner`
// consecutive rows, the blocks `*_outer` elements apart (e.g. the q slice of a packed
// (B, T, 3, H, D) projection: inner = H, outer = 3 * H * D).
extern "C" int vmoe_layernorm_fwd_strided(const void* x, const float* gamma, const float* beta,
                                          void* y, float* mean, float* rstd, int64_t rows,
                                          int64_t h, float eps, int64_t inner, int64_t x_outer,
                                          int64_t y_outer, vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (rows == 0) return 0;
  if (!ln_small(h) || inner < 1 || x_outer % 8 || y_outer % 8) {
    set_error("%s (code %d)", "layernorm_strided: h must be 16/32/64/128, outer strides % 8 == 0", 0);
    return -1;
  }
  const int threads = 256, chunks = static_cast<int>(h / 8);
  const long long warps = (rows * chunks + 31) / 32;
  const long long want = (warps * 32 + threads - 1) / threads;
  const int g = static_cast<int>(want < 148 * 8 ? want : 148 * 8);
  const RowMap xm{inner, x_outer, static_cast<int>(h)}, ym{inner, y_outer, static_cast<int>(h)};
  auto xx = static_cast<const __nv_bfloat16*>(x);
  auto yy = static_cast<__nv_bfloat16*>(y);
#define VMOE_LN_FWD_SMALL(L) layernorm_fwd_small_kernel<L><<<g, threads, 0, stream>>>( \
      xx, gamma, beta, yy, mean, rstd, rows, eps, xm, ym)
  if (chunks == 2) VMOE_LN_FWD_SMALL(2);
  else if (chunks == 4) VMOE_LN_FWD_SMALL(4);
  else if (chunks == 8) VMOE_LN_FWD_SMALL(8);
  else VMOE_LN_FWD_SMALL(16);
#undef VMOE_LN_FWD_SMALL
  return launch_status("layernorm_fwd_strided");
}

extern "C" int vmoe_layernorm_bwd_strided(const void* dy, const void* x, const float* gamma,
                                          const float* mean, const float* rstd, void* dx,
                                          float* dgamma, float* dbeta, float* scratch,
                                          int64_t rows, int64_t h, int64_t inner, int64_t dy_outer,
                                          int64_t x_outer, int64_t dx_outer,
                                          vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (rows == 0) return 0;
  if (!ln_small(h) || inner < 1 || dy_outer % 8 || x_outer % 8 || dx_outer % 8) {
    set_error("%s (code %d)", "layernorm_strided: h must be 16/32/64/128, outer strides % 8 == 0", 0);
    return -1;
  }
  const bool want = dgamma != nullptr || dbeta != nullptr;
  if (want && scratch == nullptr) {
    set_error("%s (code %d)", "layernorm_bwd_strided: scratch buffer required", 0);
    return -1;
  }
  const int threads = 128, chunks = static_cast<int>(h / 8);
  const int grid = ln_bwd_grid(rows, h);
  const size_t smem = 4 * 2 * h * sizeof(float);
  const int hh = static_cast<int>(h);
  const RowMap dym{inner, dy_outer, hh}, xm{inner, x_outer, hh}, dxm{inner, dx_outer, hh};
  auto a = static_cast<const __nv_bfloat16*>(dy);
  auto b = static_cast<const __nv_bfloat16*>(x);
  auto o = static_cast<__nv_bfloat16*>(dx);
  float* part = want ? scratch : nullptr;
#define VMOE_LN_BWD_SMALL(L) layernorm_bwd_small_kernel<L><<<grid, threads, smem, stream>>>( \
      a, b, gamma, mean, rstd, nullptr, o, part, rows, dym, xm, dxm)
  if (chunks == 2) VMOE_LN_BWD_SMALL(2);
  else if (chunks == 4) VMOE_LN_BWD_SMALL(4);
  else if (chunks == 8) VMOE_LN_BWD_SMALL(8);
  else VMOE_LN_BWD_SMALL(16);
#undef VMOE_LN_BWD_SMALL
  if (want) {
    const int n = static_cast<int>(2 * h);
    ln_reduce_partials_kernel<<<(n + 31) / 32, 256, 0, stream>>>(part, grid, hh, dgamma, dbeta);
  }
  return launch_status("layernorm_bwd_strided");
}

// ------------------------------------------------------------------ no-allocation LayerNorm backward
// Same computation as vmoe_layernorm_bwd, but the per-CTA partial sums of dgamma / dbeta live in
// the file-scope device array below instead of a caller-provided buffer, so the call allocates
// nothing. The array holds kLnStaticMaxCtas rows of 2 * kLnStaticMaxHidden floats (3.5 MiB);
// larger hidden sizes are rejected.
namespace {
constexpr int kLnStaticMaxCtas = 148 * 3;     // grid cap of the backward kernel
constexpr int kLnStaticMaxHidden = 1024;
constexpr int kLnStaticMaxDevices = 64;
static __device__ __align__(256) float g_ln_bwd_scratch[kLnStaticMaxCtas * 2 * kLnStaticMaxHidden];
// Per-device cache of the array's device address; atomic so that threads racing through the
// first call on a device publish and read the (identical) value safely.
std::atomic<float*> g_ln_bwd_scratch_ptr[kLnStaticMaxDevices];
}  // namespace

extern "C" int vmoe_layernorm_bwd_static(const void* dy, const void* x, const float* gamma,
                                         const float* mean, const float* rstd, const void* dres,
                                         void* dx, float* dgamma, float* dbeta, int64_t rows,
                                         int64_t h, vmoe_stream_t stream_) {
  if (h > kLnStaticMaxHidden) {
    set_error("%s (code %d)",
              "layernorm_bwd_static: hidden size above the static scratch limit of 1024",
              static_cast<int>(h));
    return -1;
  }
  if (ln_bwd_grid(rows, h) > kLnStaticMaxCtas) {
    set_error("%s (code %d)", "layernorm_bwd_static: grid above the static scratch limit", 0);
    return -1;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kLnStaticMaxDevices) {
    set_error("%s (code %d)", "layernorm_bwd_static: cannot identify the current device",
              static_cast<int>(e));
    return -5;
  }
  float* ptr = g_ln_bwd_scratch_ptr[dev].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    // One-time set-up per device: resolve the device address of the static array.
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_ln_bwd_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
      return -5;
    }
    g_ln_bwd_scratch_ptr[dev].store(ptr, std::memory_order_release);
  }
  return layernorm_bwd_launch(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, ptr, rows, h,
                              static_cast<cudaStream_t>(stream_));
}
