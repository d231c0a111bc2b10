// Routing and token-movement kernels of the sparse MoE layer.
//
//  * routing_plan: per group (one CTA), Top-K experts per item, optional Batch Priority
//    ordering (items served by decreasing top-1 gate, ties by index), K-major buffer positions
//    per expert, and the inverse map slot -> (item, choice). Indices form only: the
//    (S, E, C) one-hot tensors of the reference (vmoe/moe.py:547-623) are never built.
//  * gather_rows: expert-buffer rows <- item rows (dispatch; also the backward of combine).
//    The destination of every expert is a base pointer, so the same kernel writes a local
//    buffer or straight into a peer GPU's buffer over NVLink.
//  * combine_rows: item row <- residual + sum_k w_k * expert-buffer row (combine; also the
//    backward of dispatch with unit weights).
//  * combine_bwd: one pass per buffer row producing d(buffer row) = gate * dy[item] and the
//    gate gradient <dy[item], y_row>.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx_sm100.cuh"
#include "vmoe_api.h"

namespace vmoe {

void set_error(const char* fmt, const char* a, int code);

static inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
    return -5;
  }
  return 0;
}

__device__ __forceinline__ void unpack8f(const uint4& q, float (&f)[8]) {
  float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z),
         d = unpack_bf16x2(q.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8f(const float (&f)[8]) {
  uint4 q;
  q.x = pack_bf16x2(f[0], f[1]);
  q.y = pack_bf16x2(f[2], f[3]);
  q.z = pack_bf16x2(f[4], f[5]);
  q.w = pack_bf16x2(f[6], f[7]);
  return q;
}

// ----------------------------------------------------------------------------- routing plan
constexpr int PLAN_THREADS = 1024;
constexpr int PLAN_MAX_K = 8;

// smem: keys[npow2] (u64) | sorted_expert[K*S] (u16) | sorted_item[S] (i32)
__global__ void __launch_bounds__(PLAN_THREADS)
routing_plan_kernel(const float* __restrict__ gates, int* __restrict__ expert_out,
                    int* __restrict__ slot_out, int* __restrict__ slot_pair, int s, int e, int k,
                    int capacity, int batch_priority, int npow2) {
  extern __shared__ __align__(16) uint8_t plan_smem[];
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(plan_smem);
  unsigned short* sorted_expert = reinterpret_cast<unsigned short*>(keys + npow2);
  int* sorted_item = reinterpret_cast<int*>(sorted_expert + ((k * s + 1) & ~1));
  const int g = blockIdx.x;
  const float* gg = gates + static_cast<long long>(g) * s * e;
  int* eo = expert_out + static_cast<long long>(g) * s * k;
  int* so = slot_out + static_cast<long long>(g) * s * k;
  int* sp = slot_pair + static_cast<long long>(g) * e * capacity;
  const int tid = threadIdx.x;

  for (int i = tid; i < e * capacity; i += PLAN_THREADS) sp[i] = -1;

  // 1. Top-K per item (ties -> lowest expert index), sort key from the top-1 gate.
  for (int i = tid; i < npow2; i += PLAN_THREADS) {
    unsigned long long key = ~0ull;  // padding sorts last
    if (i < s) {
      const float* row = gg + static_cast<long long>(i) * e;
      int chosen[PLAN_MAX_K];
      float top1 = 0.f;
      for (int kk = 0; kk < k; ++kk) {
        float best = -INFINITY;
        int bi = 0;
        for (int j = 0; j < e; ++j) {
          bool taken = false;
          for (int t = 0; t < kk; ++t) taken |= (chosen[t] == j);
          const float v = __ldg(row + j);
          if (!taken && v > best) {
            best = v;
            bi = j;
          }
        }
        chosen[kk] = bi;
        eo[i * k + kk] = bi;
        if (kk == 0) top1 = best;
      }
      if (batch_priority) {
        // Descending gate, ascending index: gates are non-negative so their bit patterns are
        // monotone; -0.0 is canonicalised to +0.0.
        unsigned bits = __float_as_uint(top1 + 0.0f);
        if (top1 < 0.f) bits = 0u;
        key = (static_cast<unsigned long long>(0xFFFFFFFFu - bits) << 32) |
              static_cast<unsigned>(i);
      } else {
        key = static_cast<unsigned>(i);
      }
    }
    keys[i] = key;
  }
  __syncthreads();

  // 2. Bitonic sort of the keys (a total order, so the result equals a stable sort).
  if (batch_priority) {
    for (int size = 2; size <= npow2; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        for (int i = tid; i < (npow2 >> 1); i += PLAN_THREADS) {
          const int lo = 2 * i - (i & (stride - 1));
          const int hi = lo + stride;
          const bool up = (lo & size) == 0;
          const unsigned long long a = keys[lo], b = keys[hi];
          if ((a > b) == up) {
            keys[lo] = b;
            keys[hi] = a;
          }
        }
        __syncthreads();
      }
    }
  }
  for (int j = tid; j < s; j += PLAN_THREADS) {
    const int item = static_cast<int>(keys[j] & 0xFFFFFFFFu);
    sorted_item[j] = item;
    for (int kk = 0; kk < k; ++kk)
      sorted_expert[kk * s + j] = static_cast<unsigned short>(eo[item * k + kk]);
  }
  __syncthreads();

  // 3. K-major positions: warp w scans the served sequence for experts w, w+32, ...
  const int warp = tid >> 5, lane = tid & 31;
  const int total = k * s;
  for (int ex = warp; ex < e; ex += PLAN_THREADS / 32) {
    int base = 0;
    for (int j0 = 0; j0 < total; j0 += 32) {
      const int j = j0 + lane;
      const bool mine = j < total && sorted_expert[j] == ex;
      const unsigned m = __ballot_sync(0xffffffffu, mine);
      if (mine) {
        const int pos = base + __popc(m & ((1u << lane) - 1u));
        const int kk = j / s, item = sorted_item[j - kk * s];
        so[item * k + kk] = pos;
        if (pos < capacity) sp[ex * capacity + pos] = item * k + kk;
      }
      base += __popc(m);
    }
  }
}

// ----------------------------------------------------------------------------- row movement
// One warp per destination row. rows are indexed r = (g * E + e) * C + c.
// dst row address = expert_base[e] + (g * C + c) * h.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ slot_pair,
                   const float* __restrict__ weight, unsigned long long const* __restrict__ expert_base,
                   long long num_rows, int s, int e, int c, int k, int h) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int chunks = h >> 3;
  for (long long r = warp; r < num_rows; r += nwarps) {
    const int cc = static_cast<int>(r % c);
    const int ee = static_cast<int>((r / c) % e);
    const long long g = r / (static_cast<long long>(c) * e);
    const int pair = __ldg(slot_pair + r);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(expert_base[ee]) +
                                          (g * c + cc) * h);
    if (pair < 0) {
      for (int ch = lane; ch < chunks; ch += 32) dst[ch] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const int item = pair / k;
    const uint4* src = reinterpret_cast<const uint4*>(x + (g * s + item) * h);
    if (weight) {
      const float w = __ldg(weight + g * s * k + pair);
      for (int ch = lane; ch < chunks; ch += 32) {
        float f[8];
        unpack8f(__ldg(src + ch), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] *= w;
        dst[ch] = pack8f(f);
      }
    } else {
      for (int ch = lane; ch < chunks; ch += 32) dst[ch] = __ldg(src + ch);
    }
  }
}

// out[g, item] = residual[g, item] + sum_k [slot_k < C] w_k * buf[e_k][g*C + slot_k]
__global__ void __launch_bounds__(256)
combine_rows_kernel(unsigned long long const* __restrict__ expert_base,
                    const int* __restrict__ expert_idx, const int* __restrict__ slot,
                    const float* __restrict__ weight, const __nv_bfloat16* __restrict__ residual,
                    __nv_bfloat16* __restrict__ out, long long num_items, int s, int e, int c,
                    int k, int h, unsigned* status) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int chunks = h >> 3;
  for (long long t = warp; t < num_items; t += nwarps) {
    const long long g = t / s;
    for (int ch0 = 0; ch0 < chunks; ch0 += 32) {
      const int ch = ch0 + lane;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (ch < chunks && residual)
        unpack8f(__ldg(reinterpret_cast<const uint4*>(residual + t * h) + ch), acc);
      for (int kk = 0; kk < k; ++kk) {
        const int pos = __ldg(slot + t * k + kk);
        const int ee = __ldg(expert_idx + t * k + kk);
        if (pos < 0 || pos >= c) continue;
        if (ee < 0 || ee >= e) {
          if (status && lane == 0) atomicOr(status, kStatusBadIndex);
          continue;
        }
        const float w = weight ? __ldg(weight + t * k + kk) : 1.0f;
        if (ch < chunks) {
          const uint4* src = reinterpret_cast<const uint4*>(
              reinterpret_cast<const __nv_bfloat16*>(expert_base[ee]) + (g * c + pos) * h);
          float f[8];
          unpack8f(__ldg(src + ch), f);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += w * f[i];
        }
      }
      if (ch < chunks) reinterpret_cast<uint4*>(out + t * h)[ch] = pack8f(acc);
    }
  }
}

// Per buffer row r = (g, e, c): dbuf_row = gate * dy[g, item]; dgate[g, pair] = <dy, ybuf_row>.
__global__ void __launch_bounds__(256)
combine_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const int* __restrict__ slot_pair,
                   const float* __restrict__ gate, unsigned long long const* __restrict__ ybuf_base,
                   unsigned long long const* __restrict__ dbuf_base, float* __restrict__ dgate,
                   long long num_rows, int s, int e, int c, int k, int h) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int chunks = h >> 3;
  for (long long r = warp; r < num_rows; r += nwarps) {
    const int cc = static_cast<int>(r % c);
    const int ee = static_cast<int>((r / c) % e);
    const long long g = r / (static_cast<long long>(c) * e);
    const int pair = __ldg(slot_pair + r);
    const long long off = (g * c + cc) * h;
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dbuf_base[ee]) + off);
    if (pair < 0) {
      for (int ch = lane; ch < chunks; ch += 32) dst[ch] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const int item = pair / k;
    const float w = __ldg(gate + g * s * k + pair);
    const uint4* src = reinterpret_cast<const uint4*>(dy + (g * s + item) * h);
    const uint4* yb = reinterpret_cast<const uint4*>(
        reinterpret_cast<const __nv_bfloat16*>(ybuf_base[ee]) + off);
    float dot = 0.f;
    for (int ch = lane; ch < chunks; ch += 32) {
      float f[8], y[8];
      unpack8f(__ldg(src + ch), f);
      unpack8f(__ldg(yb + ch), y);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        dot += f[i] * y[i];
        f[i] *= w;
      }
      dst[ch] = pack8f(f);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane == 0) dgate[g * s * k + pair] = dot;
  }
}

static int warp_grid(long long rows) {
  long long blocks = (rows * 32 + 255) / 256;
  const long long cap = 148 * 16;
  return static_cast<int>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace vmoe

using namespace vmoe;

extern "C" int vmoe_routing_plan(const float* gates, int32_t* expert_out, int32_t* slot_out,
                                 int32_t* slot_pair, int64_t groups, int64_t s, int64_t e,
                                 int64_t k, int64_t capacity, int32_t batch_priority,
                                 vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (groups == 0) return 0;
  if (k > PLAN_MAX_K || k > e || e > 65535 || s > 16384) {
    set_error("%s (code %d)", "routing_plan: need k <= 8, k <= e, s <= 16384", 0);
    return -1;
  }
  int npow2 = 1;
  while (npow2 < s) npow2 <<= 1;
  const size_t smem = static_cast<size_t>(npow2) * 8 + ((k * s + 1) & ~1) * 2 + s * 4 + 16;
  static size_t smem_set = 0;
  if (smem > 48 * 1024 && smem > smem_set) {
    cudaError_t err = cudaFuncSetAttribute(routing_plan_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem));
    if (err != cudaSuccess) {
      set_error("%s (code %d)", cudaGetErrorString(err), static_cast<int>(err));
      return -4;
    }
    smem_set = smem;
  }
  routing_plan_kernel<<<static_cast<unsigned>(groups), PLAN_THREADS, smem, stream>>>(
      gates, expert_out, slot_out, slot_pair, static_cast<int>(s), static_cast<int>(e),
      static_cast<int>(k), static_cast<int>(capacity), batch_priority, npow2);
  return launch_status();
}

extern "C" int vmoe_moe_gather_rows(const void* x, const int32_t* slot_pair, const float* weight,
                                    const uint64_t* expert_base, int64_t groups, int64_t s,
                                    int64_t e, int64_t c, int64_t k, int64_t h,
                                    vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long rows = groups * e * c;
  if (rows == 0) return 0;
  if (h % 8) {
    set_error("%s (code %d)", "moe rows: hidden size must be a multiple of 8", 0);
    return -1;
  }
  gather_rows_kernel<<<warp_grid(rows), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), slot_pair, weight,
      reinterpret_cast<const unsigned long long*>(expert_base), rows, static_cast<int>(s),
      static_cast<int>(e), static_cast<int>(c), static_cast<int>(k), static_cast<int>(h));
  return launch_status();
}

extern "C" int vmoe_moe_combine_rows(const uint64_t* expert_base, const int32_t* expert_idx,
                                     const int32_t* slot, const float* weight, const void* residual,
                                     void* out, int64_t groups, int64_t s, int64_t e, int64_t c,
                                     int64_t k, int64_t h, uint32_t* status,
                                     vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long items = groups * s;
  if (items == 0) return 0;
  if (h % 8) {
    set_error("%s (code %d)", "moe rows: hidden size must be a multiple of 8", 0);
    return -1;
  }
  combine_rows_kernel<<<warp_grid(items), 256, 0, stream>>>(
      reinterpret_cast<const unsigned long long*>(expert_base), expert_idx, slot, weight,
      static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(out), items,
      static_cast<int>(s), static_cast<int>(e), static_cast<int>(c), static_cast<int>(k),
      static_cast<int>(h), status);
  return launch_status();
}

extern "C" int vmoe_moe_combine_bwd(const void* dy, const int32_t* slot_pair, const float* gate,
                                    const uint64_t* ybuf_base, const uint64_t* dbuf_base,
                                    float* dgate, int64_t groups, int64_t s, int64_t e, int64_t c,
                                    int64_t k, int64_t h, vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long rows = groups * e * c;
  if (rows == 0) return 0;
  if (h % 8) {
    set_error("%s (code %d)", "moe rows: hidden size must be a multiple of 8", 0);
    return -1;
  }
  combine_bwd_kernel<<<warp_grid(rows), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dy), slot_pair, gate,
      reinterpret_cast<const unsigned long long*>(ybuf_base),
      reinterpret_cast<const unsigned long long*>(dbuf_base), dgate, rows, static_cast<int>(s),
      static_cast<int>(e), static_cast<int>(c), static_cast<int>(k), static_cast<int>(h));
  return launch_status();
}

// ------------------------------------------------------------------ "experts choose" plan
// Every expert takes its `capacity` best items of the group (vmoe/moe.py:655-694,
// jax.lax.top_k over the items: larger gate first, lower item index first among equals).
// One CTA per (group, expert): the expert's column of gates is sorted in shared memory with a
// bitonic network on 64-bit keys (inverted gate bits, item index), then
//   slot_pair[g, e, c] = item * E + e   for the c-th best item (c < capacity),
//   slot[g, item, e]   = rank of the item in the expert's order, or `capacity` if not taken.
// In the indices form of the Top-K layer this is "K = E choices per item, choice j = expert j",
// so the row movers, the peer-memory exchange and the combine kernels are shared.
namespace vmoe {
constexpr int EC_MAX_ITEMS = 4096;

__global__ void __launch_bounds__(256)
experts_choose_plan_kernel(const float* __restrict__ gates, int* __restrict__ slot,
                           int* __restrict__ slot_pair, int s, int e, int capacity, int padded) {
  extern __shared__ unsigned long long ec_keys[];
  const int g = blockIdx.x / e, ee = blockIdx.x % e;
  const float* col = gates + (static_cast<long long>(g) * s) * e + ee;
  for (int i = threadIdx.x; i < padded; i += blockDim.x) {
    unsigned long long key = ~0ull;  // padding sorts last
    if (i < s) {
      const unsigned bits = __float_as_uint(col[static_cast<long long>(i) * e]);
      // gates are non-negative, so their bit patterns order like their values
      key = (static_cast<unsigned long long>(0xFFFFFFFFu - bits) << 32) | static_cast<unsigned>(i);
    }
    ec_keys[i] = key;
  }
  __syncthreads();
  for (int size = 2; size <= padded; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < (padded >> 1); t += blockDim.x) {
        const int lo = 2 * t - (t & (stride - 1));
        const int hi = lo + stride;
        const bool ascending = (lo & size) == 0;
        const unsigned long long a = ec_keys[lo], b = ec_keys[hi];
        if ((a > b) == ascending) {
          ec_keys[lo] = b;
          ec_keys[hi] = a;
        }
      }
      __syncthreads();
    }
  }
  for (int r = threadIdx.x; r < s; r += blockDim.x) {
    const int item = static_cast<int>(ec_keys[r] & 0xFFFFFFFFu);
    slot[(static_cast<long long>(g) * s + item) * e + ee] = r < capacity ? r : capacity;
    if (r < capacity)
      slot_pair[(static_cast<long long>(g) * e + ee) * capacity + r] = item * e + ee;
  }
  // capacity > s: the remaining buffer slots stay empty
  for (int r = s + threadIdx.x; r < capacity; r += blockDim.x)
    slot_pair[(static_cast<long long>(g) * e + ee) * capacity + r] = -1;
}
}  // namespace vmoe

extern "C" int vmoe_experts_choose_plan(const float* gates, int32_t* slot_out, int32_t* slot_pair,
                                        int64_t groups, int64_t s, int64_t e, int64_t capacity,
                                        vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (groups * s * e == 0) return 0;
  if (s > EC_MAX_ITEMS) {
    set_error("%s (code %d)", "experts_choose_plan: at most 4096 items per group", 0);
    return -1;
  }
  int padded = 2;
  while (padded < s) padded <<= 1;
  experts_choose_plan_kernel<<<static_cast<unsigned>(groups * e), 256, padded * 8, stream>>>(
      gates, slot_out, slot_pair, static_cast<int>(s), static_cast<int>(e),
      static_cast<int>(capacity), padded);
  return launch_status();
}
