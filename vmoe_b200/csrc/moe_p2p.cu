// Expert-parallel token movement over NVLink peer memory, fused with the expert GEMMs through
// arrival counters instead of a separate all-to-all.
//
//  * push_rows: every rank gathers the rows routed to each expert and stores them straight
//    into the row buffer of the GPU that owns the expert (plain st.global to a peer pointer).
//    Work is cut into chunks of 128 consecutive destination rows; when a chunk is written the
//    CTA adds the number of rows to the arrival counter(s) of the destination GEMM tile(s)
//    with a system-scope release. The destination's GEMM (gemm_tcgen05.cu, `a_ready`) loads an
//    A tile as soon as its counter reaches epoch * rows, so the first expert GEMM overlaps
//    the transfer tile by tile. Destinations are visited own rank first, then rank-1, rank-2,
//    ... which is the order in which the consumers rotate through their source blocks.
//    The same kernel is the backward of combine (rows scaled by the gate, plus the gate
//    gradient <dy, y>).
//  * signal: after a GEMM whose epilogue stored its output tiles into a peer's buffer (TMA
//    stores to peer memory), bump that peer's "source s is done" counter.
//  * wait_counters: bounded device-side wait on such counters, recording a status bit on
//    timeout; used in front of the combine kernels.
//
// Stands in for the all-to-alls that the reference gets from GSPMD around its dispatch and
// combine einsums (vmoe/moe.py:488-519).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "moe_push.cuh"
#include "ptx_sm100.cuh"
#include "vmoe_api.h"

namespace vmoe {

void set_error(const char* fmt, const char* a, int code);

__device__ __forceinline__ void unpack8p(const uint4& q, float (&f)[8]) {
  float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z),
         d = unpack_bf16x2(q.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8p(const float (&f)[8]) {
  uint4 q;
  q.x = pack_bf16x2(f[0], f[1]);
  q.y = pack_bf16x2(f[2], f[3]);
  q.z = pack_bf16x2(f[4], f[5]);
  q.w = pack_bf16x2(f[6], f[7]);
  return q;
}

// 128 threads and at most 48 registers per thread: small enough to be co-resident with one
// 320-thread GEMM CTA on every SM, so a push on a side stream makes progress while an
// arrival-gated GEMM occupies all SMs.
constexpr int PUSH_THREADS = 128;
__global__ void __launch_bounds__(PUSH_THREADS)
push_rows_kernel(const PushParams p) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int chunks = p.h >> 3;
  const int block_rows = p.g * p.c;                        // rows per (expert, source rank)
  const int chunks_per_expert = (block_rows + PUSH_ROWS - 1) / PUSH_ROWS;
  const long long total = static_cast<long long>(p.e) * chunks_per_expert;
  for (long long w = blockIdx.x; w < total; w += gridDim.x) {
    // Work order: destination ranks rank, rank-1, ...; inside one destination its experts.
    const int per_dst = p.el * chunks_per_expert;
    const int di = static_cast<int>(w / per_dst);
    const int rem = static_cast<int>(w % per_dst);
    const int dst = (p.rank - di + p.ep) % p.ep;
    const int ee = dst * p.el + rem / chunks_per_expert;   // global expert
    const int j0 = (rem % chunks_per_expert) * PUSH_ROWS;  // first row of the chunk in the block
    const int nrows = min(PUSH_ROWS, block_rows - j0);
    __nv_bfloat16* dbase = reinterpret_cast<__nv_bfloat16*>(p.dst_base[ee]);
    for (int jj = warp; jj < nrows; jj += PUSH_THREADS / 32) {
      const int j = j0 + jj;
      const int gi = j / p.c, ci = j - gi * p.c;
      const int pair = __ldg(p.slot_pair + (static_cast<long long>(gi) * p.e + ee) * p.c + ci);
      uint4* dst_row = reinterpret_cast<uint4*>(dbase + static_cast<long long>(j) * p.h);
      if (pair < 0) {
        for (int ch = lane; ch < chunks; ch += 32) dst_row[ch] = make_uint4(0, 0, 0, 0);
        continue;
      }
      const int item = pair / p.k;
      const uint4* src = reinterpret_cast<const uint4*>(
          p.x + (static_cast<long long>(gi) * p.s + item) * p.h);
      if (p.weight == nullptr) {
        for (int ch = lane; ch < chunks; ch += 32) dst_row[ch] = __ldg(src + ch);
      } else {
        const long long pidx = static_cast<long long>(gi) * p.s * p.k + pair;
        const float wgt = __ldg(p.weight + pidx);
        const uint4* yb = p.ybuf_base
                              ? reinterpret_cast<const uint4*>(
                                    reinterpret_cast<const __nv_bfloat16*>(p.ybuf_base[ee]) +
                                    static_cast<long long>(j) * p.h)
                              : nullptr;
        float dot = 0.f;
        for (int ch = lane; ch < chunks; ch += 32) {
          float f[8];
          unpack8p(__ldg(src + ch), f);
          if (yb) {
            float y[8];
            unpack8p(__ldg(yb + ch), y);
#pragma unroll
            for (int i = 0; i < 8; ++i) dot += f[i] * y[i];
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] *= wgt;
          dst_row[ch] = pack8p(f);
        }
        if (p.dgate) {
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
          if (lane == 0) p.dgate[pidx] = dot;
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0 && p.flag_base != nullptr) {
      __threadfence_system();  // rows written by the whole CTA are visible system-wide first
      unsigned* flags = reinterpret_cast<unsigned*>(p.flag_base[ee]);
      const int r_lo = p.row0 + j0, r_hi = r_lo + nrows;  // rows inside the expert's buffer
      for (int t = r_lo / PUSH_ROWS; t * PUSH_ROWS < r_hi; ++t) {
        const int lo = max(r_lo, t * PUSH_ROWS), hi = min(r_hi, (t + 1) * PUSH_ROWS);
        asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(flags + t), "r"(hi - lo)
                     : "memory");
      }
    }
    __syncthreads();
  }
}

__global__ void signal_kernel(unsigned* flag, unsigned value) {
  __threadfence_system();
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}

// Waits until counters[i] >= target for all i < n (bounded); sets a status bit on timeout.
__global__ void wait_counters_kernel(const unsigned* counters, int n, unsigned target,
                                     unsigned* status, long long limit_cycles) {
  const int i = threadIdx.x;
  if (i >= n) return;
  const long long t0 = clock64();
  for (;;) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(counters + i) : "memory");
    if (static_cast<int>(v - target) >= 0) return;
    if (clock64() - t0 > limit_cycles) {
      if (status) atomicOr(status, kStatusTimeoutPeer);
      return;
    }
    __nanosleep(200);
  }
}

// The bulk-copy push (moe_push.cuh) as a kernel of its own: the body that the GEMM kernel runs in
// two extra warps of each of its CTAs, launched alone so that it can be tested and timed in
// isolation.
constexpr int PUSH_KERNEL_WARPS = 8;
__global__ void __launch_bounds__(PUSH_KERNEL_WARPS * 32)
push_rows_bulk_kernel(const PushParams p, unsigned* status) {
  extern __shared__ uint8_t push_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(push_smem_raw) + 127) &
                                             ~static_cast<uintptr_t>(127));
  const int warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  push_rows_ring(p, smem + warp * PUSH_RING_BYTES,
                 smem + nwarps * PUSH_RING_BYTES + warp * PUSH_META_BYTES,
                 threadIdx.x & 31, blockIdx.x * nwarps + warp, gridDim.x * nwarps, status);
}

struct SignalAddrs {
  unsigned* f[16];
};
__global__ void signal_multi_kernel(const SignalAddrs a, int n, unsigned value) {
  __threadfence_system();
  if (threadIdx.x < n)
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(a.f[threadIdx.x]), "r"(value)
                 : "memory");
}

int fill_push_params(const VmoePushArgs* a, PushParams* p) {
  if (a->h % 8 || a->e != a->experts_per_rank * a->ep) {
    set_error("%s (code %d)", "push_rows: need h % 8 == 0 and e == experts_per_rank * ep", 0);
    return -1;
  }
  p->x = static_cast<const __nv_bfloat16*>(a->x);
  p->slot_pair = a->slot_pair;
  p->weight = a->weight;
  p->dst_base = reinterpret_cast<const unsigned long long*>(a->dst_base);
  p->flag_base = reinterpret_cast<const unsigned long long*>(a->flag_base);
  p->ybuf_base = reinterpret_cast<const unsigned long long*>(a->ybuf_base);
  p->dgate = a->dgate;
  p->g = static_cast<int>(a->groups);
  p->s = static_cast<int>(a->s);
  p->e = static_cast<int>(a->e);
  p->c = static_cast<int>(a->c);
  p->k = static_cast<int>(a->k);
  p->h = static_cast<int>(a->h);
  p->el = static_cast<int>(a->experts_per_rank);
  p->ep = static_cast<int>(a->ep);
  p->rank = static_cast<int>(a->rank);
  p->row0 = static_cast<int>(a->rank * a->groups * a->c);
  return 0;
}

}  // namespace vmoe

using namespace vmoe;

extern "C" int vmoe_moe_push_rows(const void* x, const int32_t* slot_pair, const float* weight,
                                  const uint64_t* dst_base, const uint64_t* flag_base,
                                  const uint64_t* ybuf_base, float* dgate, int64_t groups,
                                  int64_t s, int64_t e, int64_t c, int64_t k, int64_t h,
                                  int64_t experts_per_rank, int64_t ep, int64_t rank,
                                  vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (groups * e * c == 0) return 0;
  if (h % 8 || e != experts_per_rank * ep) {
    set_error("%s (code %d)", "push_rows: need h % 8 == 0 and e == experts_per_rank * ep", 0);
    return -1;
  }
  PushParams p;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.slot_pair = slot_pair;
  p.weight = weight;
  p.dst_base = reinterpret_cast<const unsigned long long*>(dst_base);
  p.flag_base = reinterpret_cast<const unsigned long long*>(flag_base);
  p.ybuf_base = reinterpret_cast<const unsigned long long*>(ybuf_base);
  p.dgate = dgate;
  p.g = static_cast<int>(groups);
  p.s = static_cast<int>(s);
  p.e = static_cast<int>(e);
  p.c = static_cast<int>(c);
  p.k = static_cast<int>(k);
  p.h = static_cast<int>(h);
  p.el = static_cast<int>(experts_per_rank);
  p.ep = static_cast<int>(ep);
  p.rank = static_cast<int>(rank);
  p.row0 = static_cast<int>(rank * groups * c);
  const long long block_rows = groups * c;
  const long long total = e * ((block_rows + PUSH_ROWS - 1) / PUSH_ROWS);
  const int grid = static_cast<int>(total < 148 * 8 ? total : 148 * 8);
  push_rows_kernel<<<grid, PUSH_THREADS, 0, stream>>>(p);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("%s (code %d)", cudaGetErrorString(err), static_cast<int>(err));
    return -5;
  }
  return 0;
}

extern "C" int vmoe_signal(uint32_t* flag, uint32_t value, vmoe_stream_t stream_) {
  signal_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream_)>>>(flag, value);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("%s (code %d)", cudaGetErrorString(err), static_cast<int>(err));
    return -5;
  }
  return 0;
}

extern "C" int vmoe_wait_counters(const uint32_t* counters, int32_t n, uint32_t target,
                                  uint32_t* status, int64_t limit_cycles, vmoe_stream_t stream_) {
  if (n <= 0) return 0;
  if (n > 1024) {
    set_error("%s (code %d)", "wait_counters: at most 1024 counters", 0);
    return -1;
  }
  wait_counters_kernel<<<1, n, 0, static_cast<cudaStream_t>(stream_)>>>(
      counters, n, target, status, limit_cycles > 0 ? limit_cycles : kWaitLimitCycles);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("%s (code %d)", cudaGetErrorString(err), static_cast<int>(err));
    return -5;
  }
  return 0;
}

extern "C" int32_t vmoe_moe_push_bulk_supported(int64_t h, int32_t with_gate_gradient) {
  return push_rows_per_slot(static_cast<int>(h), with_gate_gradient != 0) >= 1 ? 1 : 0;
}

extern "C" int vmoe_moe_push_rows_bulk(const VmoePushArgs* a, int32_t ctas, uint32_t* status,
                                       vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->groups * a->e * a->c == 0) return 0;
  PushParams p;
  int rc = fill_push_params(a, &p);
  if (rc) return rc;
  if (push_rows_per_slot(p.h, p.weight != nullptr && p.ybuf_base != nullptr) < 1) {
    set_error("%s (code %d)", "push_rows_bulk: rows too long for the shared-memory ring", p.h);
    return -1;
  }
  const int smem = PUSH_KERNEL_WARPS * (PUSH_RING_BYTES + PUSH_META_BYTES) + 128;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(push_rows_bulk_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
      set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
      return -4;
    }
    attr_set = true;
  }
  if (ctas <= 0) ctas = 37;
  int warps = PUSH_KERNEL_WARPS;
  if (const char* w = getenv("VMOE_B200_PUSH_KERNEL_WARPS")) {  // 1..8, for timing experiments
    const int v = atoi(w);
    if (v >= 1 && v <= PUSH_KERNEL_WARPS) warps = v;
  }
  push_rows_bulk_kernel<<<ctas, warps * 32, smem, stream>>>(p, status);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("%s (code %d)", cudaGetErrorString(err), static_cast<int>(err));
    return -5;
  }
  return 0;
}

// The plain (SIMT) push as a launch for callers inside the library (the GEMM falls back to it
// when the fused form does not apply).
namespace vmoe {
int launch_push_rows_plain(const PushParams& p, cudaStream_t stream) {
  const long long block_rows = static_cast<long long>(p.g) * p.c;
  const long long total = p.e * ((block_rows + PUSH_ROWS - 1) / PUSH_ROWS);
  if (total <= 0) return 0;
  const int grid = static_cast<int>(total < 148 * 8 ? total : 148 * 8);
  push_rows_kernel<<<grid, PUSH_THREADS, 0, stream>>>(p);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("%s (code %d)", cudaGetErrorString(err), static_cast<int>(err));
    return -5;
  }
  return 0;
}
}  // namespace vmoe

extern "C" int vmoe_signal_multi(const uint64_t* flags, int32_t n, uint32_t value,
                                 vmoe_stream_t stream_) {
  if (n <= 0) return 0;
  if (n > 16) {
    set_error("%s (code %d)", "signal_multi: at most 16 flags", n);
    return -1;
  }
  SignalAddrs a;
  for (int i = 0; i < 16; ++i) a.f[i] = i < n ? reinterpret_cast<unsigned*>(flags[i]) : nullptr;
  signal_multi_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_)>>>(a, n, value);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("%s (code %d)", cudaGetErrorString(err), static_cast<int>(err));
    return -5;
  }
  return 0;
}
