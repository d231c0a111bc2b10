// Softmax attention specialised for the training shape of ViT-S/B/L: self-attention on packed
// QKV, head dim 64, up to 256 tokens, no dropout. One CTA per (batch, head, 128-query tile) in
// the forward pass and per (batch, head) in the backward pass, everything of a head resident in
// shared memory and TMEM. attention_tcgen05.cu covers every other shape with persistent,
// key-blocked kernels; for this shape the one-shot kernels below are the faster of the two
// (measured: 317 / 920 us against 397 / 1180 us forward / backward at B=512, T=197, H=12), so
// vmoe_attention_fwd / vmoe_attention_bwd route it here.
//
// Forward: TMA loads Q, K, V (128B-swizzled); S = Q K^T goes to TMEM; four warps (one query row
// per thread) compute the masked softmax from TMEM and write P as a bf16 UMMA operand to shared
// memory; O = P V accumulates in TMEM (over the columns S used), is normalised and stored
// together with the row log-sum-exp.
//
// Backward: for each 128-key half and 128-query tile: S = Q K^T and dP = dO V^T (TMEM),
// P = exp(S - lse), dS = P (dP - delta) / sqrt(d) written to shared memory once and used as three
// UMMA operands: dV += P^T dO, dK += dS^T Q (MN-major A) and dQ += dS K (K-major A).
//
// Replaces the reference's flax MultiHeadDotProductAttention (vmoe/nn/vit_moe.py:165-173).
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "ptx_sm100.cuh"
#include "tma_host.h"
#include "vmoe_api.h"

namespace vmoe {

void set_error(const char* fmt, const char* a, int code);

namespace d64 {

constexpr int ATT_D = 64;            // head dim
constexpr int ATT_ROW_BYTES = 128;   // 64 bf16
constexpr int ATT_TILE = 128;        // query rows per tile / key rows per half
constexpr int ATT_TILE_BYTES = ATT_TILE * ATT_ROW_BYTES;  // 16 KiB
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* desc, uint32_t bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cta.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1), "r"(c2),
        "r"(c3)
      : "memory");
}

#ifdef ATT_TRACE
// Timing probes of the backward kernel (builds with -DATT_TRACE only): the CTA of batch 0, head 0
// records clock64 at tagged points; vmoe_attention_d64_trace_read returns them. Tags, softmax
// warp: 0 rows' delta / lse loaded, 1 S and dP of a step have arrived, 2 P and dS written, 3 the
// step's products have retired (end of a key half), 4 dV / dK stored, 5 dQ stored; MMA thread:
// 0 operands in shared memory, 1 S / dP issued, 2 P / dS arrived, 3 dV / dK / dQ products issued.
__device__ long long g_d64_trace[2][4096];
__device__ int g_d64_trace_n[2];
#define D64_STAMP(who, tag)                                                                  \
  do {                                                                                       \
    if (blockIdx.x == 0 && blockIdx.y == 0 && lane == 0 && g_d64_trace_n[who] < 2040) {     \
      const int i_ = g_d64_trace_n[who]++;                                                   \
      g_d64_trace[who][2 * i_] = (tag);                                                      \
      g_d64_trace[who][2 * i_ + 1] = clock64();                                              \
    }                                                                                        \
  } while (0)
#else
#define D64_STAMP(who, tag) do {} while (0)
#endif

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Bounded wait used by every role; on failure all roles fall through to the common exit.
#undef ATT_WAIT
#define ATT_WAIT(bar, parity, code)                                              \
  do {                                                                           \
    const bool got_ = mbar_wait((bar), (parity), abort_flag, status, (code));   \
    if (!got_) ok = false;                                                       \
  } while (0)

struct AttnParams {
  __nv_bfloat16* out;     // forward: (B, T, H, 64)
  float* lse;             // (B, H, T) natural-log sum-exp of scaled scores
  const __nv_bfloat16* o_in;  // backward: forward output
  __nv_bfloat16* dq;      // backward outputs, each addressed with the strides below
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  long long g_tok, g_head, g_batch;  // strides (elements) of dq/dk/dv
  long long o_tok, o_head, o_batch;  // strides (elements) of out / o_in / dO
  const __nv_bfloat16* d_out;        // backward: dO
  unsigned* status;
  int B, H, T;
  int BN;       // keys rounded up to a multiple of 16 (<= 256)
  float scale;  // 1 / sqrt(d)
};

// ================================================================================ forward
// smem: [V: BNx128B (<=32 KiB)] [P: 4 x 16 KiB, the first 16+32 KiB double as Q and K]
// Warp 0 loads and issues the MMAs; eight softmax warps, two threads per query row (a warp's TMEM
// lane quadrant is its index modulo 4): warps 1-4 take the even 32-key chunks of the row, warps
// 5-8 the odd ones, and the two exchange their partial row maximum and row sum through shared
// memory. Two CTAs share an SM, so every scheduler has four softmax warps to interleave.
constexpr int FWD_THREADS = 288;
constexpr int FWD_SOFTMAX_THREADS = 256;
constexpr int FWD_XCHG_BYTES = 2 * 2 * 128 * 4;  // [max | sum][half][row]
constexpr int FWD_SMEM = 32768 + 65536 + 1024 + 128 + FWD_XCHG_BYTES;

__global__ void __launch_bounds__(FWD_THREADS, 2)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                     const __grid_constant__ CUtensorMap tv, const AttnParams p) {
  extern __shared__ uint8_t att_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(att_smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sV = smem;
  uint8_t* sP = smem + 32768;  // P operand; before the softmax the same bytes hold Q and K
  uint8_t* sQ = sP;
  uint8_t* sK = sP + ATT_TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 32768 + 65536);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xchg = reinterpret_cast<float*>(smem + 32768 + 65536 + 128);
  unsigned* status = p.status;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const uint32_t bar_qk = smem_u32(bars), bar_v = smem_u32(bars + 1), bar_s = smem_u32(bars + 2),
                 bar_p = smem_u32(bars + 3), bar_o = smem_u32(bars + 4), bar_mx = smem_u32(bars + 5);
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_qk, 1);
    mbar_init(bar_v, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_p, FWD_SOFTMAX_THREADS);
    mbar_init(bar_o, 1);
    mbar_init(bar_mx, FWD_SOFTMAX_THREADS);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int BN = p.BN;
  bool ok = true;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar_qk, ATT_TILE_BYTES + BN * ATT_ROW_BYTES);
      tma_load_4d(smem_u32(sQ), &tq, bar_qk, 0, h, qt * ATT_TILE, b);
      tma_load_4d(smem_u32(sK), &tk, bar_qk, 0, h, 0, b);
      mbar_expect_tx(bar_v, BN * ATT_ROW_BYTES);
      tma_load_4d(smem_u32(sV), &tv, bar_v, 0, h, 0, b);
      ATT_WAIT(bar_qk, 0, kStatusTimeoutMma);
      if (ok) {
        tc_fence_after();
        const uint32_t idesc = umma_idesc_bf16(128, BN, 0, 0);
#pragma unroll
        for (int k = 0; k < ATT_D / 16; ++k)
          umma_bf16(tmem, umma_smem_desc(smem_u32(sQ) + k * 32, 16, 1024),
                    umma_smem_desc(smem_u32(sK) + k * 32, 16, 1024), idesc, k > 0);
        umma_commit(bar_s);
      }
      if (ok) ATT_WAIT(bar_p, 0, kStatusTimeoutMma);
      if (ok) ATT_WAIT(bar_v, 0, kStatusTimeoutMma);
      if (ok) {
        tc_fence_after();
        // O (128 x 64) = P (128 x BN, K-major) * V (BN x 64: N contiguous -> MN-major B).
        const uint32_t idesc = umma_idesc_bf16(128, ATT_D, 0, 1);
        for (int k = 0; k < BN / 16; ++k)
          umma_bf16(tmem,
                    umma_smem_desc(smem_u32(sP) + (k >> 2) * ATT_TILE_BYTES + (k & 3) * 32, 16, 1024),
                    umma_smem_desc(smem_u32(sV) + k * 2048, ATT_TILE_BYTES, 1024), idesc, k > 0);
        umma_commit(bar_o);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax / epilogue
    const int quad = warp & 3;
    const int half = (warp - 1) >> 2;      // 0: even 32-key chunks of the row, 1: odd ones
    const int r = quad * 32 + lane;        // row inside the query tile
    const int q = qt * ATT_TILE + r;       // query index
    const uint32_t trow = tmem + (static_cast<uint32_t>(quad * 32) << 16);
    const float sl2 = p.scale * kLog2e;
    const uint32_t rx = static_cast<uint32_t>(r) & 7u;
    float* xmax = xchg;            // [half][row]
    float* xsum = xchg + 2 * 128;  // [half][row]
    {
      const bool got = mbar_wait(bar_s, 0, abort_flag, status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, got);
    }
    float mx = -INFINITY, sum = 0.f;
    if (ok) {
      tc_fence_after();
      const int nchunk = (BN + 31) / 32;
      // Row maximum over this thread's chunks; the key bound is tested only where key T falls.
      for (int c = half; c < nchunk; c += 2) {
        uint32_t v[32];
        tmem_ld_32x32(trow + c * 32, v);
        tmem_ld_wait();
        const int valid = p.T - c * 32;
        if (valid >= 32) {
          float m0 = mx, m1 = mx, m2 = mx, m3 = mx;
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            m0 = max3(m0, __uint_as_float(v[i + 0]), __uint_as_float(v[i + 1]));
            m1 = max3(m1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
            m2 = max3(m2, __uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
            m3 = max3(m3, __uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
          }
          mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i < valid) mx = fmaxf(mx, __uint_as_float(v[i]));
        }
      }
      // The other thread of the row holds the maximum of the other chunks.
      xmax[half * 128 + r] = mx;
      mbar_arrive(bar_mx);
      const bool got = mbar_wait(bar_mx, 0, abort_flag, status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, got);
    }
    if (ok) {
      mx = fmaxf(mx, xmax[(half ^ 1) * 128 + r]);
      const float mxs = mx * sl2;
      const int nchunk = (BN + 31) / 32;
      const f32x2 sl = f2_pack(sl2, sl2), ms = f2_pack(-mxs, -mxs);
      for (int c = half; c < nchunk; c += 2) {
        uint32_t v[32];
        tmem_ld_32x32(trow + c * 32, v);
        tmem_ld_wait();
        float e[32];
        const int valid = p.T - c * 32;
        if (valid >= 32) {
          f32x2 s0 = f2_pack(0.f, 0.f), s1 = s0;
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float a0, a1, a2, a3;
            f2_unpack(f2_fma(f2_pack(__uint_as_float(v[i]), __uint_as_float(v[i + 1])), sl, ms), a0, a1);
            f2_unpack(f2_fma(f2_pack(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3])), sl, ms), a2,
                      a3);
            e[i] = exp2f(a0);
            e[i + 1] = exp2f(a1);
            e[i + 2] = exp2f(a2);
            e[i + 3] = exp2f(a3);
            s0 = f2_add(s0, f2_pack(e[i], e[i + 1]));
            s1 = f2_add(s1, f2_pack(e[i + 2], e[i + 3]));
          }
          float a0, a1;
          f2_unpack(f2_add(s0, s1), a0, a1);
          sum += a0 + a1;
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            e[i] = i < valid ? exp2f(__uint_as_float(v[i]) * sl2 - mxs) : 0.f;
            sum += e[i];
          }
        }
        // Row r of the 64-key chunk (c / 2): 16-byte units j = 4 * (c & 1) + i, 128B swizzle.
        uint8_t* base = sP + (c >> 1) * ATT_TILE_BYTES + r * ATT_ROW_BYTES;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 u;
          u.x = pack_bf16x2(e[8 * i + 0], e[8 * i + 1]);
          u.y = pack_bf16x2(e[8 * i + 2], e[8 * i + 3]);
          u.z = pack_bf16x2(e[8 * i + 4], e[8 * i + 5]);
          u.w = pack_bf16x2(e[8 * i + 6], e[8 * i + 7]);
          const uint32_t j = static_cast<uint32_t>(4 * (c & 1) + i);
          *reinterpret_cast<uint4*>(base + ((j ^ rx) << 4)) = u;
        }
      }
      xsum[half * 128 + r] = sum;  // visible to the row's other thread once bar_o completes
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(bar_p);
      const bool got = mbar_wait(bar_o, 0, abort_flag, status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, got);
    }
    if (ok) {
      tc_fence_after();
      sum += xsum[(half ^ 1) * 128 + r];
      const float inv = 1.0f / sum;
      __nv_bfloat16* orow = p.out + b * p.o_batch + static_cast<long long>(q) * p.o_tok + h * p.o_head;
      {
        const int c = half;  // 32 of the 64 output columns per thread
        uint32_t v[32];
        tmem_ld_32x32(trow + c * 32, v);
        tmem_ld_wait();
        if (q < p.T) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(v[8 * i + 0]) * inv, __uint_as_float(v[8 * i + 1]) * inv);
            u.y = pack_bf16x2(__uint_as_float(v[8 * i + 2]) * inv, __uint_as_float(v[8 * i + 3]) * inv);
            u.z = pack_bf16x2(__uint_as_float(v[8 * i + 4]) * inv, __uint_as_float(v[8 * i + 5]) * inv);
            u.w = pack_bf16x2(__uint_as_float(v[8 * i + 6]) * inv, __uint_as_float(v[8 * i + 7]) * inv);
            reinterpret_cast<uint4*>(orow + c * 32)[i] = u;
          }
        }
      }
      if (half == 0 && q < p.T && p.lse)
        p.lse[(static_cast<long long>(b) * p.H + h) * p.T + q] = mx * p.scale + __logf(sum);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

// ================================================================================ backward
// smem: Q, dO (2 tiles each), K, V (2 halves each): 8 x 16 KiB; P and dS: 2 x 16 KiB each.
constexpr int BWD_THREADS = 160;
constexpr int BWD_SMEM = 12 * ATT_TILE_BYTES + 1024 + 256;
constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DV = 256, TM_DK = 320, TM_DQ = 384;

__global__ void __launch_bounds__(BWD_THREADS, 1)
attention_bwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                     const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                     const AttnParams p) {
  extern __shared__ uint8_t att_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(att_smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;                         // 2 x 16 KiB (query tiles)
  uint8_t* sDO = smem + 2 * ATT_TILE_BYTES;   // 2 x 16 KiB
  uint8_t* sK = smem + 4 * ATT_TILE_BYTES;    // 2 x 16 KiB (key halves)
  uint8_t* sV = smem + 6 * ATT_TILE_BYTES;    // 2 x 16 KiB
  uint8_t* sP = smem + 8 * ATT_TILE_BYTES;    // 128 q x 128 keys bf16: 2 chunks of 16 KiB
  uint8_t* sDS = smem + 10 * ATT_TILE_BYTES;  // same layout
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 12 * ATT_TILE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  unsigned* status = p.status;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, b = blockIdx.y;
  const uint32_t bar_ld = smem_u32(bars), bar_s = smem_u32(bars + 1), bar_p = smem_u32(bars + 2),
                 bar_mma = smem_u32(bars + 3), bar_acc = smem_u32(bars + 4);
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_ld, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_p, 128);
    mbar_init(bar_mma, 1);
    mbar_init(bar_acc, 128);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int BN = p.BN, T = p.T;
  const int n_qt = (T + ATT_TILE - 1) / ATT_TILE;
  const int n_kh = (BN + ATT_TILE - 1) / ATT_TILE;
  bool ok = true;

  if (warp == 0) {
    if (lane == 0) {
      // Everything for this (batch, head) is loaded once: rows beyond T are zero filled.
      mbar_expect_tx(bar_ld, (2 * n_qt + 2 * n_kh) * ATT_TILE_BYTES);
      for (int i = 0; i < n_qt; ++i) {
        tma_load_4d(smem_u32(sQ + i * ATT_TILE_BYTES), &tq, bar_ld, 0, h, i * ATT_TILE, b);
        tma_load_4d(smem_u32(sDO + i * ATT_TILE_BYTES), &tdo, bar_ld, 0, h, i * ATT_TILE, b);
      }
      for (int i = 0; i < n_kh; ++i) {
        tma_load_4d(smem_u32(sK + i * ATT_TILE_BYTES), &tk, bar_ld, 0, h, i * ATT_TILE, b);
        tma_load_4d(smem_u32(sV + i * ATT_TILE_BYTES), &tv, bar_ld, 0, h, i * ATT_TILE, b);
      }
      ATT_WAIT(bar_ld, 0, kStatusTimeoutMma);
      D64_STAMP(1, 0);
      int it = 0;
      for (int kh = 0; kh < n_kh && ok; ++kh) {
        const int nk = min(ATT_TILE, BN - kh * ATT_TILE);  // keys in this half (multiple of 16)
        const uint32_t kbase = smem_u32(sK + kh * ATT_TILE_BYTES);
        const uint32_t vbase = smem_u32(sV + kh * ATT_TILE_BYTES);
        if (kh > 0) {
          // The epilogue warps must have drained dV/dK of the previous half.
          ATT_WAIT(bar_acc, (kh - 1) & 1, kStatusTimeoutMma);
          if (!ok) break;
        }
        for (int qt = 0; qt < n_qt && ok; ++qt, ++it) {
          const uint32_t qbase = smem_u32(sQ + qt * ATT_TILE_BYTES);
          const uint32_t dobase = smem_u32(sDO + qt * ATT_TILE_BYTES);
          // S/dP TMEM is free: the softmax warps arrived on bar_p (waited for below, in the
          // previous step) after their last TMEM read. No wait for the previous step's
          // dV/dK/dQ MMAs is needed before issuing: MMAs of one thread execute in order, so
          // the commit on bar_s below also covers them, and the softmax warps overwrite the
          // P/dS shared-memory tiles only after bar_s.
          tc_fence_after();
          const uint32_t id_s = umma_idesc_bf16(128, nk, 0, 0);
#pragma unroll
          for (int k = 0; k < ATT_D / 16; ++k)
            umma_bf16(tmem + TM_S, umma_smem_desc(qbase + k * 32, 16, 1024),
                      umma_smem_desc(kbase + k * 32, 16, 1024), id_s, k > 0);
#pragma unroll
          for (int k = 0; k < ATT_D / 16; ++k)
            umma_bf16(tmem + TM_DP, umma_smem_desc(dobase + k * 32, 16, 1024),
                      umma_smem_desc(vbase + k * 32, 16, 1024), id_s, k > 0);
          umma_commit(bar_s);
          D64_STAMP(1, 1);
          ATT_WAIT(bar_p, it & 1, kStatusTimeoutMma);
          D64_STAMP(1, 2);
          if (!ok) break;
          tc_fence_after();
          // dV[kh] += P^T dO, dK[kh] += dS^T Q: A read MN-major (M = keys), B MN-major (N = d).
          const uint32_t id_t = umma_idesc_bf16(128, ATT_D, 1, 1);
#pragma unroll
          for (int k = 0; k < ATT_TILE / 16; ++k)
            umma_bf16(tmem + TM_DV, umma_smem_desc(smem_u32(sP) + k * 2048, ATT_TILE_BYTES, 1024),
                      umma_smem_desc(dobase + k * 2048, ATT_TILE_BYTES, 1024), id_t,
                      (qt > 0 || k > 0));
#pragma unroll
          for (int k = 0; k < ATT_TILE / 16; ++k)
            umma_bf16(tmem + TM_DK, umma_smem_desc(smem_u32(sDS) + k * 2048, ATT_TILE_BYTES, 1024),
                      umma_smem_desc(qbase + k * 2048, ATT_TILE_BYTES, 1024), id_t,
                      (qt > 0 || k > 0));
          // dQ[qt] += dS K[kh]: A K-major (M = queries, K = keys), B MN-major.
          const uint32_t id_q = umma_idesc_bf16(128, ATT_D, 0, 1);
          for (int k = 0; k < nk / 16; ++k)
            umma_bf16(tmem + TM_DQ + qt * 64,
                      umma_smem_desc(smem_u32(sDS) + (k >> 2) * ATT_TILE_BYTES + (k & 3) * 32, 16, 1024),
                      umma_smem_desc(kbase + k * 2048, ATT_TILE_BYTES, 1024), id_q,
                      (kh > 0 || k > 0));
          umma_commit(bar_mma);
          D64_STAMP(1, 3);
        }
      }
      // Final: make sure the last MMAs retired before the epilogue reads dV/dK/dQ.
      if (ok) ATT_WAIT(bar_mma, (it - 1) & 1, kStatusTimeoutMma);
    }
  } else {
    // ---------------------------------------------------------------- softmax-backward warps
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t trow = tmem + (static_cast<uint32_t>(quad * 32) << 16);
    const float sl2 = p.scale * kLog2e;
    // delta = rowsum(dO * O) and lse for this thread's rows of both query tiles.
    float delta[2] = {0.f, 0.f}, lse2[2] = {0.f, 0.f};
    for (int qt = 0; qt < n_qt; ++qt) {
      const int q = qt * ATT_TILE + r;
      if (q < T) {
        const long long off = b * p.o_batch + static_cast<long long>(q) * p.o_tok + h * p.o_head;
        const uint4* a4 = reinterpret_cast<const uint4*>(p.d_out + off);
        const uint4* o4 = reinterpret_cast<const uint4*>(p.o_in + off);
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint4 x = __ldg(a4 + i), y = __ldg(o4 + i);
          const float2 x0 = unpack_bf16x2(x.x), x1 = unpack_bf16x2(x.y), x2 = unpack_bf16x2(x.z),
                       x3 = unpack_bf16x2(x.w);
          const float2 y0 = unpack_bf16x2(y.x), y1 = unpack_bf16x2(y.y), y2 = unpack_bf16x2(y.z),
                       y3 = unpack_bf16x2(y.w);
          acc += x0.x * y0.x + x0.y * y0.y + x1.x * y1.x + x1.y * y1.y + x2.x * y2.x +
                 x2.y * y2.y + x3.x * y3.x + x3.y * y3.y;
        }
        delta[qt] = acc;
        lse2[qt] = p.lse[(static_cast<long long>(b) * p.H + h) * T + q] * kLog2e;
      }
    }
    int it = 0;
    if (warp == 1) D64_STAMP(0, 0);
    for (int kh = 0; kh < n_kh && ok; ++kh) {
      const int nk = min(ATT_TILE, BN - kh * ATT_TILE);
      for (int qt = 0; qt < n_qt && ok; ++qt, ++it) {
        {
          const bool got = mbar_wait(bar_s, it & 1, abort_flag, status, kStatusTimeoutEpilogue);
          ok = __all_sync(0xffffffffu, got);
        }
        if (warp == 1) D64_STAMP(0, 1);
        if (!ok) break;
        tc_fence_after();
        const int q = qt * ATT_TILE + r;
        const bool qv = q < T;
        const float dl = delta[qt], ls = lse2[qt];
        for (int c = 0; c < (nk + 31) / 32; ++c) {
          uint32_t sv[32], dv[32];
          tmem_ld_32x32(trow + TM_S + c * 32, sv);
          tmem_ld_32x32(trow + TM_DP + c * 32, dv);
          tmem_ld_wait();
          float pe[32], de[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = kh * ATT_TILE + c * 32 + i;
            const bool v = qv && key < T;
            const float pr = v ? exp2f(__uint_as_float(sv[i]) * sl2 - ls) : 0.f;
            pe[i] = pr;
            de[i] = v ? pr * (__uint_as_float(dv[i]) - dl) * p.scale : 0.f;
          }
          const uint32_t off = (c >> 1) * ATT_TILE_BYTES + r * ATT_ROW_BYTES;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t j = static_cast<uint32_t>(4 * (c & 1) + i);
            const uint32_t sw = (j ^ (static_cast<uint32_t>(r) & 7u)) << 4;
            uint4 u;
            u.x = pack_bf16x2(pe[8 * i + 0], pe[8 * i + 1]);
            u.y = pack_bf16x2(pe[8 * i + 2], pe[8 * i + 3]);
            u.z = pack_bf16x2(pe[8 * i + 4], pe[8 * i + 5]);
            u.w = pack_bf16x2(pe[8 * i + 6], pe[8 * i + 7]);
            *reinterpret_cast<uint4*>(sP + off + sw) = u;
            u.x = pack_bf16x2(de[8 * i + 0], de[8 * i + 1]);
            u.y = pack_bf16x2(de[8 * i + 2], de[8 * i + 3]);
            u.z = pack_bf16x2(de[8 * i + 4], de[8 * i + 5]);
            u.w = pack_bf16x2(de[8 * i + 6], de[8 * i + 7]);
            *reinterpret_cast<uint4*>(sDS + off + sw) = u;
          }
        }
        // Key columns [nk, 128) of P^T / dS^T feed rows of dV / dK that are never stored, but
        // they must not hold NaN bit patterns that would poison nothing else; zero them once.
        if (it == 0 || nk < ATT_TILE) {
          for (int c = (nk + 31) / 32; c < 4; ++c) {
            const uint32_t off = (c >> 1) * ATT_TILE_BYTES + r * ATT_ROW_BYTES;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t j = static_cast<uint32_t>(4 * (c & 1) + i);
              const uint32_t sw = (j ^ (static_cast<uint32_t>(r) & 7u)) << 4;
              *reinterpret_cast<uint4*>(sP + off + sw) = make_uint4(0, 0, 0, 0);
              *reinterpret_cast<uint4*>(sDS + off + sw) = make_uint4(0, 0, 0, 0);
            }
          }
        }
        fence_proxy_async();
        tc_fence_before();
        mbar_arrive(bar_p);
        if (warp == 1) D64_STAMP(0, 2);
      }
      if (!ok) break;
      // dV / dK of this key half are complete once the last step's MMAs retire.
      {
        const bool got = mbar_wait(bar_mma, (it - 1) & 1, abort_flag, status, kStatusTimeoutEpilogue);
        ok = __all_sync(0xffffffffu, got);
      }
      if (!ok) break;
      if (warp == 1) D64_STAMP(0, 3);
      tc_fence_after();
      const int key = kh * ATT_TILE + r;
      const long long goff = b * p.g_batch + static_cast<long long>(key) * p.g_tok + h * p.g_head;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* dst = (which == 0 ? p.dv : p.dk) + goff;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(trow + (which == 0 ? TM_DV : TM_DK) + c * 32, v);
          tmem_ld_wait();
          if (key < T) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 u;
              u.x = pack_bf16x2(__uint_as_float(v[8 * i + 0]), __uint_as_float(v[8 * i + 1]));
              u.y = pack_bf16x2(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3]));
              u.z = pack_bf16x2(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5]));
              u.w = pack_bf16x2(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7]));
              reinterpret_cast<uint4*>(dst + c * 32)[i] = u;
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(bar_acc);
      if (warp == 1) D64_STAMP(0, 4);
    }
    if (ok) {
      // dQ of both query tiles (accumulated over the key halves).
      tc_fence_after();
      for (int qt = 0; qt < n_qt; ++qt) {
        const int q = qt * ATT_TILE + r;
        __nv_bfloat16* dst = p.dq + b * p.g_batch + static_cast<long long>(q) * p.g_tok + h * p.g_head;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(trow + TM_DQ + qt * 64 + c * 32, v);
          tmem_ld_wait();
          if (q < T) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 u;
              u.x = pack_bf16x2(__uint_as_float(v[8 * i + 0]), __uint_as_float(v[8 * i + 1]));
              u.y = pack_bf16x2(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3]));
              u.z = pack_bf16x2(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5]));
              u.w = pack_bf16x2(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7]));
              reinterpret_cast<uint4*>(dst + c * 32)[i] = u;
            }
          }
        }
      }
      if (warp == 1) D64_STAMP(0, 5);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------- host side
// (64, H, T, B) view of a bf16 tensor with element strides (1, head, tok, batch); a box is
// 64 x 1 x rows x 1, i.e. rows of one head, 128 bytes each.
static int make_head_map(CUtensorMap* map, const void* ptr, int64_t t, int64_t h, int64_t b,
                         int64_t tok, int64_t head, int64_t batch, uint32_t box_rows) {
  cuuint64_t dims[4] = {64, static_cast<cuuint64_t>(h), static_cast<cuuint64_t>(t),
                        static_cast<cuuint64_t>(b)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(head) * 2, static_cast<cuuint64_t>(tok) * 2,
                           static_cast<cuuint64_t>(batch) * 2};
  cuuint32_t box[4] = {64, 1, box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = tma_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr),
                                dims, strides, box, estr, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != CUDA_SUCCESS) {
    set_error("%s (code %d)", "cuTensorMapEncodeTiled (attention) failed", static_cast<int>(r));
    return -3;
  }
  return 0;
}

static int check_attn(const VmoeAttnArgs* a) {
  if (a->D != 64 || a->T < 1 || a->T > 256) {
    set_error("%s (code %d)", "attention kernel supports head_dim 64 and 1 <= T <= 256", 0);
    return -1;
  }
  const int64_t strides[] = {a->q_tok, a->q_head, a->q_batch, a->o_tok, a->o_head, a->o_batch};
  for (int64_t s : strides)
    if (s % 8) {
      set_error("%s (code %d)", "attention strides must be multiples of 8 elements", 0);
      return -1;
    }
  return 0;
}

}  // namespace d64
}  // namespace vmoe

using namespace vmoe;
using namespace vmoe::d64;

namespace vmoe {
int attention_d64_fwd(const VmoeAttnArgs* a, vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->B == 0 || a->H == 0) return 0;
  int rc = check_attn(a);
  if (rc) return rc;
  const int BN = static_cast<int>((a->T + 15) / 16 * 16);
  CUtensorMap tq, tk, tv;
  if ((rc = make_head_map(&tq, a->q, a->T, a->H, a->B, a->q_tok, a->q_head, a->q_batch, 128))) return rc;
  if ((rc = make_head_map(&tk, a->k, a->T, a->H, a->B, a->q_tok, a->q_head, a->q_batch, BN))) return rc;
  if ((rc = make_head_map(&tv, a->v, a->T, a->H, a->B, a->q_tok, a->q_head, a->q_batch, BN))) return rc;
  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.lse = a->lse;
  p.o_tok = a->o_tok;
  p.o_head = a->o_head;
  p.o_batch = a->o_batch;
  p.status = a->status;
  p.B = static_cast<int>(a->B);
  p.H = static_cast<int>(a->H);
  p.T = static_cast<int>(a->T);
  p.BN = BN;
  p.scale = a->scale;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(attention_fwd_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM);
    if (e != cudaSuccess) {
      set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
      return -4;
    }
    attr = true;
  }
  dim3 grid(static_cast<unsigned>((a->T + ATT_TILE - 1) / ATT_TILE), static_cast<unsigned>(a->H),
            static_cast<unsigned>(a->B));
  attention_fwd_kernel<<<grid, FWD_THREADS, FWD_SMEM, stream>>>(tq, tk, tv, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
    return -5;
  }
  return 0;
}

}  // namespace vmoe

namespace vmoe {
int attention_d64_bwd(const VmoeAttnArgs* a, vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->B == 0 || a->H == 0) return 0;
  int rc = check_attn(a);
  if (rc) return rc;
  if (a->g_tok % 8 || a->g_head % 8 || a->g_batch % 8) {
    set_error("%s (code %d)", "attention gradient strides must be multiples of 8 elements", 0);
    return -1;
  }
  const int BN = static_cast<int>((a->T + 15) / 16 * 16);
  CUtensorMap tq, tk, tv, tdo;
  if ((rc = make_head_map(&tq, a->q, a->T, a->H, a->B, a->q_tok, a->q_head, a->q_batch, 128))) return rc;
  if ((rc = make_head_map(&tk, a->k, a->T, a->H, a->B, a->q_tok, a->q_head, a->q_batch, 128))) return rc;
  if ((rc = make_head_map(&tv, a->v, a->T, a->H, a->B, a->q_tok, a->q_head, a->q_batch, 128))) return rc;
  if ((rc = make_head_map(&tdo, a->d_out, a->T, a->H, a->B, a->o_tok, a->o_head, a->o_batch, 128)))
    return rc;
  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.lse = a->lse;
  p.o_in = static_cast<const __nv_bfloat16*>(a->out);
  p.d_out = static_cast<const __nv_bfloat16*>(a->d_out);
  p.dq = static_cast<__nv_bfloat16*>(a->dq);
  p.dk = static_cast<__nv_bfloat16*>(a->dk);
  p.dv = static_cast<__nv_bfloat16*>(a->dv);
  p.g_tok = a->g_tok;
  p.g_head = a->g_head;
  p.g_batch = a->g_batch;
  p.o_tok = a->o_tok;
  p.o_head = a->o_head;
  p.o_batch = a->o_batch;
  p.status = a->status;
  p.B = static_cast<int>(a->B);
  p.H = static_cast<int>(a->H);
  p.T = static_cast<int>(a->T);
  p.BN = BN;
  p.scale = a->scale;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(attention_bwd_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM);
    if (e != cudaSuccess) {
      set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
      return -4;
    }
    attr = true;
  }
  dim3 grid(static_cast<unsigned>(a->H), static_cast<unsigned>(a->B));
  attention_bwd_kernel<<<grid, BWD_THREADS, BWD_SMEM, stream>>>(tq, tk, tv, tdo, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
    return -5;
  }
  return 0;
}
}  // namespace vmoe

#ifdef ATT_TRACE
// Copies the stamps of role `who` (0 softmax warp, 1 MMA thread) of the one-shot backward kernel
// as (tag, clock) pairs into `out` (4096 values), resets the list, returns the number of stamps.
extern "C" VMOE_API int vmoe_attention_d64_trace_read(long long* out, int who) {
  int n = 0;
  cudaMemcpyFromSymbol(&n, vmoe::d64::g_d64_trace_n, sizeof(int), who * sizeof(int));
  cudaMemcpyFromSymbol(out, vmoe::d64::g_d64_trace, sizeof(long long) * 4096,
                       who * 4096 * sizeof(long long));
  int zero = 0;
  cudaMemcpyToSymbol(vmoe::d64::g_d64_trace_n, &zero, sizeof(int), who * sizeof(int));
  return n;
}
#endif
