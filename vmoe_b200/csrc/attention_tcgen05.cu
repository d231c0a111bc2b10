// Fused non-causal softmax attention on tcgen05 tensor cores, forward and backward, for the
// sequence lengths and head sizes of Vision Transformers: any number of queries, up to ~700
// keys (the keys and values of one head stay in shared memory), head dim a multiple of 16 up
// to 80 (ViT-S/B/L: 64, ViT-H: 80). Queries and keys / values may come from different tensors
// and sequences (cross-attention of a pooling head), or all three from the packed output of the
// QKV projection, whose packed gradient the backward kernel writes. Optional dropout of the
// attention weights: the keep mask is a counter-based hash of (seed, batch, head, query, key),
// evaluated again in the backward pass instead of being stored.
//
// Forward: persistent CTAs, one work item per (batch, head, 128-query tile). Keys are visited
// in blocks of up to 256: S = Q K^T of a block goes to TMEM; four warps (one query row per
// thread) take the row maximum, rescale the running output when a later block raises it,
// exponentiate and write P as a bf16 UMMA operand, 64 keys at a time; O += P V is issued chunk
// by chunk as P arrives. With a single block (up to 256 keys) O reuses the TMEM columns of S and
// P the shared memory of Q and K, so two CTAs share an SM. The loads of the next item are issued
// as soon as the buffers of the current one are free.
//
// Backward: persistent CTAs, one work item per (batch, head). Outer loop over 128-key blocks
// (K, V double-buffered), inner loop over 128-query tiles (Q, dO double-buffered). S = Q K^T and
// dP = dO V^T are computed 64 keys at a time into two TMEM buffers, so the tensor core produces
// the next half while the softmax warps turn the current one into P = exp(S - lse) and
// dS = P (dP - delta) / sqrt(d), written to shared memory once and used as three UMMA operands:
// dV += P^T dO, dK += dS^T Q (MN-major A) and dQ += dS K (K-major A). dQ stays in TMEM when all
// query tiles fit, else it is added to an fp32 buffer and converted by a second kernel.
//
// Replaces the reference's flax MultiHeadDotProductAttention (vmoe/nn/vit_moe.py:165-173),
// which XLA runs as four library GEMMs plus a softmax fusion.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "ptx_sm100.cuh"
#include "tma_host.h"
#include "vmoe_api.h"

namespace vmoe {

void set_error(const char* fmt, const char* a, int code);

constexpr int ATT_ROW_BYTES = 128;   // 64 bf16: one swizzle row
constexpr int ATT_TILE = 128;        // query rows per tile
constexpr int ATT_TILE_BYTES = ATT_TILE * ATT_ROW_BYTES;  // 16 KiB
constexpr int ATT_KBLOCK = 256;      // keys per forward block (one MMA of N <= 256)
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

// 32 lanes x 32 consecutive 32-bit columns back to TMEM (lane t of the warp writes lane base+t).
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Bounded wait used by every role; on failure all roles fall through to the common exit.
#define ATT_WAIT(bar, parity, code)                                              \
  do {                                                                           \
    const bool got_ = mbar_wait((bar), (parity), abort_flag, status, (code));   \
    if (!got_) ok = false;                                                       \
  } while (0)
// The same for the warps whose TMEM loads need all 32 lanes to agree.
#define ATT_WAIT_WARP(bar, parity, code)                                         \
  do {                                                                           \
    const bool got_ = mbar_wait((bar), (parity), abort_flag, status, (code));   \
    ok = __all_sync(0xffffffffu, got_ && ok);                                    \
  } while (0)

struct AttnParams {
  __nv_bfloat16* out;     // forward: (B, Tq, H, D) through the o_* strides
  float* lse;             // (B, H, Tq) natural-log sum-exp of the scaled scores
  const __nv_bfloat16* o_in;  // backward: forward output
  const __nv_bfloat16* d_out; // backward: dO
  __nv_bfloat16* dq;      // backward outputs
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  float* dq_acc;          // fp32 (B, Tq, H, D) contiguous, zeroed: dQ when it leaves TMEM early
  long long gq_tok, gq_head, gq_batch;     // strides (elements) of dq
  long long gkv_tok, gkv_head, gkv_batch;  // strides of dk / dv
  long long o_tok, o_head, o_batch;        // strides of out / o_in / dO
  unsigned* status;
  int B, H, Tq, Tk, D;
  int nch;      // 64-element chunks of the head dim (1 or 2)
  int kr;       // key rows held in shared memory (Tk rounded up to 64)
  int n_qt;     // query tiles
  float scale;  // 1 / sqrt(d)
  // dropout of the attention weights: keep iff hash byte < keep_q; kept weights scale by inv_keep
  unsigned keep_q;   // 256 = no dropout
  float inv_keep;
  unsigned seed_lo, seed_hi;
};

// ---- dropout mask: one 32-bit hash per (batch*head, query, group of 4 keys), one byte per key
__device__ __forceinline__ unsigned mix32(unsigned x) {
  x ^= x >> 16;
  x *= 0x7feb352du;
  x ^= x >> 15;
  x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}
__device__ __forceinline__ unsigned dropout_word(const AttnParams& p, int bh, int q, int key4) {
  const unsigned idx = (static_cast<unsigned>(bh) * static_cast<unsigned>(p.Tq) +
                        static_cast<unsigned>(q)) * static_cast<unsigned>((p.Tk + 3) >> 2) +
                       static_cast<unsigned>(key4);
  return mix32(mix32(idx ^ p.seed_lo) ^ p.seed_hi);
}

__device__ __forceinline__ uint4 pack8_bf16(const float* e) {
  uint4 u;
  u.x = pack_bf16x2(e[0], e[1]);
  u.y = pack_bf16x2(e[2], e[3]);
  u.z = pack_bf16x2(e[4], e[5]);
  u.w = pack_bf16x2(e[6], e[7]);
  return u;
}

#ifdef ATT_TRACE
// Timing probes (builds with -DATT_TRACE only): CTA 0 records clock64 at tagged points, read
// back with vmoe_attention_trace_read (python -m vmoe_b200.ops.bench_kernels attention_trace).
// Forward tags, softmax warp: 0 before / 1 after the wait for S, 2 after the row maximum, 3 after
// P is written, 4 after the wait for O, 5 after the output is stored; MMA thread: 0 / 1 around
// the wait for Q and K, 4 when the item's products are issued, 5 when they have retired.
__device__ long long g_att_trace[2][4096];
__device__ int g_att_trace_n[2];
#define ATT_STAMP(who, tag)                                                         \
  do {                                                                              \
    if (blockIdx.x == 0 && lane == 0 && g_att_trace_n[who] < 2040) {               \
      const int i_ = g_att_trace_n[who]++;                                          \
      g_att_trace[who][2 * i_] = (tag);                                             \
      g_att_trace[who][2 * i_ + 1] = clock64();                                     \
    }                                                                               \
  } while (0)
#else
#define ATT_STAMP(who, tag) do {} while (0)
#endif

// ================================================================================ forward
constexpr int FWD_THREADS = 160;   // warp 0: TMA + MMA issue (one lane); warps 1-4: softmax
constexpr int FWD_NBARS = 16;
// bars: 0 qk, 1 v, 2 s, 3 sfree, 4 o, 5 resc, 6..9 p[chunk], 10..13 pfree[slot], 14 done

struct FwdLayout {
  int off_q, off_k, off_v, off_p;  // byte offsets from the 1024-aligned base
  int np;                          // P slots (64 keys x 128 queries each)
  int nkb;                         // key blocks
  int aliased;                     // single block: P over Q/K, O over S
  int bar_off, total;
  int tmem_cols, o_col;
};

static FwdLayout fwd_layout(int Tk, int D) {
  FwdLayout L;
  const int nch = (D + 63) / 64;
  const int kr = (Tk + 63) / 64 * 64;
  const int tk16 = (Tk + 15) / 16 * 16;
  L.nkb = (tk16 + ATT_KBLOCK - 1) / ATT_KBLOCK;
  L.aliased = L.nkb == 1;
  const int qb = nch * ATT_TILE_BYTES, kb = nch * kr * ATT_ROW_BYTES;
  if (L.aliased) {
    L.np = kr / 64;
    L.off_v = 0;
    L.off_p = kb;  // V first, then the region shared by P and Q/K
    L.off_q = L.off_p;
    L.off_k = L.off_p + qb;
    const int region = L.np * ATT_TILE_BYTES > qb + kb ? L.np * ATT_TILE_BYTES : qb + kb;
    L.bar_off = L.off_p + region;
    int cols = tk16 > D ? tk16 : D;
    int c2 = 32;
    while (c2 < cols) c2 <<= 1;
    L.tmem_cols = c2;
    L.o_col = 0;
  } else {
    L.np = 2;
    L.off_q = 0;
    L.off_k = qb;
    L.off_v = qb + kb;
    L.off_p = qb + 2 * kb;
    L.bar_off = L.off_p + 2 * ATT_TILE_BYTES;
    L.tmem_cols = 512;
    L.o_col = ATT_KBLOCK;
  }
  L.total = L.bar_off + FWD_NBARS * 8 + 64 + 1024;
  return L;
}

__global__ void __launch_bounds__(FWD_THREADS)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                     const __grid_constant__ CUtensorMap tv, const AttnParams p, const FwdLayout L) {
  extern __shared__ uint8_t att_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(att_smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem + L.off_q;
  uint8_t* sK = smem + L.off_k;
  uint8_t* sV = smem + L.off_v;
  uint8_t* sP = smem + L.off_p;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L.bar_off);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + FWD_NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  unsigned* status = p.status;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_qk = bar0, bar_v = bar0 + 8, bar_s = bar0 + 16, bar_sfree = bar0 + 24,
                 bar_o = bar0 + 32, bar_resc = bar0 + 40, bar_p = bar0 + 48, bar_pfree = bar0 + 80,
                 bar_done = bar0 + 112;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_qk, 1);
    mbar_init(bar_v, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_sfree, 128);
    mbar_init(bar_o, 1);
    mbar_init(bar_resc, 128);
    mbar_init(bar_done, 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(bar_p + 8 * i, 128);
      mbar_init(bar_pfree + 8 * i, 1);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tq);
    tma_prefetch_desc(&tk);
    tma_prefetch_desc(&tv);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), L.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int nch = p.nch, kr = p.kr, D = p.D;
  const int tk16 = (p.Tk + 15) / 16 * 16;
  const int n_items = p.B * p.H * p.n_qt;
  const int k_chunk_bytes = kr * ATT_ROW_BYTES;  // one 64-element chunk of K or V
  bool ok = true;

  if (warp == 0) {
    if (lane == 0) {
      auto load_qk = [&](int item) {
        const int qt = item % p.n_qt, bh = item / p.n_qt, h = bh % p.H, b = bh / p.H;
        mbar_expect_tx(bar_qk, nch * (ATT_TILE_BYTES + k_chunk_bytes));
        for (int j = 0; j < nch; ++j) {
          tma_load_4d(smem_u32(sQ + j * ATT_TILE_BYTES), &tq, bar_qk, 64 * j, h, qt * ATT_TILE, b);
          for (int r = 0; r < kr; r += 64)
            tma_load_4d(smem_u32(sK + j * k_chunk_bytes + r * ATT_ROW_BYTES), &tk, bar_qk, 64 * j, h,
                        r, b);
        }
      };
      auto load_v = [&](int item) {
        const int bh = item / p.n_qt, h = bh % p.H, b = bh / p.H;
        mbar_expect_tx(bar_v, nch * k_chunk_bytes);
        for (int j = 0; j < nch; ++j)
          for (int r = 0; r < kr; r += 64)
            tma_load_4d(smem_u32(sV + j * k_chunk_bytes + r * ATT_ROW_BYTES), &tv, bar_v, 64 * j, h,
                        r, b);
      };
      uint32_t n_item = 0, n_s = 0, n_resc = 0;
      uint32_t n_p[4] = {0, 0, 0, 0};
      if (static_cast<int>(blockIdx.x) < n_items) {
        load_qk(blockIdx.x);
        load_v(blockIdx.x);
      }
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++n_item) {
        const int next = item + gridDim.x;
        ATT_STAMP(1, 0);
        ATT_WAIT(bar_qk, n_item & 1, kStatusTimeoutMma | (1u << (7 + 1)));
        ATT_STAMP(1, 1);
        for (int kb = 0; kb < L.nkb && ok; ++kb) {
          const int nk = min(ATT_KBLOCK, tk16 - kb * ATT_KBLOCK);
          // S (and, aliased, O) columns are free once the softmax warps have read them.
          if (n_s > 0) ATT_WAIT(bar_sfree, (n_s - 1) & 1, kStatusTimeoutMma | (1u << (7 + 2)));
          if (!ok) break;
          tc_fence_after();
          const uint32_t idesc = umma_idesc_bf16(128, nk, 0, 0);
          for (int k = 0; k < D / 16; ++k)
            umma_bf16(tmem,
                      umma_smem_desc(smem_u32(sQ) + (k >> 2) * ATT_TILE_BYTES + (k & 3) * 32, 16, 1024),
                      umma_smem_desc(smem_u32(sK) + (k >> 2) * k_chunk_bytes +
                                         kb * ATT_KBLOCK * ATT_ROW_BYTES + (k & 3) * 32, 16, 1024),
                      idesc, k > 0);
          umma_commit(bar_s);
          ++n_s;
          if (!L.aliased && kb == L.nkb - 1) {
            // Q and K are free when the last S has been computed: fetch the next item's.
            ATT_WAIT(bar_s, (n_s - 1) & 1, kStatusTimeoutMma | (1u << (7 + 3)));
            if (ok && next < n_items) load_qk(next);
          }
          if (kb == 0) ATT_WAIT(bar_v, n_item & 1, kStatusTimeoutMma | (1u << (7 + 4)));
          if (kb > 0) {  // the running output has been rescaled for this block's maximum
            ATT_WAIT(bar_resc, n_resc & 1, kStatusTimeoutMma | (1u << (7 + 5)));
            ++n_resc;
          }
          if (!ok) break;
          const int nchunks = (nk + 63) / 64;
          const uint32_t id_pv = umma_idesc_bf16(128, D, 0, 1);
          for (int c = 0; c < nchunks && ok; ++c) {
            ATT_WAIT(bar_p + 8 * c, n_p[c] & 1, kStatusTimeoutMma | (1u << (7 + 6)));
            ++n_p[c];
            if (L.aliased && c == 0 && D > 64 && nchunks > 1) {
              // O covers more columns than the first 64 keys of S: wait for the next chunk too.
              ATT_WAIT(bar_p + 8, n_p[1] & 1, kStatusTimeoutMma | (1u << (7 + 7)));
            }
            if (!ok) break;
            tc_fence_after();
            const int slot = c % L.np;
            const int steps = min(64, nk - 64 * c) / 16;
            for (int kk = 0; kk < steps; ++kk) {
              const int key = kb * ATT_KBLOCK + 64 * c + 16 * kk;
              umma_bf16(tmem + L.o_col,
                        umma_smem_desc(smem_u32(sP) + slot * ATT_TILE_BYTES + kk * 32, 16, 1024),
                        umma_smem_desc(smem_u32(sV) + key * ATT_ROW_BYTES, k_chunk_bytes, 1024),
                        id_pv, (kb > 0 || c > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(bar_pfree + 8 * slot);
          }
          umma_commit(bar_o);  // per block, for the softmax warps
        }
        // All MMAs of the item retire in order. bar_o may complete several phases per item
        // (one per key block), which a waiter that is not in step with them cannot tell apart,
        // so this thread has a barrier of its own with one phase per item.
        umma_commit(bar_done);
        ATT_STAMP(1, 4);
        if (ok) ATT_WAIT(bar_done, n_item & 1, kStatusTimeoutMma | (1u << 15));
        ATT_STAMP(1, 5);
        if (ok && next < n_items) {
          if (L.aliased) load_qk(next);
          load_v(next);
        }
      }
      if (!ok) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) __nanosleep(256);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax / epilogue warps
    const int quad = warp & 3;             // TMEM lane quadrant this warp may read
    const int r = quad * 32 + lane;        // row inside the query tile
    const uint32_t trow = tmem + (static_cast<uint32_t>(quad * 32) << 16);
    const float sl2 = p.scale * kLog2e;
    const bool drop = p.keep_q < 256u;
    uint32_t n_s = 0, n_o = 0;
    uint32_t n_fill[4] = {0, 0, 0, 0};
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const int qt = item % p.n_qt, bh = item / p.n_qt, h = bh % p.H, b = bh / p.H;
      const int q = qt * ATT_TILE + r;       // query index
      // A warp whose 32 rows all lie past the last query only keeps the barriers moving.
      const bool warp_live = qt * ATT_TILE + quad * 32 < p.Tq;
      float m_run = -INFINITY, l_run = 0.f;
      for (int kb = 0; kb < L.nkb && ok; ++kb) {
        const int nk = min(ATT_KBLOCK, tk16 - kb * ATT_KBLOCK);
        const int key0 = kb * ATT_KBLOCK;
        const int n32 = (nk + 31) / 32;
        if (warp == 1) ATT_STAMP(0, 0);
        ATT_WAIT_WARP(bar_s, n_s & 1, kStatusTimeoutEpilogue);
        if (warp == 1) ATT_STAMP(0, 1);
        ++n_s;
        if (!ok) break;
        tc_fence_after();
        float mx = m_run;
        if (warp_live) {
          for (int c = 0; c < n32; ++c) {
            uint32_t v[32];
            tmem_ld_32x32(trow + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (key0 + c * 32 + i < p.Tk) mx = fmaxf(mx, __uint_as_float(v[i]));
          }
        }
        if (kb > 0) {
          // A later block raised the maximum: bring the running sum and output to the new one.
          ATT_WAIT_WARP(bar_o, n_o & 1, kStatusTimeoutEpilogue);
          ++n_o;
          if (!ok) break;
          tc_fence_after();
          if (warp_live) {
            const float alpha = exp2f((m_run - mx) * sl2);
            l_run *= alpha;
            for (int c = 0; c < (D + 31) / 32; ++c) {
              uint32_t v[32];
              tmem_ld_32x32(trow + L.o_col + c * 32, v);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
              tmem_st_32x32(trow + L.o_col + c * 32, v);
            }
            tmem_st_wait();
          }
          tc_fence_before();
          mbar_arrive(bar_resc);
        }
        m_run = mx;
        const float mxs = mx * sl2;
        if (warp == 1) ATT_STAMP(0, 2);
        for (int c = 0; c < n32; ++c) {
          const int chunk = c >> 1, slot = chunk % L.np;
          if ((c & 1) == 0) {
            // The PV product that read this slot last must have retired.
            if (n_fill[slot] > 0)
              ATT_WAIT_WARP(bar_pfree + 8 * slot, (n_fill[slot] - 1) & 1, kStatusTimeoutEpilogue);
            ++n_fill[slot];
            if (!ok) break;
          }
          if (warp_live) {
            uint32_t v[32];
            tmem_ld_32x32(trow + c * 32, v);
            tmem_ld_wait();
            float e[32];
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              e[i] = (key0 + c * 32 + i < p.Tk) ? exp2f(__uint_as_float(v[i]) * sl2 - mxs) : 0.f;
              sum += e[i];
            }
            l_run += sum;
            if (drop) {
#pragma unroll
              for (int i4 = 0; i4 < 8; ++i4) {
                const unsigned w = dropout_word(p, bh, q, (key0 + c * 32) / 4 + i4);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  e[4 * i4 + j] = ((w >> (8 * j)) & 0xffu) < p.keep_q ? e[4 * i4 + j] * p.inv_keep : 0.f;
              }
            }
            // Row r of the 64-key chunk: 16-byte units j = 4 * (c & 1) + i, 128B swizzle.
            uint8_t* base = sP + slot * ATT_TILE_BYTES + r * ATT_ROW_BYTES;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t j = static_cast<uint32_t>(4 * (c & 1) + i);
              *reinterpret_cast<uint4*>(base + ((j ^ (static_cast<uint32_t>(r) & 7u)) << 4)) =
                  pack8_bf16(e + 8 * i);
            }
          }
          if ((c & 1) == 1 || c == n32 - 1) {
            fence_proxy_async();
            tc_fence_before();
            mbar_arrive(bar_p + 8 * chunk);
          }
        }
        if (!ok) break;
        if (kb < L.nkb - 1) {
          tc_fence_before();
          mbar_arrive(bar_sfree);  // S of this block has been read
        }
      }
      if (!ok) break;
      if (warp == 1) ATT_STAMP(0, 3);
      ATT_WAIT_WARP(bar_o, n_o & 1, kStatusTimeoutEpilogue);
      if (warp == 1) ATT_STAMP(0, 4);
      ++n_o;
      if (!ok) break;
      tc_fence_after();
      if (warp_live) {
        const float inv = 1.0f / l_run;
        __nv_bfloat16* orow = p.out + b * p.o_batch + static_cast<long long>(q) * p.o_tok + h * p.o_head;
        for (int c = 0; c < (D + 31) / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(trow + L.o_col + c * 32, v);
          tmem_ld_wait();
          if (q < p.Tq) {
            float f[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]) * inv;
#pragma unroll
            for (int i = 0; i < 4; ++i)
              if (c * 32 + 8 * i < D) reinterpret_cast<uint4*>(orow + c * 32)[i] = pack8_bf16(f + 8 * i);
          }
        }
        if (q < p.Tq && p.lse)
          p.lse[(static_cast<long long>(b) * p.H + h) * p.Tq + q] = m_run * p.scale + __logf(l_run);
      }
      if (warp == 1) ATT_STAMP(0, 5);
      tc_fence_before();
      mbar_arrive(bar_sfree);  // O (and the last S) have been read: the next item may start
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, L.tmem_cols);
  }
}

// ================================================================================ backward
constexpr int BWD_THREADS = 192;  // warp 0: TMA loads, warp 1: MMA issue, warps 2-5: softmax bwd
constexpr int BWD_NBARS = 20;
// bars: 0,1 kvfull[stage]; 2,3 kvfree; 4,5 qfull; 6,7 qfree; 8,9 s[half]; 10,11 sfree[half];
//       12 pd; 13 mma; 14 accfree
constexpr uint32_t TM_DV = 256;   // S0 0, dP0 64, S1 128, dP1 192, then dV, dK, dQ

struct BwdLayout {
  int off_k, off_v, off_q, off_do, off_p, off_ds;
  int nkv, nq;          // pipeline stages of (K, V) and of (Q, dO)
  int tile_bytes;       // one 128-row operand: nch * 16 KiB
  int dq_resident;      // dQ of all query tiles stays in TMEM until the item ends
  int dq_col;
  int bar_off, total;
};

static BwdLayout bwd_layout(int Tq, int D) {
  BwdLayout L;
  const int nch = (D + 63) / 64;
  const int n_qt = (Tq + ATT_TILE - 1) / ATT_TILE;
  L.tile_bytes = nch * ATT_TILE_BYTES;
  const int budget = 227 * 1024 - 2048 - 4 * ATT_TILE_BYTES;  // minus P, dS, barriers, alignment
  // Prefer double-buffering both operand pairs, then (Q, dO) alone, then neither.
  L.nkv = 1;
  L.nq = 1;
  if (8 * L.tile_bytes <= budget) {
    L.nkv = 2;
    L.nq = 2;
  } else if (6 * L.tile_bytes <= budget) {
    L.nq = 2;
  }
  int off = 0;
  L.off_k = off;  off += L.nkv * L.tile_bytes;
  L.off_v = off;  off += L.nkv * L.tile_bytes;
  L.off_q = off;  off += L.nq * L.tile_bytes;
  L.off_do = off; off += L.nq * L.tile_bytes;
  L.off_p = off;  off += 2 * ATT_TILE_BYTES;
  L.off_ds = off; off += 2 * ATT_TILE_BYTES;
  L.bar_off = off;
  L.total = off + BWD_NBARS * 8 + 64 + 1024;
  L.dq_col = TM_DV + 2 * D;
  L.dq_resident = L.dq_col + n_qt * D <= 512;
  return L;
}

__global__ void __launch_bounds__(BWD_THREADS, 1)
attention_bwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                     const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                     const AttnParams p, const BwdLayout L) {
  extern __shared__ uint8_t att_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(att_smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem + L.off_k;
  uint8_t* sV = smem + L.off_v;
  uint8_t* sQ = smem + L.off_q;
  uint8_t* sDO = smem + L.off_do;
  uint8_t* sP = smem + L.off_p;    // 128 q x 128 keys bf16: 2 chunks of 16 KiB (64 keys each)
  uint8_t* sDS = smem + L.off_ds;  // same layout
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L.bar_off);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + BWD_NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  unsigned* status = p.status;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_kvfull = bar0, bar_kvfree = bar0 + 16, bar_qfull = bar0 + 32,
                 bar_qfree = bar0 + 48, bar_s = bar0 + 64, bar_sfree = bar0 + 80,
                 bar_pd = bar0 + 96, bar_mma = bar0 + 104, bar_accfree = bar0 + 112;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_kvfull + 8 * i, 1);
      mbar_init(bar_kvfree + 8 * i, 1);
      mbar_init(bar_qfull + 8 * i, 1);
      mbar_init(bar_qfree + 8 * i, 1);
      mbar_init(bar_s + 8 * i, 1);
      mbar_init(bar_sfree + 8 * i, 128);
    }
    mbar_init(bar_pd, 128);
    mbar_init(bar_mma, 1);
    mbar_init(bar_accfree, 128);
    fence_mbar_init();
    tma_prefetch_desc(&tq);
    tma_prefetch_desc(&tk);
    tma_prefetch_desc(&tv);
    tma_prefetch_desc(&tdo);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int D = p.D, nch = p.nch, Tq = p.Tq, Tk = p.Tk;
  const int n_qt = p.n_qt;
  const int tk16 = (Tk + 15) / 16 * 16;
  const int n_kb = (tk16 + ATT_TILE - 1) / ATT_TILE;
  const int n_items = p.B * p.H;
  const int TB = L.tile_bytes;
  const uint32_t tm_dk = TM_DV + D, tm_dq = L.dq_col;
  bool ok = true;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA loader
    if (lane == 0) {
      uint32_t n_kv = 0, n_q = 0;  // loads issued so far (stage = count % stages)
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
        const int h = item % p.H, b = item / p.H;
        for (int kb = 0; kb < n_kb && ok; ++kb) {
          {
            const uint32_t st = n_kv % L.nkv, use = n_kv / L.nkv;
            if (use > 0) ATT_WAIT(bar_kvfree + 8 * st, (use - 1) & 1, kStatusTimeoutProducer);
            if (!ok) break;
            mbar_expect_tx(bar_kvfull + 8 * st, 2 * TB);
            for (int j = 0; j < nch; ++j) {
              tma_load_4d(smem_u32(sK + st * TB + j * ATT_TILE_BYTES), &tk, bar_kvfull + 8 * st,
                          64 * j, h, kb * ATT_TILE, b);
              tma_load_4d(smem_u32(sV + st * TB + j * ATT_TILE_BYTES), &tv, bar_kvfull + 8 * st,
                          64 * j, h, kb * ATT_TILE, b);
            }
            ++n_kv;
          }
          for (int qt = 0; qt < n_qt && ok; ++qt) {
            const uint32_t st = n_q % L.nq, use = n_q / L.nq;
            if (use > 0) ATT_WAIT(bar_qfree + 8 * st, (use - 1) & 1, kStatusTimeoutProducer);
            if (!ok) break;
            mbar_expect_tx(bar_qfull + 8 * st, 2 * TB);
            for (int j = 0; j < nch; ++j) {
              tma_load_4d(smem_u32(sQ + st * TB + j * ATT_TILE_BYTES), &tq, bar_qfull + 8 * st,
                          64 * j, h, qt * ATT_TILE, b);
              tma_load_4d(smem_u32(sDO + st * TB + j * ATT_TILE_BYTES), &tdo, bar_qfull + 8 * st,
                          64 * j, h, qt * ATT_TILE, b);
            }
            ++n_q;
          }
        }
      }
      if (!ok) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) __nanosleep(256);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // Steps are numbered over the whole life of the CTA: step = (item, key block, query tile).
      const int steps_per_item = n_kb * n_qt;
      int my_items = 0;
      for (int item = blockIdx.x; item < n_items; item += gridDim.x) ++my_items;
      const long long total_steps = static_cast<long long>(my_items) * steps_per_item;
      uint32_t n_sh[2] = {0, 0};   // S/dP halves issued into each buffer
      uint32_t n_acc = 0;          // key blocks whose dV/dK accumulation has started
      auto halves_of = [&](long long s) {
        const int kb = static_cast<int>((s % steps_per_item) / n_qt);
        const int nkeys = min(ATT_TILE, tk16 - kb * ATT_TILE);
        return nkeys > 64 ? 2 : 1;
      };
      // Issues S and dP of half `hf` of step s; its operands must have been waited for.
      auto issue_sdp = [&](long long s, int hf) {
        const int kb = static_cast<int>((s % steps_per_item) / n_qt);
        const int nkeys = min(ATT_TILE, tk16 - kb * ATT_TILE);
        const int nkh = min(64, nkeys - 64 * hf);
        const uint32_t qs = static_cast<uint32_t>(s % L.nq);
        const uint32_t kvs = static_cast<uint32_t>((s / n_qt) % L.nkv);
        const uint32_t qb = smem_u32(sQ + qs * TB), dob = smem_u32(sDO + qs * TB);
        const uint32_t kbase = smem_u32(sK + kvs * TB) + hf * 64 * ATT_ROW_BYTES;
        const uint32_t vbase = smem_u32(sV + kvs * TB) + hf * 64 * ATT_ROW_BYTES;
        const uint32_t id_s = umma_idesc_bf16(128, nkh, 0, 0);
        for (int k = 0; k < D / 16; ++k)
          umma_bf16(tmem + hf * 128,
                    umma_smem_desc(qb + (k >> 2) * ATT_TILE_BYTES + (k & 3) * 32, 16, 1024),
                    umma_smem_desc(kbase + (k >> 2) * ATT_TILE_BYTES + (k & 3) * 32, 16, 1024), id_s,
                    k > 0);
        for (int k = 0; k < D / 16; ++k)
          umma_bf16(tmem + hf * 128 + 64,
                    umma_smem_desc(dob + (k >> 2) * ATT_TILE_BYTES + (k & 3) * 32, 16, 1024),
                    umma_smem_desc(vbase + (k >> 2) * ATT_TILE_BYTES + (k & 3) * 32, 16, 1024), id_s,
                    k > 0);
        umma_commit(bar_s + 8 * hf);
        ++n_sh[hf];
      };
      // Waits until half-buffer hf may be overwritten (its previous contents have been read).
      auto wait_sfree = [&](int hf) {
        if (n_sh[hf] > 0) ATT_WAIT(bar_sfree + 8 * hf, (n_sh[hf] - 1) & 1, kStatusTimeoutMma);
      };
      // Waits for the operands of step s (K, V when it opens a key block; Q, dO always).
      auto wait_operands = [&](long long s) {
        if (s % n_qt == 0) {
          const long long blk = s / n_qt;
          ATT_WAIT(bar_kvfull + 8 * static_cast<uint32_t>(blk % L.nkv),
                   static_cast<uint32_t>(blk / L.nkv) & 1, kStatusTimeoutMma);
        }
        if (ok)
          ATT_WAIT(bar_qfull + 8 * static_cast<uint32_t>(s % L.nq),
                   static_cast<uint32_t>(s / L.nq) & 1, kStatusTimeoutMma);
      };
      if (total_steps > 0) {
        wait_operands(0);
        if (ok) {
          tc_fence_after();
          issue_sdp(0, 0);
          if (halves_of(0) > 1) issue_sdp(0, 1);
        }
      }
      for (long long s = 0; s < total_steps && ok; ++s) {
        const int in_item = static_cast<int>(s % steps_per_item);
        const int kb = in_item / n_qt, qt = in_item % n_qt;
        const int nkeys = min(ATT_TILE, tk16 - kb * ATT_TILE);
        const uint32_t qs = static_cast<uint32_t>(s % L.nq);
        const uint32_t kvs = static_cast<uint32_t>((s / n_qt) % L.nkv);
        const bool has_next = s + 1 < total_steps;
        // The next step's operands can be waited for now only if their loads do not depend on
        // buffers that this step's products still have to release.
        const bool early = has_next && L.nq == 2 && ((s + 1) % n_qt != 0 || L.nkv == 2);
        if (early) {
          wait_operands(s + 1);
          ATT_STAMP(1, 5);
          if (ok) wait_sfree(0);
          if (!ok) break;
          tc_fence_after();
          issue_sdp(s + 1, 0);
          ATT_STAMP(1, 6);
        }
        ATT_STAMP(1, 1);
        ATT_WAIT(bar_pd, static_cast<uint32_t>(s) & 1, kStatusTimeoutMma);
        ATT_STAMP(1, 2);
        if (ok && qt == 0 && n_acc > 0)
          ATT_WAIT(bar_accfree, (n_acc - 1) & 1, kStatusTimeoutMma);  // dV/dK of the last block read
        if (!ok) break;
        if (qt == 0) ++n_acc;
        tc_fence_after();
        const uint32_t qb = smem_u32(sQ + qs * TB), dob = smem_u32(sDO + qs * TB);
        const uint32_t kbase = smem_u32(sK + kvs * TB);
        // dV += P^T dO, dK += dS^T Q: A read MN-major (M = keys), B MN-major (N = d).
        const uint32_t id_t = umma_idesc_bf16(128, D, 1, 1);
        for (int k = 0; k < ATT_TILE / 16; ++k)
          umma_bf16(tmem + TM_DV, umma_smem_desc(smem_u32(sP) + k * 2048, ATT_TILE_BYTES, 1024),
                    umma_smem_desc(dob + k * 2048, ATT_TILE_BYTES, 1024), id_t, (qt > 0 || k > 0));
        for (int k = 0; k < ATT_TILE / 16; ++k)
          umma_bf16(tmem + tm_dk, umma_smem_desc(smem_u32(sDS) + k * 2048, ATT_TILE_BYTES, 1024),
                    umma_smem_desc(qb + k * 2048, ATT_TILE_BYTES, 1024), id_t, (qt > 0 || k > 0));
        // dQ += dS K: A K-major (M = queries, K = keys), B MN-major.
        const uint32_t id_q = umma_idesc_bf16(128, D, 0, 1);
        const uint32_t dq_at = tm_dq + (L.dq_resident ? qt * D : 0);
        for (int k = 0; k < nkeys / 16; ++k)
          umma_bf16(tmem + dq_at,
                    umma_smem_desc(smem_u32(sDS) + (k >> 2) * ATT_TILE_BYTES + (k & 3) * 32, 16, 1024),
                    umma_smem_desc(kbase + k * 2048, ATT_TILE_BYTES, 1024), id_q,
                    ((L.dq_resident && kb > 0) || k > 0));
        umma_commit(bar_mma);
        umma_commit(bar_qfree + 8 * qs);
        if (qt == n_qt - 1) umma_commit(bar_kvfree + 8 * kvs);
        ATT_STAMP(1, 3);
        if (has_next) {
          if (!early) {
            wait_operands(s + 1);
            if (ok) wait_sfree(0);
            if (!ok) break;
            tc_fence_after();
            issue_sdp(s + 1, 0);
          }
          if (halves_of(s + 1) > 1) {
            wait_sfree(1);
            if (!ok) break;
            tc_fence_after();
            issue_sdp(s + 1, 1);
            ATT_STAMP(1, 4);
          }
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax-backward warps
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t trow = tmem + (static_cast<uint32_t>(quad * 32) << 16);
    const float sl2 = p.scale * kLog2e;
    const bool drop = p.keep_q < 256u;
    uint32_t n_sh[2] = {0, 0};   // halves consumed from each S/dP buffer
    uint32_t n_step = 0;         // steps started
    uint32_t n_mma_seen = 0;     // bar_mma phases already waited for
    // Waits until the dV/dK/dQ products of all steps before `upto` have retired.
    auto wait_mma = [&](uint32_t upto) {
      while (n_mma_seen < upto && ok) {
        ATT_WAIT_WARP(bar_mma, n_mma_seen & 1, kStatusTimeoutEpilogue);
        ++n_mma_seen;
      }
    };
    // dQ of one query tile leaves TMEM: bf16 store (resident mode) or fp32 accumulation.
    auto emit_dq = [&](int b, int h, int qt, uint32_t col, bool to_acc) {
      const int q = qt * ATT_TILE + r;
      for (int c = 0; c < (D + 31) / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(trow + col + c * 32, v);
        tmem_ld_wait();
        if (q >= Tq) continue;
        if (to_acc) {
          float* dst = p.dq_acc + ((static_cast<long long>(b) * Tq + q) * p.H + h) * D + c * 32;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < D) atomicAdd(dst + i, __uint_as_float(v[i]));
        } else {
          __nv_bfloat16* dst = p.dq + b * p.gq_batch + static_cast<long long>(q) * p.gq_tok +
                               h * p.gq_head + c * 32;
          float f[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (c * 32 + 8 * i < D) reinterpret_cast<uint4*>(dst)[i] = pack8_bf16(f + 8 * i);
        }
      }
    };
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const int h = item % p.H, b = item / p.H;
      float delta_c[2] = {0.f, 0.f}, lse_c[2] = {0.f, 0.f};
      int flush_qt = -1;  // query tile whose dQ (non-resident mode) still sits in TMEM
      for (int kb = 0; kb < n_kb && ok; ++kb) {
        const int nkeys = min(ATT_TILE, tk16 - kb * ATT_TILE);
        const int nh = nkeys > 64 ? 2 : 1;
        for (int qt = 0; qt < n_qt && ok; ++qt) {
          const int q = qt * ATT_TILE + r;
          const bool qv = q < Tq;
          // delta = rowsum(dO * O) and lse of this thread's query row (kept for two tiles).
          float dl = 0.f, ls = 0.f;
          if (qt < 2 && kb > 0) {
            dl = delta_c[qt];
            ls = lse_c[qt];
          } else if (qv) {
            const long long off = b * p.o_batch + static_cast<long long>(q) * p.o_tok + h * p.o_head;
            const uint4* a4 = reinterpret_cast<const uint4*>(p.d_out + off);
            const uint4* o4 = reinterpret_cast<const uint4*>(p.o_in + off);
            float acc = 0.f;
            for (int i = 0; i < D / 8; ++i) {
              const uint4 x = __ldg(a4 + i), y = __ldg(o4 + i);
              const float2 x0 = unpack_bf16x2(x.x), x1 = unpack_bf16x2(x.y), x2 = unpack_bf16x2(x.z),
                           x3 = unpack_bf16x2(x.w);
              const float2 y0 = unpack_bf16x2(y.x), y1 = unpack_bf16x2(y.y), y2 = unpack_bf16x2(y.z),
                           y3 = unpack_bf16x2(y.w);
              acc += x0.x * y0.x + x0.y * y0.y + x1.x * y1.x + x1.y * y1.y + x2.x * y2.x +
                     x2.y * y2.y + x3.x * y3.x + x3.y * y3.y;
            }
            dl = acc;
            ls = p.lse[(static_cast<long long>(b) * p.H + h) * Tq + q] * kLog2e;
            if (qt < 2) {
              delta_c[qt] = dl;
              lse_c[qt] = ls;
            }
          }
          const uint32_t step = n_step++;
          if (warp == 2) ATT_STAMP(0, 1);
          for (int hf = 0; hf < nh && ok; ++hf) {
            const int nkh = min(64, nkeys - 64 * hf);
            ATT_WAIT_WARP(bar_s + 8 * hf, n_sh[hf] & 1, kStatusTimeoutEpilogue);
            if (warp == 2) ATT_STAMP(0, 2 + hf * 10);
            ++n_sh[hf];
            if (!ok) break;
            tc_fence_after();
            uint32_t pp[32], pd[32];  // 64 keys of P and dS, two bf16 per register
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              if (c * 32 < nkh) {
                uint32_t sv[32], dv[32];
                tmem_ld_32x32(trow + hf * 128 + c * 32, sv);
                tmem_ld_32x32(trow + hf * 128 + 64 + c * 32, dv);
                tmem_ld_wait();
                const int key0 = kb * ATT_TILE + hf * 64 + c * 32;
                float pe[32], de[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                  const bool v = qv && key0 + i < Tk;
                  const float pr = v ? exp2f(__uint_as_float(sv[i]) * sl2 - ls) : 0.f;
                  pe[i] = pr;
                  de[i] = __uint_as_float(dv[i]);
                }
                if (drop) {
#pragma unroll
                  for (int i4 = 0; i4 < 8; ++i4) {
                    const unsigned w = dropout_word(p, b * p.H + h, q, key0 / 4 + i4);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                      const float mk = ((w >> (8 * j)) & 0xffu) < p.keep_q ? p.inv_keep : 0.f;
                      de[4 * i4 + j] *= mk;             // dP of the undropped weights
                      const float pr = pe[4 * i4 + j];
                      pe[4 * i4 + j] = pr * mk;         // dropped weights feed dV
                      de[4 * i4 + j] = pr * (de[4 * i4 + j] - dl) * p.scale;
                    }
                  }
                } else {
#pragma unroll
                  for (int i = 0; i < 32; ++i) de[i] = pe[i] * (de[i] - dl) * p.scale;
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  pp[c * 16 + i] = pack_bf16x2(pe[2 * i], pe[2 * i + 1]);
                  pd[c * 16 + i] = pack_bf16x2(de[2 * i], de[2 * i + 1]);
                }
              } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) pp[c * 16 + i] = pd[c * 16 + i] = 0u;
              }
            }
            if (warp == 2) ATT_STAMP(0, 3 + hf * 10);
            tc_fence_before();
            mbar_arrive(bar_sfree + 8 * hf);
            if (hf == 0) {
              // The products of the previous step read P and dS: they must have retired. In
              // non-resident mode that step's dQ tile leaves TMEM now, before it is overwritten.
              wait_mma(step);
              if (!ok) break;
              if (flush_qt >= 0) {
                tc_fence_after();
                emit_dq(b, h, flush_qt, tm_dq, true);
                flush_qt = -1;
              }
            }
            if (warp == 2) ATT_STAMP(0, 4 + hf * 10);
            const uint32_t off = hf * ATT_TILE_BYTES + r * ATT_ROW_BYTES;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t sw = (static_cast<uint32_t>(j) ^ (static_cast<uint32_t>(r) & 7u)) << 4;
              *reinterpret_cast<uint4*>(sP + off + sw) =
                  make_uint4(pp[4 * j], pp[4 * j + 1], pp[4 * j + 2], pp[4 * j + 3]);
              *reinterpret_cast<uint4*>(sDS + off + sw) =
                  make_uint4(pd[4 * j], pd[4 * j + 1], pd[4 * j + 2], pd[4 * j + 3]);
            }
          }
          if (!ok) break;
          fence_proxy_async();
          tc_fence_before();
          mbar_arrive(bar_pd);
          if (warp == 2) ATT_STAMP(0, 5);
          if (!L.dq_resident) flush_qt = qt;
        }
        if (!ok) break;
        // dV / dK of this key block are complete once the last step's products retire.
        wait_mma(n_step);
        if (!ok) break;
        tc_fence_after();
        if (flush_qt >= 0) {
          emit_dq(b, h, flush_qt, tm_dq, true);
          flush_qt = -1;
        }
        const int key = kb * ATT_TILE + r;
        const long long goff = b * p.gkv_batch + static_cast<long long>(key) * p.gkv_tok + h * p.gkv_head;
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          __nv_bfloat16* dst = (which == 0 ? p.dv : p.dk) + goff;
          for (int c = 0; c < (D + 31) / 32; ++c) {
            uint32_t v[32];
            tmem_ld_32x32(trow + (which == 0 ? TM_DV : tm_dk) + c * 32, v);
            tmem_ld_wait();
            if (key < Tk) {
              float f[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
#pragma unroll
              for (int i = 0; i < 4; ++i)
                if (c * 32 + 8 * i < D) reinterpret_cast<uint4*>(dst + c * 32)[i] = pack8_bf16(f + 8 * i);
            }
          }
        }
        if (kb == n_kb - 1 && L.dq_resident)
          for (int qt = 0; qt < n_qt; ++qt) emit_dq(b, h, qt, tm_dq + qt * D, false);
        tc_fence_before();
        mbar_arrive(bar_accfree);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// dq (bf16, strided) = dq_acc (fp32, (B, Tq, H, D) contiguous), eight elements per thread.
__global__ void attention_dq_convert_kernel(const float* acc, __nv_bfloat16* dq, long long n8, int Tq,
                                            int H, int D, long long tok, long long head,
                                            long long batch) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const long long e = i * 8;
  const int d = static_cast<int>(e % D);
  const long long row = e / D;
  const int h = static_cast<int>(row % H);
  const long long bq = row / H;
  const int q = static_cast<int>(bq % Tq);
  const long long b = bq / Tq;
  const float4 a = reinterpret_cast<const float4*>(acc + e)[0];
  const float4 c = reinterpret_cast<const float4*>(acc + e)[1];
  const float f[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
  *reinterpret_cast<uint4*>(dq + b * batch + q * tok + h * head + d) = pack8_bf16(f);
}

// ------------------------------------------------------------------------------- host side
// (D, H, T, B) view of a bf16 tensor with element strides (1, head, tok, batch); a box is
// 64 x 1 x rows x 1: rows of one head, 128 bytes each (elements past D read as zero).
static int make_head_map(CUtensorMap* map, const void* ptr, int64_t d, int64_t t, int64_t h,
                         int64_t b, int64_t tok, int64_t head, int64_t batch, uint32_t box_rows) {
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(h),
                        static_cast<cuuint64_t>(t), static_cast<cuuint64_t>(b)};
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

struct AttnGeom {
  int64_t Tq, Tk;
  int64_t kv_tok, kv_head, kv_batch;
  int64_t gkv_tok, gkv_head, gkv_batch;
};

static int check_attn(const VmoeAttnArgs* a, AttnGeom* g, bool backward) {
  g->Tq = a->T;
  g->Tk = a->Tk > 0 ? a->Tk : a->T;
  const bool own_kv = a->kv_tok != 0 || a->kv_head != 0 || a->kv_batch != 0;
  g->kv_tok = own_kv ? a->kv_tok : a->q_tok;
  g->kv_head = own_kv ? a->kv_head : a->q_head;
  g->kv_batch = own_kv ? a->kv_batch : a->q_batch;
  const bool own_g = a->gkv_tok != 0 || a->gkv_head != 0 || a->gkv_batch != 0;
  g->gkv_tok = own_g ? a->gkv_tok : a->g_tok;
  g->gkv_head = own_g ? a->gkv_head : a->g_head;
  g->gkv_batch = own_g ? a->gkv_batch : a->g_batch;
  if (a->D % 16 || a->D < 16 || a->D > 80 || g->Tq < 1 || g->Tk < 1) {
    set_error("%s (code %d)", "attention kernel needs head_dim in {16, 32, ..., 80} and T >= 1",
              static_cast<int>(a->D));
    return -1;
  }
  if (fwd_layout(static_cast<int>(g->Tk), static_cast<int>(a->D)).total > 227 * 1024) {
    set_error("%s (code %d)", "attention kernel: keys and values of one head exceed shared memory",
              static_cast<int>(g->Tk));
    return -1;
  }
  if (a->dropout_p < 0.f || a->dropout_p >= 1.f) {
    set_error("%s (code %d)", "attention dropout must be in [0, 1)", 0);
    return -1;
  }
  const int64_t strides[] = {a->q_tok, a->q_head, a->q_batch, g->kv_tok, g->kv_head, g->kv_batch,
                             a->o_tok, a->o_head, a->o_batch};
  for (int64_t s : strides)
    if (s % 8) {
      set_error("%s (code %d)", "attention strides must be multiples of 8 elements", 0);
      return -1;
    }
  if (backward) {
    const int64_t gs[] = {a->g_tok, a->g_head, a->g_batch, g->gkv_tok, g->gkv_head, g->gkv_batch};
    for (int64_t s : gs)
      if (s % 8) {
        set_error("%s (code %d)", "attention gradient strides must be multiples of 8 elements", 0);
        return -1;
      }
  }
  return 0;
}

static void fill_params(AttnParams* p, const VmoeAttnArgs* a, const AttnGeom& g) {
  memset(p, 0, sizeof(*p));
  p->out = static_cast<__nv_bfloat16*>(a->out);
  p->lse = a->lse;
  p->o_tok = a->o_tok;
  p->o_head = a->o_head;
  p->o_batch = a->o_batch;
  p->status = a->status;
  p->B = static_cast<int>(a->B);
  p->H = static_cast<int>(a->H);
  p->Tq = static_cast<int>(g.Tq);
  p->Tk = static_cast<int>(g.Tk);
  p->D = static_cast<int>(a->D);
  p->nch = static_cast<int>((a->D + 63) / 64);
  p->kr = static_cast<int>((g.Tk + 63) / 64 * 64);
  p->n_qt = static_cast<int>((g.Tq + ATT_TILE - 1) / ATT_TILE);
  p->scale = a->scale;
  // Keep probability in steps of 1/256 (one hash byte per weight); the kept weights are scaled
  // by the reciprocal of the probability that is actually applied, so the estimate is unbiased.
  int keep = static_cast<int>((1.0f - a->dropout_p) * 256.0f + 0.5f);
  if (keep < 1) keep = 1;
  if (keep > 256 || a->dropout_p <= 0.f) keep = 256;
  p->keep_q = static_cast<unsigned>(keep);
  p->inv_keep = 256.0f / static_cast<float>(keep);
  p->seed_lo = static_cast<unsigned>(a->seed & 0xffffffffu);
  p->seed_hi = static_cast<unsigned>(a->seed >> 32);
}

static int sm_count_cached() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

// attention_d64_tcgen05.cu: one-shot kernels for packed self-attention, D = 64, T <= 256.
int attention_d64_fwd(const VmoeAttnArgs* a, vmoe_stream_t stream);
int attention_d64_bwd(const VmoeAttnArgs* a, vmoe_stream_t stream);

// The shape and layout the one-shot kernels cover; VMOE_B200_ATTN_GENERAL=1 routes it to the
// general kernels instead (tests run both).
static bool use_d64_kernels(const VmoeAttnArgs* a, bool backward) {
  const char* env = getenv("VMOE_B200_ATTN_GENERAL");
  if (env != nullptr && env[0] == '1') return false;
  const bool own_kv = a->kv_tok != 0 || a->kv_head != 0 || a->kv_batch != 0;
  const bool same_kv = !own_kv || (a->kv_tok == a->q_tok && a->kv_head == a->q_head &&
                                   a->kv_batch == a->q_batch);
  const bool own_g = a->gkv_tok != 0 || a->gkv_head != 0 || a->gkv_batch != 0;
  const bool same_g = !backward || !own_g || (a->gkv_tok == a->g_tok && a->gkv_head == a->g_head &&
                                              a->gkv_batch == a->g_batch);
  return a->D == 64 && a->T >= 1 && a->T <= 256 && (a->Tk == 0 || a->Tk == a->T) && same_kv &&
         same_g && a->dropout_p <= 0.f;
}

}  // namespace vmoe

using namespace vmoe;

extern "C" int32_t vmoe_attention_supported(int64_t tq, int64_t tk, int64_t d) {
  if (d % 16 || d < 16 || d > 80 || tq < 1 || tk < 1) return 0;
  return fwd_layout(static_cast<int>(tk), static_cast<int>(d)).total <= 227 * 1024 ? 1 : 0;
}

// 1 when the backward pass of this shape needs VmoeAttnArgs.dq_acc (fp32 zeros, B*Tq*H*D).
extern "C" int32_t vmoe_attention_bwd_needs_dq_acc(int64_t tq, int64_t d) {
  return bwd_layout(static_cast<int>(tq), static_cast<int>(d)).dq_resident ? 0 : 1;
}

extern "C" int vmoe_attention_fwd(const VmoeAttnArgs* a, vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->B == 0 || a->H == 0) return 0;
  if (use_d64_kernels(a, false)) return attention_d64_fwd(a, stream_);
  AttnGeom g;
  int rc = check_attn(a, &g, false);
  if (rc) return rc;
  CUtensorMap tq, tk, tv;
  if ((rc = make_head_map(&tq, a->q, a->D, g.Tq, a->H, a->B, a->q_tok, a->q_head, a->q_batch, 128)))
    return rc;
  if ((rc = make_head_map(&tk, a->k, a->D, g.Tk, a->H, a->B, g.kv_tok, g.kv_head, g.kv_batch, 64)))
    return rc;
  if ((rc = make_head_map(&tv, a->v, a->D, g.Tk, a->H, a->B, g.kv_tok, g.kv_head, g.kv_batch, 64)))
    return rc;
  AttnParams p;
  fill_params(&p, a, g);
  const FwdLayout L = fwd_layout(p.Tk, p.D);
  static int attr_bytes = 0;
  if (L.total > attr_bytes) {
    cudaError_t e = cudaFuncSetAttribute(attention_fwd_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L.total);
    if (e != cudaSuccess) {
      set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
      return -4;
    }
    attr_bytes = L.total;
  }
  // Resident CTAs per SM: bounded by shared memory and by the TMEM columns each one allocates.
  int per_sm = (226 * 1024) / (L.total + 1024);
  if (per_sm > 512 / L.tmem_cols) per_sm = 512 / L.tmem_cols;
  if (per_sm > 4) per_sm = 4;
  if (per_sm < 1) per_sm = 1;
  const long long items = static_cast<long long>(p.B) * p.H * p.n_qt;
  const long long cap = static_cast<long long>(sm_count_cached()) * per_sm;
  const unsigned grid = static_cast<unsigned>(items < cap ? items : cap);
  attention_fwd_kernel<<<grid, FWD_THREADS, L.total, stream>>>(tq, tk, tv, p, L);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
    return -5;
  }
  return 0;
}

extern "C" int vmoe_attention_bwd(const VmoeAttnArgs* a, vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->B == 0 || a->H == 0) return 0;
  if (use_d64_kernels(a, true)) return attention_d64_bwd(a, stream_);
  AttnGeom g;
  int rc = check_attn(a, &g, true);
  if (rc) return rc;
  CUtensorMap tq, tk, tv, tdo;
  if ((rc = make_head_map(&tq, a->q, a->D, g.Tq, a->H, a->B, a->q_tok, a->q_head, a->q_batch, 128)))
    return rc;
  if ((rc = make_head_map(&tk, a->k, a->D, g.Tk, a->H, a->B, g.kv_tok, g.kv_head, g.kv_batch, 128)))
    return rc;
  if ((rc = make_head_map(&tv, a->v, a->D, g.Tk, a->H, a->B, g.kv_tok, g.kv_head, g.kv_batch, 128)))
    return rc;
  if ((rc = make_head_map(&tdo, a->d_out, a->D, g.Tq, a->H, a->B, a->o_tok, a->o_head, a->o_batch,
                          128)))
    return rc;
  AttnParams p;
  fill_params(&p, a, g);
  p.o_in = static_cast<const __nv_bfloat16*>(a->out);
  p.d_out = static_cast<const __nv_bfloat16*>(a->d_out);
  p.dq = static_cast<__nv_bfloat16*>(a->dq);
  p.dk = static_cast<__nv_bfloat16*>(a->dk);
  p.dv = static_cast<__nv_bfloat16*>(a->dv);
  p.dq_acc = a->dq_acc;
  p.gq_tok = a->g_tok;
  p.gq_head = a->g_head;
  p.gq_batch = a->g_batch;
  p.gkv_tok = g.gkv_tok;
  p.gkv_head = g.gkv_head;
  p.gkv_batch = g.gkv_batch;
  const BwdLayout L = bwd_layout(p.Tq, p.D);
  if (!L.dq_resident && a->dq_acc == nullptr) {
    set_error("%s (code %d)", "attention backward of this shape needs the fp32 dq_acc buffer", 0);
    return -1;
  }
  static int attr_bytes = 0;
  if (L.total > attr_bytes) {
    cudaError_t e = cudaFuncSetAttribute(attention_bwd_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L.total);
    if (e != cudaSuccess) {
      set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
      return -4;
    }
    attr_bytes = L.total;
  }
  const long long items = static_cast<long long>(p.B) * p.H;
  const long long cap = sm_count_cached();
  const unsigned grid = static_cast<unsigned>(items < cap ? items : cap);
  attention_bwd_kernel<<<grid, BWD_THREADS, L.total, stream>>>(tq, tk, tv, tdo, p, L);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess && !L.dq_resident) {
    const long long n8 = static_cast<long long>(p.B) * p.Tq * p.H * p.D / 8;
    attention_dq_convert_kernel<<<static_cast<unsigned>((n8 + 255) / 256), 256, 0, stream>>>(
        a->dq_acc, p.dq, n8, p.Tq, p.H, p.D, p.gq_tok, p.gq_head, p.gq_batch);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
    return -5;
  }
  return 0;
}

#ifdef ATT_TRACE
// Copies the stamps of role `who` (0 softmax warp, 1 MMA thread) as (tag, clock) pairs into
// `out` (4096 values), resets the list and returns the number of stamps.
extern "C" VMOE_API int vmoe_attention_trace_read(long long* out, int who) {
  int n = 0;
  cudaMemcpyFromSymbol(&n, g_att_trace_n, sizeof(int), who * sizeof(int));
  cudaMemcpyFromSymbol(out, g_att_trace, sizeof(long long) * 4096, who * 4096 * sizeof(long long));
  int zero = 0;
  cudaMemcpyToSymbol(g_att_trace_n, &zero, sizeof(int), who * sizeof(int));
  return n;
}
#endif
