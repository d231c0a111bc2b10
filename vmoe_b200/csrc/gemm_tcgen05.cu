// Persistent warp-specialised bf16 GEMM for sm_100a: TMA -> 128B-swizzled shared memory ->
// tcgen05.mma (UMMA 128x256x16, fp32 accumulators in TMEM, double-buffered) -> tcgen05.ld
// epilogue with bias / GELU / GELU-grad / residual / column-sum / bf16|fp32|atomic stores.
//
// Roles (320 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..9 = epilogue (warp w reads TMEM lanes 32*(w%4) .. 32*(w%4)+31 and half of the
// tile's columns). bf16 outputs leave through 64B-swizzled shared-memory staging and TMA
// stores, which clip rows and columns that fall outside the matrix.
//
// Two instantiations: one CTA per 128 x 256 tile (cta_group::1), and CTA pairs launched as
// 2-CTA clusters that share one 256 x 256 tile (cta_group::2). In a pair each CTA stages its own
// 128 rows of A and one half (128 columns) of B, the even CTA issues the MMAs for both, and
// each CTA's TMEM receives the accumulator rows of its own A tile. Per MMA every SM then moves
// 8 KB instead of 12 KB through its shared memory, which is what bounds the single-CTA tile.
//
// This one kernel covers every dense and expert matmul of the model: forward (x W^T), dgrad
// (dy W, B read MN-major) and wgrad (dy^T x, both operands MN-major, split-K with fp32
// atomics), batched over experts through the third TMA coordinate. It replaces the matmuls
// that the reference leaves to XLA (vmoe/nn/vit_moe.py:38-45 MlpBlock, vmoe/moe.py:429-444
// vmapped experts).
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "moe_push.cuh"
#include "ptx_sm100.cuh"
#include "tma_host.h"
#include "vmoe_api.h"

namespace vmoe {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KiB
constexpr int CHUNK_BYTES = 64 * BK * 2;    // one 64 x 64 MN-major box = 8 KiB
constexpr int TMEM_COLS = 512;              // two 128 x 256 fp32 accumulators
constexpr int EPI_WARPS = 8;                // two per TMEM lane quadrant, 128 columns each
constexpr int GEMM_THREADS = 64 + 32 * EPI_WARPS;
constexpr int EPI_CHUNK_BYTES = 32 * 32 * 2;  // 32 rows x 32 bf16 columns
// Staging per epilogue warp: two 32 x 32 tiles (64 B swizzled rows) for C and the second output /
// epilogue input. (Measured: 32 x 64 tiles with 128-byte rows for every output, paid for with one
// pipeline stage less in pair mode, did not make the K = 768 GEMMs faster and cost the long-K
// ones 5 %; knocking out the stores alone gains 10-15 %, their requests' size does not matter.)
constexpr int EPI_WARP_BYTES = 2 * EPI_CHUNK_BYTES;
constexpr int EPI_WARP_BYTES_PAIR = 2 * EPI_CHUNK_BYTES;
constexpr int STAGES_PAIR = 6;                   // pair mode stages half of B per CTA
constexpr int B_HALF_BYTES = B_STAGE_BYTES / 2;  // 16 KiB
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + EPI_WARPS * EPI_WARP_BYTES +
                           1024 /*align*/ + 256;
// Pair mode with the fused row push: one pipeline stage less, its 32 KiB hold the rings of the
// two push warps (warps 10 and 11 of a 384-thread CTA); their small metadata follows the barriers.
constexpr int STAGES_PAIR_PUSH = STAGES_PAIR - 1;
constexpr int PUSH_WARPS_PER_CTA = 2;
constexpr int GEMM_THREADS_PUSH = GEMM_THREADS + 32 * PUSH_WARPS_PER_CTA;
constexpr int SMEM_BYTES_PUSH = SMEM_BYTES + PUSH_WARPS_PER_CTA * PUSH_META_BYTES;
static_assert(PUSH_WARPS_PER_CTA * PUSH_RING_BYTES == A_STAGE_BYTES + B_HALF_BYTES,
              "the push rings take the place of one pipeline stage");
static_assert(SMEM_BYTES_PUSH <= 227 * 1024, "shared memory budget");
static_assert(STAGES_PAIR * (A_STAGE_BYTES + B_HALF_BYTES) + EPI_WARPS * EPI_WARP_BYTES_PAIR ==
                  STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + EPI_WARPS * EPI_WARP_BYTES,
              "both modes use the same shared-memory budget");

struct GemmParams {
  void* C;
  void* C2;
  const float* bias;
  const __nv_bfloat16* residual;
  const __nv_bfloat16* gelu_pre;
  float* colsum;
  const unsigned* a_ready;
  unsigned* status;
  long long ldc, ldr, ldr2;
  long long c_batch_stride, bias_batch_stride, r_batch_stride;
  int M, N, K, batch;
  int a_mn_major, b_mn_major;
  int c_fp32, c_atomic, act, split_k;
  unsigned a_ready_epoch;
  int tma_store;  // bf16 outputs go through smem staging + TMA stores
  int c2_gelu_grad;  // C2 receives gelu'(pre-activation) instead of the pre-activation
  int pre_is_grad;   // gelu_pre already holds gelu'(x): plain multiply
  int mt_offset;     // rotation of the m-tile order
  int c_multi_rows;  // > 0: rows per destination block of the multi-destination output
  int signal_count;  // > 0: the last GEMM CTA to finish bumps signal_flags[0 .. signal_count)
  unsigned* done_counter;
  unsigned* signal_flags[8];
};

// Output split over several destinations (row block j of every batch goes to destination j).
constexpr int MAX_C_DESTS = 8;
struct CMultiMaps {
  CUtensorMap m[MAX_C_DESTS];
};

struct TileCoord {
  int b, mt, nt, ks;
};

__device__ __forceinline__ TileCoord decode_tile(int tile, int num_m, int num_n, int split_k,
                                                 int mt_offset = 0) {
  // n fastest, then split, then m, then batch: CTAs that run together share an A panel
  // through L2 while the (small) B matrix stays L2 resident.
  TileCoord t;
  t.nt = tile % num_n;
  tile /= num_n;
  t.ks = tile % split_k;
  tile /= split_k;
  t.mt = (tile % num_m + mt_offset) % num_m;
  t.b = tile / num_m;
  return t;
}

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Sum v[i] over the 32 lanes of the warp for all 32 register columns with 31 shuffles; on
// return lane L holds the total of column L in v[0].
__device__ __forceinline__ void warp_transpose_reduce(float (&v)[32], int lane) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int j = 0; j < off; ++j) {
      float send = upper ? v[j] : v[j + off];
      float keep = upper ? v[j + off] : v[j];
      v[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
}

template <bool PAIR, bool PUSHW>
__global__ void __launch_bounds__(PUSHW ? GEMM_THREADS_PUSH : GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ CUtensorMap tma_c, const __grid_constant__ CUtensorMap tma_c2,
                 const __grid_constant__ CMultiMaps cmaps, const GemmParams p,
                 const PushParams pp) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  static_assert(PAIR || !PUSHW, "the fused push needs the pair mode's shared-memory layout");
  constexpr int NSTAGE = PAIR ? (PUSHW ? STAGES_PAIR_PUSH : STAGES_PAIR) : STAGES;
  constexpr int BSTAGE = PAIR ? B_HALF_BYTES : B_STAGE_BYTES;  // B bytes this CTA stages
  constexpr int B_ROWS = PAIR ? BN / 2 : BN;                   // N rows of B this CTA stages
  constexpr int TM = PAIR ? 2 * BM : BM;                       // rows of one tile
  uint8_t* sA = smem;
  uint8_t* sB = smem + NSTAGE * A_STAGE_BYTES;
  uint8_t* sEpi = smem + NSTAGE * (A_STAGE_BYTES + BSTAGE);
  constexpr int EPI_WARP = PAIR ? EPI_WARP_BYTES_PAIR : EPI_WARP_BYTES;
  uint8_t* sPush = sEpi + EPI_WARPS * EPI_WARP;  // rings of the push warps (PUSHW only)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sPush + (PUSHW ? PUSH_WARPS_PER_CTA * PUSH_RING_BYTES : 0));
  // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * NSTAGE + 4);
  // Pair mode: rank 0 (the even CTA) leads. `cta` / `ncta` index tiles per CTA or per pair.
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const int cta = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int ncta = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = smem_u32(bars + NSTAGE);
  const uint32_t bar_tfull = smem_u32(bars + 2 * NSTAGE);
  const uint32_t bar_tempty = smem_u32(bars + 2 * NSTAGE + 2);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_tfull + 8 * s, 1);
      // one arrival per epilogue warp (of both CTAs in pair mode; only the leader's is used)
      mbar_init(bar_tempty + 8 * s, PAIR ? 2 * EPI_WARPS : EPI_WARPS);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    if (p.tma_store) {
      tma_prefetch_desc(&tma_c);
      if (p.C2) tma_prefetch_desc(&tma_c2);
    }
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  // Pair mode: the peer's barriers must be initialised before anything arrives on them.
  if (PAIR) cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_m = (p.M + TM - 1) / TM;
  const int num_m128 = (p.M + BM - 1) / BM;
  const int mt_rot = PAIR ? p.mt_offset / 2 : p.mt_offset;
  const int num_n = (p.N + BN - 1) / BN;
  const int k_tiles = (p.K + BK - 1) / BK;
  const int k_per_split = (k_tiles + p.split_k - 1) / p.split_k;
  const int num_tiles = p.batch * num_m * num_n * p.split_k;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // Pair mode: completion bytes of both CTAs are counted on the leader's full barrier.
      const uint32_t full_base = PAIR ? mapa_shared(bar_full, 0) : bar_full;
      for (int tile = cta; tile < num_tiles && ok; tile += ncta) {
        const TileCoord t = decode_tile(tile, num_m, num_n, p.split_k, mt_rot);
        const int m0 = t.mt * TM + static_cast<int>(rank) * BM;
        const int n0 = t.nt * BN + static_cast<int>(rank) * B_ROWS;  // this CTA's rows of B
        const int kt0 = t.ks * k_per_split;
        const int kt1 = min(k_tiles, kt0 + k_per_split);
        if (p.a_ready != nullptr && kt0 < kt1 && m0 < p.M) {
          // Rows of this A tile are produced by another kernel (possibly on a peer GPU) that
          // adds the number of rows it wrote to a counter, release at system scope.
          const unsigned rows = static_cast<unsigned>(min(BM, p.M - m0));
          const unsigned want = p.a_ready_epoch * rows;
          const unsigned* flag = p.a_ready + (static_cast<long long>(t.b) * num_m128 + m0 / BM);
          const long long t0 = clock64();
          while (static_cast<int>(ld_acquire_sys(flag) - want) < 0) {
            if (*abort_flag || clock64() - t0 > kWaitLimitCycles) {
              *abort_flag = 1;
              if (p.status) atomicOr(p.status, kStatusTimeoutFlag);
              ok = false;
              break;
            }
            __nanosleep(64);
          }
          if (!ok) break;
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kt = kt0; kt < kt1; ++kt) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.status,
                         kStatusTimeoutProducer)) {
            ok = false;
            break;
          }
          const uint32_t full = full_base + 8 * stage;
          if (!PAIR) {
            mbar_expect_tx(full, A_STAGE_BYTES + BSTAGE);
          } else if (rank == 0) {
            mbar_expect_tx(bar_full + 8 * stage, 2 * (A_STAGE_BYTES + BSTAGE));
          }
          const uint32_t a_dst = smem_u32(sA + stage * A_STAGE_BYTES);
          const uint32_t b_dst = smem_u32(sB + stage * BSTAGE);
          const int k0 = kt * BK;
          auto load = [&](uint32_t dst, const CUtensorMap* map, int c0, int c1) {
            if (PAIR) {
              tma_load_3d_pair(dst, map, full, c0, c1, t.b);
            } else {
              tma_load_3d(dst, map, full, c0, c1, t.b);
            }
          };
          if (!p.a_mn_major) {
            load(a_dst, &tma_a, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) load(a_dst + j * CHUNK_BYTES, &tma_a, m0 + 64 * j, k0);
          }
          if (!p.b_mn_major) {
            load(b_dst, &tma_b, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < B_ROWS / 64; ++j)
              load(b_dst + j * CHUNK_BYTES, &tma_b, n0 + 64 * j, k0);
          }
          if (++stage == NSTAGE) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // Give copies that are still in flight a bounded chance to land before the CTA exits.
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) __nanosleep(256);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc_bf16(TM, BN, p.a_mn_major, p.b_mn_major);
      // K-major: 8-row groups 1024 B apart, 32 B per UMMA_K step inside the swizzle row.
      // MN-major: 64-element chunks CHUNK_BYTES apart (LBO), 8-row K groups 1024 B apart
      // (SBO), 16 K rows = 2048 B per UMMA_K step.
      const uint32_t a_lbo = p.a_mn_major ? CHUNK_BYTES : 16, a_step = p.a_mn_major ? 2048 : 32;
      const uint32_t b_lbo = p.b_mn_major ? CHUNK_BYTES : 16, b_step = p.b_mn_major ? 2048 : 32;
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += ncta, ++local) {
        const TileCoord t = decode_tile(tile, num_m, num_n, p.split_k, mt_rot);
        const int kt0 = t.ks * k_per_split;
        const int kt1 = min(k_tiles, kt0 + k_per_split);
        const int slot = local & 1;
        const uint32_t use = static_cast<uint32_t>(local >> 1);
        if (!mbar_wait(bar_tempty + 8 * slot, (use & 1) ^ 1, abort_flag, p.status,
                       kStatusTimeoutMma)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + slot * BN;
        for (int kt = kt0; kt < kt1; ++kt) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, kStatusTimeoutMma)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * A_STAGE_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * BSTAGE);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = umma_smem_desc(a_addr + k * a_step, a_lbo, 1024);
            const uint64_t bdesc = umma_smem_desc(b_addr + k * b_step, b_lbo, 1024);
            if (PAIR) {
              umma_bf16_pair(d_tmem, adesc, bdesc, idesc, (kt > kt0 || k > 0) ? 1u : 0u);
            } else {
              umma_bf16(d_tmem, adesc, bdesc, idesc, (kt > kt0 || k > 0) ? 1u : 0u);
            }
          }
          // Frees the smem stage (in both CTAs of a pair) once these MMAs retire.
          if (PAIR) {
            umma_commit_pair(bar_empty + 8 * stage, 3);
          } else {
            umma_commit(bar_empty + 8 * stage);
          }
          if (++stage == NSTAGE) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        // accumulator complete -> epilogue (of both CTAs in pair mode)
        if (PAIR) {
          umma_commit_pair(bar_tfull + 8 * slot, 3);
        } else {
          umma_commit(bar_tfull + 8 * slot);
        }
      }
    }
  } else if (PUSHW && warp >= 2 + EPI_WARPS) {
    // ------------------------------------------------------------------ row push
    // Two warps of every CTA deliver this rank's rows to the expert owners (this GPU included)
    // while the other warps multiply the tiles that have arrived.
    const int pw = warp - (2 + EPI_WARPS);
    uint8_t* meta = reinterpret_cast<uint8_t*>(bars) + 256 + pw * PUSH_META_BYTES;
    push_rows_ring(pp, sPush + pw * PUSH_RING_BYTES, meta, lane,
                   static_cast<int>(blockIdx.x) * PUSH_WARPS_PER_CTA + pw,
                   static_cast<int>(gridDim.x) * PUSH_WARPS_PER_CTA, p.status);
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;         // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;  // which 128 columns of the tile this warp handles
    uint8_t* stage_c = sEpi + (warp - 2) * EPI_WARP;
    uint8_t* stage_c2 = stage_c + EPI_WARP / 2;
    // Wide staging (multi-destination output): two 32-column chunks share one 32 x 64 tile with
    // 128-byte swizzled rows, spanning both 32 x 32 staging tiles, and leave in one TMA store.
    const bool wide = p.c_multi_rows > 0;
    const uint32_t wrow = static_cast<uint32_t>(lane) * 128u;
    const uint32_t wxor = static_cast<uint32_t>(lane) & 7u;
    // 64B-swizzled position of this lane's row inside a 32 x 32 bf16 staging tile.
    const uint32_t st_row = static_cast<uint32_t>(lane) * 64u;
    const uint32_t st_xor = (static_cast<uint32_t>(lane) >> 1) & 3u;
    int local = 0;
    bool ok = true;
    const uint32_t tempty_base = PAIR ? mapa_shared(bar_tempty, 0) : bar_tempty;
    for (int tile = cta; tile < num_tiles && ok; tile += ncta, ++local) {
      const TileCoord t = decode_tile(tile, num_m, num_n, p.split_k, mt_rot);
      const int kt0 = t.ks * k_per_split;
      const int kt1 = min(k_tiles, kt0 + k_per_split);
      const int slot = local & 1;
      const uint32_t use = static_cast<uint32_t>(local >> 1);
      const bool got = mbar_wait(bar_tfull + 8 * slot, use & 1, abort_flag, p.status,
                                 kStatusTimeoutEpilogue);
      if (!__all_sync(0xffffffffu, got)) {  // warp-uniform so the aligned TMEM loads converge
        ok = false;
        break;
      }
      tc_fence_after();
      const bool empty_k = kt0 >= kt1;  // a split with no K tiles contributes nothing
      const int row0 = t.mt * TM + static_cast<int>(rank) * BM + quad * 32;
      const int row = row0 + lane;
      const bool row_ok = row < p.M;
      const int n0 = t.nt * BN;
      const long long crow = static_cast<long long>(t.b) * p.c_batch_stride +
                             static_cast<long long>(row) * p.ldc;
      const float* bias = p.bias ? p.bias + static_cast<long long>(t.b) * p.bias_batch_stride
                                 : nullptr;
      // Only the first split adds bias/residual so that atomically summed splits count them once.
      const bool first_split = t.ks == 0;
      // Epilogue input tile (gelu_pre or residual): fetched one chunk ahead with coalesced
      // 16-byte loads (8 rows x 64 B per instruction), then re-distributed to one row per lane
      // through the (otherwise unused) second staging tile.
      const __nv_bfloat16* in_ptr = nullptr;
      long long in_ld = 0;
      if (!p.C2 && !(p.gelu_pre && p.residual)) {
        if (p.gelu_pre) {
          in_ptr = p.gelu_pre;
          in_ld = p.ldr2;
        } else if (p.residual && first_split) {
          in_ptr = p.residual;
          in_ld = p.ldr;
        }
        if (in_ld % 8 || p.N % 8) in_ptr = nullptr;
      }
      const int pf_r = lane >> 2, pf_c = lane & 3;
      uint4 pf[4];
      auto prefetch_input = [&](int cc) {
        const int colp = n0 + cc * 32 + pf_c * 8;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int rw = row0 + pf_r + 8 * i;
          pf[i] = make_uint4(0, 0, 0, 0);
          if (rw < p.M && colp + 8 <= p.N)
            pf[i] = __ldg(reinterpret_cast<const uint4*>(
                in_ptr + static_cast<long long>(t.b) * p.r_batch_stride +
                static_cast<long long>(rw) * in_ld + colp));
        }
      };
      if (in_ptr && n0 + half * 128 < p.N) prefetch_input(half * 4);
      // Writes this lane's 32 values (one row of a chunk) as bf16 into a staging tile.
      auto stage_row = [&](uint8_t* tile, const float (&x)[32], int c) {
        const uint32_t cc = static_cast<uint32_t>(c & 1);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 q;
          q.x = pack_bf16x2(x[8 * i + 0], x[8 * i + 1]);
          q.y = pack_bf16x2(x[8 * i + 2], x[8 * i + 3]);
          q.z = pack_bf16x2(x[8 * i + 4], x[8 * i + 5]);
          q.w = pack_bf16x2(x[8 * i + 6], x[8 * i + 7]);
          if (wide) {
            *reinterpret_cast<uint4*>(tile + wrow + (((4u * cc + i) ^ wxor) << 4)) = q;
          } else {
            *reinterpret_cast<uint4*>(tile + st_row + ((static_cast<uint32_t>(i) ^ st_xor) << 4)) = q;
          }
        }
      };
#pragma unroll 1
      for (int c = half * 4; c < half * 4 + 4; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;
        uint4 in_row[4];
        if (in_ptr) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t rr = static_cast<uint32_t>(pf_r + 8 * i);
            *reinterpret_cast<uint4*>(stage_c2 + rr * 64u +
                                      ((static_cast<uint32_t>(pf_c) ^ ((rr >> 1) & 3u)) << 4)) = pf[i];
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 4; ++i)
            in_row[i] = *reinterpret_cast<const uint4*>(
                stage_c2 + st_row + ((static_cast<uint32_t>(i) ^ st_xor) << 4));
          __syncwarp();
          if (c + 1 < half * 4 + 4 && col0 + 32 < p.N) prefetch_input(c + 1);
        }
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + slot * BN + c * 32,
                      r);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = empty_k ? 0.0f : __uint_as_float(r[i]);
        const bool full_cols = col0 + 32 <= p.N;
        if (bias && first_split) {
          if (full_cols) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 b4 = __ldg(reinterpret_cast<const float4*>(bias + col0) + i);
              v[4 * i + 0] += b4.x;
              v[4 * i + 1] += b4.y;
              v[4 * i + 2] += b4.z;
              v[4 * i + 3] += b4.w;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i < p.N) v[i] += __ldg(bias + col0 + i);
          }
        }
        if (p.tma_store) {
          // The staging tiles are reused every chunk: wait until the TMA engine has read the
          // previous contents.
          if (!wide || (c & 1) == 0) {
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            __syncwarp();
          }
        }
        const bool vec_bf16 = full_cols && (p.ldc % 8 == 0);
        if (p.C2 && p.c2_gelu_grad) {
          // Fused forward: C = gelu(v) and C2 = gelu'(v) share one tanh.
          float a[32];
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            gelu_and_grad_pair(v[i], v[i + 1], a[i], a[i + 1], v[i], v[i + 1]);
          // v now holds gelu' (stored to C2 below); a holds the activation (restored after).
          if (p.tma_store) {
            stage_row(stage_c2, v, c);
          } else if (row_ok) {
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C2) + crow + col0;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i < p.N) out[i] = __float2bfloat16(v[i]);
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = a[i];
        } else if (p.C2) {
          if (p.tma_store) {
            stage_row(stage_c2, v, c);
          } else if (row_ok) {
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C2) + crow + col0;
            if (vec_bf16) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint4 q;
                q.x = pack_bf16x2(v[8 * i + 0], v[8 * i + 1]);
                q.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
                q.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
                q.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
                reinterpret_cast<uint4*>(out)[i] = q;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N) out[i] = __float2bfloat16(v[i]);
            }
          }
        }
        if (p.act == 1 && !(p.C2 && p.c2_gelu_grad)) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) gelu_pair(v[i], v[i + 1], v[i], v[i + 1]);
        }
        if (p.gelu_pre && row_ok) {
          const __nv_bfloat16* pre = p.gelu_pre + static_cast<long long>(t.b) * p.r_batch_stride +
                                     static_cast<long long>(row) * p.ldr2 + col0;
          if (in_ptr == p.gelu_pre || (full_cols && (p.ldr2 % 8 == 0))) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint4 q = (in_ptr == p.gelu_pre)
                                  ? in_row[i]
                                  : __ldg(reinterpret_cast<const uint4*>(pre) + i);
              const float2 f0 = unpack_bf16x2(q.x), f1 = unpack_bf16x2(q.y);
              const float2 f2 = unpack_bf16x2(q.z), f3 = unpack_bf16x2(q.w);
              if (p.pre_is_grad) {
                v[8 * i + 0] *= f0.x;
                v[8 * i + 1] *= f0.y;
                v[8 * i + 2] *= f1.x;
                v[8 * i + 3] *= f1.y;
                v[8 * i + 4] *= f2.x;
                v[8 * i + 5] *= f2.y;
                v[8 * i + 6] *= f3.x;
                v[8 * i + 7] *= f3.y;
              } else {
                float d0, d1;
                gelu_grad_pair(f0.x, f0.y, d0, d1);
                v[8 * i + 0] *= d0;
                v[8 * i + 1] *= d1;
                gelu_grad_pair(f1.x, f1.y, d0, d1);
                v[8 * i + 2] *= d0;
                v[8 * i + 3] *= d1;
                gelu_grad_pair(f2.x, f2.y, d0, d1);
                v[8 * i + 4] *= d0;
                v[8 * i + 5] *= d1;
                gelu_grad_pair(f3.x, f3.y, d0, d1);
                v[8 * i + 6] *= d0;
                v[8 * i + 7] *= d1;
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i < p.N) {
                const float pv = __bfloat162float(pre[i]);
                v[i] *= p.pre_is_grad ? pv : gelu_tanh_grad(pv);
              }
          }
        }
        if (p.residual && row_ok && first_split) {
          const __nv_bfloat16* res = p.residual + static_cast<long long>(t.b) * p.r_batch_stride +
                                     static_cast<long long>(row) * p.ldr + col0;
          if (in_ptr == p.residual || (full_cols && (p.ldr % 8 == 0))) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint4 q = (in_ptr == p.residual)
                                  ? in_row[i]
                                  : __ldg(reinterpret_cast<const uint4*>(res) + i);
              const float2 f0 = unpack_bf16x2(q.x), f1 = unpack_bf16x2(q.y);
              const float2 f2 = unpack_bf16x2(q.z), f3 = unpack_bf16x2(q.w);
              v[8 * i + 0] += f0.x;
              v[8 * i + 1] += f0.y;
              v[8 * i + 2] += f1.x;
              v[8 * i + 3] += f1.y;
              v[8 * i + 4] += f2.x;
              v[8 * i + 5] += f2.y;
              v[8 * i + 6] += f3.x;
              v[8 * i + 7] += f3.y;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i < p.N) v[i] += __bfloat162float(res[i]);
          }
        }
        if (p.tma_store && wide) {
          // Two 32-column chunks share one 32 x 64 staging tile (128-byte rows, 128B swizzle) and
          // leave in one store per output, so that memory (or, for a multi-destination output,
          // the NVLink to a peer GPU) sees 128-byte row segments instead of 64-byte ones.
          const int cc = c & 1;
          stage_row(stage_c, v, c);
          if (cc == 1 || col0 + 32 >= p.N) {
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              const int x0 = col0 - 32 * cc;
              if (p.c_multi_rows > 0) {
                // Boxes that start past the last row have no destination (and no map): skip.
                if (row0 < p.M) {
                  const int j = row0 / p.c_multi_rows;
                  tma_store_3d(&cmaps.m[j], smem_u32(stage_c), x0, row0 - j * p.c_multi_rows, t.b);
                }
              } else {
                tma_store_3d(&tma_c, smem_u32(stage_c), x0, row0, t.b);
                if (p.C2) tma_store_3d(&tma_c2, smem_u32(stage_c2), x0, row0, t.b);
              }
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          }
        } else if (p.tma_store) {
          stage_row(stage_c, v, c);
          fence_proxy_async();  // make the staged tile visible to the TMA engine
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(&tma_c, smem_u32(stage_c), col0, row0, t.b);
            if (p.C2) tma_store_3d(&tma_c2, smem_u32(stage_c2), col0, row0, t.b);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        } else if (row_ok) {
          if (!p.c_fp32) {
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + crow + col0;
            if (vec_bf16) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint4 q;
                q.x = pack_bf16x2(v[8 * i + 0], v[8 * i + 1]);
                q.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
                q.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
                q.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
                reinterpret_cast<uint4*>(out)[i] = q;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N) out[i] = __float2bfloat16(v[i]);
            }
          } else {
            float* out = reinterpret_cast<float*>(p.C) + crow + col0;
            if (p.c_atomic && p.split_k == 1) {
              // Accumulating output without split-K: every element belongs to this thread alone,
              // so it is read, added and written back with plain 16-byte accesses. (Atomics cost
              // 12x the store time on the weight gradients of 128 experts: 1.2 GB of output.)
              if (full_cols && (p.ldc % 4 == 0)) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  float4 o = reinterpret_cast<float4*>(out)[i];
                  o.x += v[4 * i];
                  o.y += v[4 * i + 1];
                  o.z += v[4 * i + 2];
                  o.w += v[4 * i + 3];
                  reinterpret_cast<float4*>(out)[i] = o;
                }
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (col0 + i < p.N) out[i] += v[i];
              }
            } else if (p.c_atomic) {
              // Split-K: the pieces of a tile meet in the output. 16-byte vector atomics where the
              // row allows them: a quarter of the requests of scalar ones.
              if (full_cols && (p.ldc % 4 == 0)) {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  atomicAdd(reinterpret_cast<float4*>(out) + i,
                            make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]));
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (col0 + i < p.N) atomicAdd(out + i, v[i]);
              }
            } else if (full_cols && (p.ldc % 4 == 0)) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                reinterpret_cast<float4*>(out)[i] =
                    make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N) out[i] = v[i];
            }
          }
        }
        if (p.colsum) {
          if (!row_ok) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0.0f;
          }
          warp_transpose_reduce(v, lane);
          if (col0 + lane < p.N)
            atomicAdd(p.colsum + static_cast<long long>(t.b) * p.bias_batch_stride + col0 + lane,
                      v[0]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) {
          mbar_arrive_cluster(tempty_base + 8 * slot);
        } else {
          mbar_arrive(bar_tempty + 8 * slot);
        }
      }
    }
    // Outstanding TMA stores must finish reading shared memory before the CTA exits.
    if (p.tma_store && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  tc_fence_before();
  __syncthreads();
  if (p.signal_count > 0 && threadIdx.x == 0) {
    // Every epilogue warp has waited for its own output stores (bulk wait above, plain stores
    // are ordered by the barrier). The CTA that takes the last ticket tells the destinations.
    __threadfence_system();
    if (atomicAdd(p.done_counter, 1u) == gridDim.x - 1) {
      *p.done_counter = 0;
      asm volatile("fence.proxy.async.global;" ::: "memory");
      __threadfence_system();
      for (int i = 0; i < p.signal_count; ++i)
        asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.signal_flags[i]), "r"(1u)
                     : "memory");
    }
  }
  if (PAIR) {
    // Neither CTA may free TMEM or exit while its peer can still touch its barriers or TMEM.
    cluster_sync_all();
  }
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) {
      tmem_dealloc_pair(tmem_base, TMEM_COLS);
    } else {
      tmem_dealloc(tmem_base, TMEM_COLS);
    }
  }
}

// ------------------------------------------------------------------------------- host side
static thread_local char g_err[512] = "";

void set_error(const char* fmt, const char* a, int code) {
  snprintf(g_err, sizeof(g_err), fmt, a, code);
}

// bf16 matrix stored [batch][rows][ld] viewed as a 3-D tensor (inner, rows, batch) with a
// 64-element (128 B) swizzled inner box.
int make_bf16_map(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t rows, uint64_t batch,
                  uint64_t ld_elems, uint64_t batch_stride_elems, uint32_t box_rows,
                  uint32_t box_inner = 64, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  cuuint64_t dims[3] = {inner, rows, batch};
  cuuint64_t strides[2] = {ld_elems * 2, (batch > 1 ? batch_stride_elems : rows * ld_elems) * 2};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = tma_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr),
                                dims, strides, box, estr, swizzle);
  if (r != CUDA_SUCCESS) {
    set_error("%s (code %d)", "cuTensorMapEncodeTiled failed", static_cast<int>(r));
    return -3;
  }
  return 0;
}

int fill_push_params(const VmoePushArgs* a, PushParams* p);      // moe_p2p.cu
int launch_push_rows_plain(const PushParams& p, cudaStream_t stream);  // moe_p2p.cu

}  // namespace vmoe

extern "C" const char* vmoe_last_error(void) { return vmoe::g_err; }

extern "C" int vmoe_gemm_bf16(const VmoeGemmArgs* a, vmoe_stream_t stream_) {
  using namespace vmoe;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  g_err[0] = 0;
  if (a->M <= 0 || a->N <= 0 || a->K <= 0 || a->batch <= 0) return 0;  // nothing to do
  if ((a->lda % 8) || (a->ldb % 8) || (reinterpret_cast<uintptr_t>(a->A) & 15) ||
      (reinterpret_cast<uintptr_t>(a->B) & 15) || (a->a_batch_stride % 8) ||
      (a->b_batch_stride % 8)) {
    set_error("%s (code %d)", "gemm operands must be 16-byte aligned with ld % 8 == 0", 0);
    return -1;
  }
  if ((a->split_k > 1 || a->c_atomic) && !(a->c_fp32 && a->c_atomic)) {
    set_error("%s (code %d)", "split_k / atomic output needs c_fp32 and c_atomic", 0);
    return -1;
  }
  static int sm_count = 0;
  static int max_pairs = 0;  // CTA pairs (2-CTA clusters) that can be resident at once
  static bool attr_set = false;
  if (!attr_set) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<false, false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemm_bf16_kernel<true, false>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemm_bf16_kernel<true, true>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES_PUSH);
    if (e != cudaSuccess) {
      set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
      return -4;
    }
    cudaLaunchConfig_t probe;
    memset(&probe, 0, sizeof(probe));
    cudaLaunchAttribute pattr;
    pattr.id = cudaLaunchAttributeClusterDimension;
    pattr.val.clusterDim.x = 2;
    pattr.val.clusterDim.y = 1;
    pattr.val.clusterDim.z = 1;
    probe.gridDim = dim3(static_cast<unsigned>(sm_count & ~1));
    probe.blockDim = dim3(GEMM_THREADS);
    probe.dynamicSmemBytes = SMEM_BYTES;
    probe.attrs = &pattr;
    probe.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, gemm_bf16_kernel<true, false>, &probe) != cudaSuccess) {
      cudaGetLastError();
      clusters = 0;
    }
    max_pairs = clusters;
    attr_set = true;
  }
  const char* env_pair = getenv("VMOE_B200_GEMM_PAIR");  // "0" / "1" override for experiments
  int pair_mode = a->cta_pair;
  if (pair_mode == 0 && env_pair != nullptr) pair_mode = env_pair[0] == '0' ? 1 : 2;
  bool pair = false;
  if (max_pairs > 0) {
    if (pair_mode == 2) {
      pair = true;
    } else if (pair_mode == 0) {
      // Pairs pay off once there is at least one 256 x 256 tile per pair of SMs.
      const long long pair_tiles = a->batch * ((a->M + 2 * BM - 1) / (2 * BM)) *
                                   ((a->N + BN - 1) / BN) * (a->split_k > 1 ? a->split_k : 1);
      pair = a->M >= 2 * BM && a->N >= BN / 2 && pair_tiles >= max_pairs / 2;
    }
  }
  PushParams pp;
  memset(&pp, 0, sizeof(pp));
  bool fused_push = false;
  if (a->push != nullptr) {
    const VmoePushArgs* pa = static_cast<const VmoePushArgs*>(a->push);
    if (pa->groups * pa->e * pa->c > 0) {
      int prc = fill_push_params(pa, &pp);
      if (prc) return prc;
      const char* env_fuse = getenv("VMOE_B200_FUSED_PUSH");  // "0": always a separate launch
      // Rows that must be scaled (backward of combine) keep two warps per SM busy for longer
      // than the GEMM runs (measured), so that push stays a launch of its own unless forced
      // with VMOE_B200_FUSED_PUSH=2.
      const bool force = env_fuse != nullptr && env_fuse[0] == '2';
      fused_push = pair && a->a_ready != nullptr &&
                   push_rows_per_slot(pp.h, pp.weight != nullptr && pp.ybuf_base != nullptr) >= 1 &&
                   !(env_fuse != nullptr && env_fuse[0] == '0') &&
                   (pp.weight == nullptr || force);
      if (!fused_push) {
        prc = launch_push_rows_plain(pp, stream);
        if (prc) return prc;
      }
    }
  }
  if (a->signal_count < 0 || a->signal_count > 8 || (a->signal_count > 0 && !a->done_counter)) {
    set_error("%s (code %d)", "completion signal needs 1..8 flags and a done_counter", 0);
    return -1;
  }
  CUtensorMap ma, mb;
  int rc;
  if (!a->a_mn_major)
    rc = make_bf16_map(&ma, a->A, a->K, a->M, a->batch, a->lda, a->a_batch_stride, BM);
  else
    rc = make_bf16_map(&ma, a->A, a->M, a->K, a->batch, a->lda, a->a_batch_stride, BK);
  if (rc) return rc;
  if (!a->b_mn_major)
    rc = make_bf16_map(&mb, a->B, a->K, a->N, a->batch, a->ldb, a->b_batch_stride,
                       pair ? BN / 2 : BN);
  else
    rc = make_bf16_map(&mb, a->B, a->N, a->K, a->batch, a->ldb, a->b_batch_stride, BK);
  if (rc) return rc;

  // bf16 outputs: 32 x 32 boxes with 64B swizzle, written by TMA from the epilogue staging.
  CUtensorMap mc, mc2;
  memset(&mc, 0, sizeof(mc));
  memset(&mc2, 0, sizeof(mc2));
  const bool tma_store = !a->c_fp32 && (a->ldc % 8 == 0) && (a->c_batch_stride % 8 == 0) &&
                         !(reinterpret_cast<uintptr_t>(a->C) & 15) &&
                         (a->C2 == nullptr || !(reinterpret_cast<uintptr_t>(a->C2) & 15));
  if (tma_store) {
    const uint32_t box_w = 32;
    const CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_64B;
    rc = make_bf16_map(&mc, a->C, a->N, a->M, a->batch, a->ldc, a->c_batch_stride, 32, box_w, sw);
    if (rc) return rc;
    if (a->C2) {
      rc = make_bf16_map(&mc2, a->C2, a->N, a->M, a->batch, a->ldc, a->c_batch_stride, 32, box_w,
                         sw);
      if (rc) return rc;
    }
  }
  static CMultiMaps cm_zero;  // zero-initialised; copied when the output has one destination
  CMultiMaps cm = cm_zero;
  int c_multi_rows = 0;
  if (a->c_multi_count > 0) {
    if (!tma_store || a->C2 != nullptr || a->residual != nullptr || a->gelu_pre != nullptr ||
        a->c_multi_count > MAX_C_DESTS ||
        a->c_multi_rows <= 0 || a->c_multi_rows % 32 ||
        a->c_multi_rows * a->c_multi_count < a->M) {
      set_error("%s (code %d)",
                "multi-destination output needs bf16 TMA stores, no second output / residual / "
                "gelu_pre, <= 8 destinations and a row block that is a multiple of 32", 0);
      return -1;
    }
    for (int j = 0; j < a->c_multi_count; ++j) {
      if (reinterpret_cast<uintptr_t>(a->c_multi[j]) & 15) {
        set_error("%s (code %d)", "multi-destination output bases must be 16-byte aligned", j);
        return -1;
      }
      rc = make_bf16_map(&cm.m[j], a->c_multi[j], a->N, a->c_multi_rows, a->batch, a->ldc,
                         a->c_batch_stride, 32, 64, CU_TENSOR_MAP_SWIZZLE_128B);
      if (rc) return rc;
    }
    c_multi_rows = static_cast<int>(a->c_multi_rows);
  }
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.c_multi_rows = c_multi_rows;
  p.tma_store = tma_store ? 1 : 0;
  p.C = a->C;
  p.C2 = a->C2;
  p.bias = a->bias;
  p.residual = static_cast<const __nv_bfloat16*>(a->residual);
  p.gelu_pre = static_cast<const __nv_bfloat16*>(a->gelu_pre);
  p.colsum = a->colsum;
  p.a_ready = a->a_ready;
  p.status = a->status;
  p.ldc = a->ldc;
  p.ldr = a->ldr;
  p.ldr2 = a->ldr2;
  p.c_batch_stride = a->c_batch_stride;
  p.bias_batch_stride = a->bias_batch_stride;
  p.r_batch_stride = a->r_batch_stride;
  p.M = static_cast<int>(a->M);
  p.N = static_cast<int>(a->N);
  p.K = static_cast<int>(a->K);
  p.batch = static_cast<int>(a->batch);
  p.a_mn_major = a->a_mn_major;
  p.b_mn_major = a->b_mn_major;
  p.c_fp32 = a->c_fp32;
  p.c_atomic = a->c_atomic;
  p.act = a->act;
  p.split_k = a->split_k > 1 ? a->split_k : 1;
  p.a_ready_epoch = a->a_ready_epoch;
  p.c2_gelu_grad = a->c2_gelu_grad;
  p.pre_is_grad = a->pre_is_grad;
  p.mt_offset = a->mt_offset > 0 ? static_cast<int>(a->mt_offset % ((a->M + BM - 1) / BM)) : 0;
  p.signal_count = a->signal_count;
  p.done_counter = a->done_counter;
  for (int i = 0; i < a->signal_count; ++i)
    p.signal_flags[i] = static_cast<unsigned*>(const_cast<void*>(a->signal_flags[i]));

  if (pair) {
    const long long num_m2 = (a->M + 2 * BM - 1) / (2 * BM), num_n = (a->N + BN - 1) / BN;
    const long long tiles = a->batch * num_m2 * num_n * p.split_k;
    int limit = max_pairs;
    if (a->num_sms > 0 && a->num_sms / 2 < limit) limit = a->num_sms / 2 > 0 ? a->num_sms / 2 : 1;
    const int pairs = static_cast<int>(tiles < limit ? tiles : limit);
    p.mt_offset = a->mt_offset > 0 ? static_cast<int>(a->mt_offset % (2 * num_m2)) : 0;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
    cfg.blockDim = dim3(fused_push ? GEMM_THREADS_PUSH : GEMM_THREADS);
    cfg.dynamicSmemBytes = fused_push ? SMEM_BYTES_PUSH : SMEM_BYTES;
    cfg.stream = stream;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaError_t le =
        fused_push ? cudaLaunchKernelEx(&cfg, gemm_bf16_kernel<true, true>, ma, mb, mc, mc2, cm, p, pp)
                   : cudaLaunchKernelEx(&cfg, gemm_bf16_kernel<true, false>, ma, mb, mc, mc2, cm, p, pp);
    if (le != cudaSuccess) {
      set_error("%s (code %d)", cudaGetErrorString(le), static_cast<int>(le));
      return -5;
    }
    return 0;
  }
  const long long num_m = (a->M + BM - 1) / BM, num_n = (a->N + BN - 1) / BN;
  const long long tiles = a->batch * num_m * num_n * p.split_k;
  int max_ctas = a->num_sms > 0 && a->num_sms < sm_count ? a->num_sms : sm_count;
  int grid = static_cast<int>(tiles < max_ctas ? tiles : max_ctas);
  gemm_bf16_kernel<false, false><<<grid, GEMM_THREADS, SMEM_BYTES, stream>>>(ma, mb, mc, mc2, cm, p,
                                                                             pp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
    return -5;
  }
  return 0;
}
