// Row push of the expert-parallel dispatch as a device function that a warp of ANY kernel can
// run beside the kernel's own work: the rows routed to every expert are fetched from this GPU's
// memory into a small shared-memory ring with bulk asynchronous copies and stored, again as bulk
// copies, into the row buffer of the GPU that owns the expert (a peer pointer over NVLink).
// Nothing passes through registers unless rows have to be scaled (backward of combine).
//
// The GEMM kernel (gemm_tcgen05.cu) runs this in two extra warps of EVERY CTA of the first
// expert GEMM: the push is spread over all SMs (a few GB/s each, so the per-SM limit on bytes in
// flight to a peer does not bound it), and the MMA / epilogue warps of the same CTAs consume the
// rows tile by tile through the arrival counters. Dispatch and GEMM are one launch whose CTAs
// are resident together by construction (grid <= number of SMs, one CTA per SM). A standalone
// kernel with the same body exists for tests (moe_p2p.cu).
//
// Stands in for the all-to-all that the reference gets from GSPMD around its dispatch einsum
// (vmoe/moe.py:488-519).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx_sm100.cuh"

namespace vmoe {

constexpr int PUSH_ROWS = 128;  // destination rows per chunk (= GEMM tile height)

struct PushParams {
  const __nv_bfloat16* x;       // (G, S, H) local rows (tokens or dy)
  const int* slot_pair;         // (G, E, C)
  const float* weight;          // (G, S, K) or NULL
  const unsigned long long* dst_base;   // [E] address of this rank's block of expert e's buffer
  const unsigned long long* flag_base;  // [E] address of expert e's tile counters (on its owner)
  const unsigned long long* ybuf_base;  // [E] local expert outputs (gate gradient) or NULL
  float* dgate;                 // (G, S, K) or NULL
  int g, s, e, c, k, h;
  int el;         // experts per rank
  int ep;         // ranks in the expert group
  int rank;       // this rank's index in the group
  int row0;       // first row of this rank's block inside an expert buffer (= rank * G * C)
};

// ---- bulk (non-tensor) asynchronous copies
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      :
      : "r"(dst_smem), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               :
               : "l"(reinterpret_cast<uint64_t>(dst)), "r"(src_smem), "r"(bytes)
               : "memory");
}

constexpr int PUSH_NSLOT = 4;       // ring slots per warp
constexpr int PUSH_DEPTH = 2;       // slots whose loads are in flight ahead of the store
constexpr int PUSH_SIGNAL_LAG = 4;  // stores of the next unit committed before a unit is signalled
constexpr int PUSH_UNIT_ROWS = 32;  // rows per work unit (a quarter of a chunk / GEMM tile)
constexpr int PUSH_RING_BYTES = 16384;  // ring of one warp
constexpr int PUSH_META_BYTES = 192;    // per warp: 32 routing entries, 4 mbarriers, abort flag

// Rows per ring slot (0: the rows do not fit and the caller must push with the plain kernel).
// With `with_y` a slot also holds the expert-output rows used for the gate gradient.
__host__ __device__ inline int push_rows_per_slot(int h, bool with_y) {
  const int per_row = h * 2 * (with_y ? 2 : 1);
  int sr = (PUSH_RING_BYTES / PUSH_NSLOT) / per_row;
  return sr > 4 ? 4 : sr;
}

// Runs the push over the work units u = wid, wid + nw, ... (a unit = 32 consecutive rows of one
// (expert, chunk); chunks in the order destination rank, rank-1, ... so that every consumer
// receives its tiles in the order in which it visits them). `ring`: PUSH_RING_BYTES of shared
// memory, 128-byte aligned; `meta`: PUSH_META_BYTES, 8-byte aligned; both private to the warp.
// Call with all 32 lanes. Every wait is bounded: on expiry the status bit is set and the warp
// stops pushing (rows it did not deliver are never signalled, so the consumer's own bounded
// wait reports them).
__device__ __forceinline__ void push_rows_ring(const PushParams& p, uint8_t* ring, uint8_t* meta,
                                               int lane, int wid, int nw, unsigned* status) {
  const int row_bytes = p.h * 2;
  const bool with_y = p.weight != nullptr && p.ybuf_base != nullptr;
  const int SR = push_rows_per_slot(p.h, with_y);
  constexpr int slot_stride = PUSH_RING_BYTES / PUSH_NSLOT;
  const int y_off = SR * row_bytes;  // expert-output rows follow the pushed rows inside a slot
  int* sidx = reinterpret_cast<int*>(meta + 64);
  uint64_t* bars = reinterpret_cast<uint64_t*>(meta);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(meta + 32);
  const uint32_t bar0 = smem_u32(bars);
  if (lane == 0) {
    *abort_flag = 0;
    for (int i = 0; i < PUSH_NSLOT; ++i) mbar_init(bar0 + 8 * i, 1);
    fence_mbar_init();
  }
  __syncwarp();
  if (SR < 1) return;

  const int block_rows = p.g * p.c;                        // rows per (expert, source rank)
  const int chunks_per_expert = (block_rows + PUSH_ROWS - 1) / PUSH_ROWS;
  constexpr int UPC = PUSH_ROWS / PUSH_UNIT_ROWS;          // units per chunk
  const long long total = static_cast<long long>(p.e) * chunks_per_expert * UPC;
  const int per_dst = p.el * chunks_per_expert;
  const int row_u4 = row_bytes >> 4;
  unsigned g_issue = 0, g_cons = 0;  // slots issued / stored so far (ring position and parity)
  bool ok = true;
  // Counters of the unit whose stores were committed last but are not yet known complete.
  unsigned* pend_flags = nullptr;
  int pend_lo = 0, pend_hi = 0;
  bool have_pending = false;
  // `all`: wait for every committed store; otherwise for all but the PUSH_SIGNAL_LAG newest.
  auto signal_pending = [&](bool all) {
    if (lane == 0) {
      if (all) {
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      } else {
        asm volatile("cp.async.bulk.wait_group %0;" ::"n"(PUSH_SIGNAL_LAG) : "memory");
      }
      if (pend_flags != nullptr) {
        // The bulk stores are complete (wait above); the release of the reduction below orders
        // them, through the proxy fence, before the counter update at system scope.
        asm volatile("fence.proxy.async.global;" ::: "memory");
        for (int tt = pend_lo / PUSH_ROWS; tt * PUSH_ROWS < pend_hi; ++tt) {
          const int lo = max(pend_lo, tt * PUSH_ROWS), hi = min(pend_hi, (tt + 1) * PUSH_ROWS);
          asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(pend_flags + tt),
                       "r"(hi - lo)
                       : "memory");
        }
      }
    }
    have_pending = false;
  };

  for (long long u = wid; u < total && ok; u += nw) {
    const long long w = u / UPC;
    const int sub = static_cast<int>(u % UPC);
    const int di = static_cast<int>(w / per_dst);
    const int rem = static_cast<int>(w % per_dst);
    const int dst = (p.rank - di + p.ep) % p.ep;
    const int ee = dst * p.el + rem / chunks_per_expert;   // global expert
    const int j0 = (rem % chunks_per_expert) * PUSH_ROWS + sub * PUSH_UNIT_ROWS;
    const int nrows = min(PUSH_UNIT_ROWS, block_rows - j0);
    if (nrows <= 0) continue;
    uint8_t* dbase = reinterpret_cast<uint8_t*>(p.dst_base[ee]) +
                     static_cast<long long>(j0) * row_bytes;
    const uint8_t* ybase =
        with_y ? reinterpret_cast<const uint8_t*>(p.ybuf_base[ee]) +
                     static_cast<long long>(j0) * row_bytes
               : nullptr;
    {  // routing entries of the unit's rows
      int pr = -1;
      if (lane < nrows) {
        const int j = j0 + lane;
        const int gi = j / p.c, ci = j - gi * p.c;
        pr = __ldg(p.slot_pair + (static_cast<long long>(gi) * p.e + ee) * p.c + ci);
      }
      sidx[lane] = pr;
    }
    __syncwarp();
    const int nslots = (nrows + SR - 1) / SR;
    for (int t = 0; t < nslots + PUSH_DEPTH && ok; ++t) {
      if (t < nslots) {
        // ---- fill ring slot: its previous store must have finished reading shared memory
        const unsigned s = g_issue % PUSH_NSLOT;
        if (lane == 0)
          asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(PUSH_NSLOT - PUSH_DEPTH - 1)
                       : "memory");
        __syncwarp();
        const int r = t * SR + lane;
        int pair = -1;
        const bool in_slot = lane < SR && r < nrows;
        if (in_slot) pair = sidx[r];
        const unsigned m_load = __ballot_sync(0xffffffffu, in_slot && pair >= 0);
        unsigned m_zero = __ballot_sync(0xffffffffu, in_slot && pair < 0);
        uint8_t* slot = ring + s * slot_stride;
        const uint32_t slot_addr = smem_u32(slot);
        const uint32_t full = bar0 + 8 * s;
        if (lane == 0)
          mbar_expect_tx(full, static_cast<uint32_t>(__popc(m_load)) * row_bytes * (with_y ? 2 : 1));
        __syncwarp();
        if (in_slot && pair >= 0) {
          const int gi = (j0 + r) / p.c;
          const int item = pair / p.k;
          bulk_load(slot_addr + lane * row_bytes,
                    p.x + (static_cast<long long>(gi) * p.s + item) * p.h, row_bytes, full);
          if (with_y)
            bulk_load(slot_addr + y_off + lane * row_bytes,
                      ybase + static_cast<long long>(r) * row_bytes, row_bytes, full);
        }
        while (m_zero) {  // empty capacity slots travel as zero rows
          const int zr = __ffs(m_zero) - 1;
          m_zero &= m_zero - 1;
          uint4* zrow = reinterpret_cast<uint4*>(slot + zr * row_bytes);
          for (int ch = lane; ch < row_u4; ch += 32) zrow[ch] = make_uint4(0, 0, 0, 0);
        }
        ++g_issue;
      }
      if (t >= PUSH_DEPTH) {
        // ---- drain ring slot: wait for its rows, (scale them,) store them to the owner
        const int tc = t - PUSH_DEPTH;
        const unsigned s = g_cons % PUSH_NSLOT;
        const bool got = mbar_wait(bar0 + 8 * s, (g_cons / PUSH_NSLOT) & 1, abort_flag, status,
                                   kStatusTimeoutProducer);
        if (!__all_sync(0xffffffffu, got)) {
          ok = false;
          break;
        }
        uint8_t* slot = ring + s * slot_stride;
        const int rows_here = min(SR, nrows - tc * SR);
        if (p.weight != nullptr) {
          for (int kr = 0; kr < rows_here; ++kr) {
            const int r = tc * SR + kr;
            const int pair = sidx[r];
            if (pair < 0) continue;
            const int gi = (j0 + r) / p.c;
            const long long pidx = static_cast<long long>(gi) * p.s * p.k + pair;
            const float wgt = __ldg(p.weight + pidx);
            uint4* srow = reinterpret_cast<uint4*>(slot + kr * row_bytes);
            const uint4* yrow = reinterpret_cast<const uint4*>(slot + y_off + kr * row_bytes);
            float dot = 0.f;
            for (int ch = lane; ch < row_u4; ch += 32) {
              uint4 q = srow[ch];
              float2 f0 = unpack_bf16x2(q.x), f1 = unpack_bf16x2(q.y), f2 = unpack_bf16x2(q.z),
                     f3 = unpack_bf16x2(q.w);
              if (with_y) {
                const uint4 yq = yrow[ch];
                const float2 y0 = unpack_bf16x2(yq.x), y1 = unpack_bf16x2(yq.y),
                             y2 = unpack_bf16x2(yq.z), y3 = unpack_bf16x2(yq.w);
                dot += f0.x * y0.x + f0.y * y0.y + f1.x * y1.x + f1.y * y1.y + f2.x * y2.x +
                       f2.y * y2.y + f3.x * y3.x + f3.y * y3.y;
              }
              q.x = pack_bf16x2(f0.x * wgt, f0.y * wgt);
              q.y = pack_bf16x2(f1.x * wgt, f1.y * wgt);
              q.z = pack_bf16x2(f2.x * wgt, f2.y * wgt);
              q.w = pack_bf16x2(f3.x * wgt, f3.y * wgt);
              srow[ch] = q;
            }
            if (p.dgate && with_y) {
#pragma unroll
              for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
              if (lane == 0) p.dgate[pidx] = dot;
            }
          }
        }
        fence_proxy_async();  // zero rows / scaled rows written by threads -> bulk store
        __syncwarp();
        if (lane == 0) {
          bulk_store(dbase + static_cast<long long>(tc) * SR * row_bytes, smem_u32(slot),
                     static_cast<uint32_t>(rows_here) * row_bytes);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        ++g_cons;
        if (have_pending && tc == PUSH_SIGNAL_LAG - 1) signal_pending(false);
      }
    }
    if (!ok) break;
    // ---- unit handed to the copy engine. Its counters are bumped once its stores are known
    // to be complete: after PUSH_SIGNAL_LAG stores of the next unit have been committed (see
    // the drain step above), so that the warp does not idle for a round trip per unit.
    if (have_pending) signal_pending(true);
    pend_flags = p.flag_base != nullptr ? reinterpret_cast<unsigned*>(p.flag_base[ee]) : nullptr;
    pend_lo = p.row0 + j0;
    pend_hi = pend_lo + nrows;
    have_pending = true;
    __syncwarp();
  }
  if (have_pending && ok) signal_pending(true);
  // Stores still in flight must finish reading shared memory before the CTA may exit.
  if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  __syncwarp();
}

}  // namespace vmoe
