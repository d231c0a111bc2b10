// Gradient all-reduce over NVLink peer memory, one range of the flat gradient buffer at a
// time, so that ranges can be reduced on a side stream while the backward pass is still
// producing later ones.
//
// Every rank keeps its gradients in a symmetric buffer (same layout on all ranks, peers mapped
// into the address space). A range is reduced in two kernels:
//   reduce: announce "my range is complete" to every peer, wait until all peers announced the
//           same, then sum this rank's 1/W slice of the range over all peers' buffers (peer
//           loads over NVLink) into the own buffer and announce "slice reduced".
//   gather: wait until all peers reduced their slices, copy those slices from the peers'
//           buffers into the own buffer and announce "done" (peers may overwrite their range
//           only after everybody is done; the host queues one wait on the done counters before
//           the optimizer runs).
// Waiting happens only at the start of a kernel, on counters that other ranks' kernels (or
// earlier kernels of this rank) advance; no CTA ever waits for a sibling CTA, so the kernels do
// not need to be co-resident. Counters grow monotonically: the target of step `epoch` is
// epoch * W. All waits are bounded and report through a status word.
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx_sm100.cuh"
#include "vmoe_api.h"

namespace vmoe {

void set_error(const char* fmt, const char* a, int code);

namespace {

constexpr int kMaxPeers = 16;

struct ArPeers {
  float* buf[kMaxPeers];       // base of every rank's gradient buffer
  unsigned* flags[kMaxPeers];  // base of every rank's counters: [3][num_ranges]
};

__device__ __forceinline__ void signal_sys(unsigned* p) {
  asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p) : "memory");
}
__device__ __forceinline__ unsigned load_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 load_peer(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Thread 0 waits (bounded) until *counter >= target; the whole CTA learns the outcome.
__device__ __forceinline__ bool cta_wait_counter(const unsigned* counter, unsigned target,
                                                 unsigned* status, long long limit) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = 1;
    const long long t0 = clock64();
    while (static_cast<int>(load_acquire_sys(counter) - target) < 0) {
      if (clock64() - t0 > limit) {
        ok = 0;
        if (status) atomicOr(status, kStatusTimeoutPeer);
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
  return ok != 0;
}

// The last CTA to get here resets the local counter and signals `which` on every peer.
__device__ __forceinline__ void cta_done_signal(const ArPeers& peers, int world, unsigned* local,
                                                int flag_index) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(local, 1u);
    if (prev == gridDim.x - 1) {
      *local = 0;
      __threadfence_system();
      for (int p = 0; p < world; ++p) signal_sys(peers.flags[p] + flag_index);
    }
  }
}

__global__ void __launch_bounds__(256)
allreduce_reduce_kernel(ArPeers peers, int world, int rank, long long offset, long long count,
                        int range, int num_ranges, unsigned target, unsigned* local,
                        unsigned* status, long long limit) {
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    signal_sys(peers.flags[threadIdx.x] + range);  // "my range is complete"
  }
  const bool ok = cta_wait_counter(peers.flags[rank] + range, target, status, limit);
  if (ok) {
    const long long per = count / world;  // multiple of 4 (ranges are multiples of 1024)
    const long long base = offset + static_cast<long long>(rank) * per;
    float* mine = peers.buf[rank] + base;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
    for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
         i < per; i += stride) {
      float4 acc = *reinterpret_cast<const float4*>(mine + i);
      for (int p = 1; p < world; ++p) {
        const int q = (rank + p) % world;
        const float4 v = load_peer(peers.buf[q] + base + i);
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
      }
      *reinterpret_cast<float4*>(mine + i) = acc;
    }
  }
  cta_done_signal(peers, world, local, num_ranges + range);  // "slice reduced"
}

__global__ void __launch_bounds__(256)
allreduce_gather_kernel(ArPeers peers, int world, int rank, long long offset, long long count,
                        int range, int num_ranges, unsigned target, unsigned* local,
                        unsigned* status, long long limit) {
  const bool ok = cta_wait_counter(peers.flags[rank] + num_ranges + range, target, status, limit);
  if (ok) {
    const long long per = count / world;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
    for (int p = 1; p < world; ++p) {
      const int q = (rank + p) % world;
      const long long base = offset + static_cast<long long>(q) * per;
      const float* src = peers.buf[q] + base;
      float* dst = peers.buf[rank] + base;
      for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
           i < per; i += stride)
        *reinterpret_cast<float4*>(dst + i) = load_peer(src + i);
    }
  }
  cta_done_signal(peers, world, local, 2 * num_ranges + range);  // "done with the peers' data"
}

int fill_peers(ArPeers* peers, const uint64_t* bufs, const uint64_t* flags, int world) {
  if (world < 1 || world > kMaxPeers) {
    set_error("%s (code %d)", "allreduce: world size must be in [1, 16]", world);
    return -1;
  }
  for (int p = 0; p < kMaxPeers; ++p) {
    peers->buf[p] = p < world ? reinterpret_cast<float*>(bufs[p]) : nullptr;
    peers->flags[p] = p < world ? reinterpret_cast<unsigned*>(flags[p]) : nullptr;
  }
  return 0;
}

int finish_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s (code %d)", cudaGetErrorString(e), static_cast<int>(e));
    return -5;
  }
  return 0;
}

}  // namespace
}  // namespace vmoe

using namespace vmoe;

extern "C" int vmoe_allreduce_range(const uint64_t* bufs, const uint64_t* flags, int32_t world,
                                    int32_t rank, int64_t offset, int64_t count, int32_t range,
                                    int32_t num_ranges, uint32_t epoch, uint32_t* local_counters,
                                    uint32_t* status, int32_t ctas, int64_t limit_cycles,
                                    vmoe_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  ArPeers peers;
  if (int rc = fill_peers(&peers, bufs, flags, world)) return rc;
  if (count <= 0) return 0;
  if (count % (4 * world) || offset % 4 || range < 0 || range >= num_ranges) {
    set_error("%s (code %d)", "allreduce: count must be a multiple of 4 * world, offset of 4", 0);
    return -1;
  }
  const long long limit = limit_cycles > 0 ? limit_cycles : kWaitLimitCycles;
  const unsigned target = epoch * static_cast<unsigned>(world);
  const long long per = count / world;
  long long want = (per / 4 + 255) / 256;
  if (want < 1) want = 1;
  const int grid = static_cast<int>(want < ctas ? want : (ctas > 0 ? ctas : 1));
  allreduce_reduce_kernel<<<grid, 256, 0, stream>>>(peers, world, rank, offset, count, range,
                                                    num_ranges, target, local_counters + 2 * range,
                                                    status, limit);
  allreduce_gather_kernel<<<grid, 256, 0, stream>>>(peers, world, rank, offset, count, range,
                                                    num_ranges, target,
                                                    local_counters + 2 * range + 1, status, limit);
  return finish_launch();
}
