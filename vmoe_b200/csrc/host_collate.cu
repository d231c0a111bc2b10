// Host-side batch assembly for the input pipeline (no device code): copies N equally sized
// examples into one contiguous (usually pinned) batch buffer with several threads, optionally
// converting uint8 pixels to float32 with an affine map on the way (the `value_range` step of
// the pre-processing string). A 512 x 224 x 224 x 3 float batch is 308 MB: one thread needs
// tens of milliseconds for it, about as long as a training step, so the copy is spread over
// cores. The calls block until all worker threads have joined and hold no state.
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <thread>
#include <vector>

#include "vmoe_api.h"

namespace vmoe {
namespace {

template <typename Fn>
void parallel_for(int64_t n, int threads, Fn fn) {
  if (n <= 0) return;
  int t = threads > 0 ? threads : static_cast<int>(std::thread::hardware_concurrency());
  t = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(t, 64), n)));
  if (t == 1) {
    fn(0, n);
    return;
  }
  std::vector<std::thread> pool;
  pool.reserve(t - 1);
  const int64_t per = (n + t - 1) / t;
  for (int i = 1; i < t; ++i) {
    const int64_t lo = i * per, hi = std::min(n, lo + per);
    if (lo >= hi) break;
    pool.emplace_back([=] { fn(lo, hi); });
  }
  fn(0, std::min(n, per));
  for (auto& th : pool) th.join();
}

}  // namespace
}  // namespace vmoe

using namespace vmoe;

extern "C" int vmoe_collate_rows(const void* const* srcs, int64_t n, int64_t bytes_each, void* dst,
                                 int32_t threads) {
  if (n < 0 || bytes_each < 0 || (n > 0 && (srcs == nullptr || dst == nullptr))) return -1;
  char* out = static_cast<char*>(dst);
  parallel_for(n, threads, [=](int64_t lo, int64_t hi) {
    for (int64_t i = lo; i < hi; ++i)
      memcpy(out + i * bytes_each, srcs[i], static_cast<size_t>(bytes_each));
  });
  return 0;
}

extern "C" int vmoe_collate_u8_to_f32(const uint8_t* const* srcs, int64_t n, int64_t elems_each,
                                      float* dst, float scale, float shift, int32_t threads) {
  if (n < 0 || elems_each < 0 || (n > 0 && (srcs == nullptr || dst == nullptr))) return -1;
  parallel_for(n, threads, [=](int64_t lo, int64_t hi) {
    for (int64_t i = lo; i < hi; ++i) {
      const uint8_t* s = srcs[i];
      float* d = dst + i * elems_each;
      for (int64_t j = 0; j < elems_each; ++j) d[j] = static_cast<float>(s[j]) * scale + shift;
    }
  });
  return 0;
}
