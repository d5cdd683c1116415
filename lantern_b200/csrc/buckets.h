// Cutting the gradient slab into all-reduce buckets: plain host arithmetic shared by the CUDA library (comm.cu) and
// by the CPU build of the same data-parallel step, so that both reduce exactly the same spans.
#pragma once
#include <cstdint>

namespace ltb {

constexpr int kMaxBuckets = 8;

// Splits n floats into at most kMaxBuckets spans. Every span but the last is a multiple of 1024 floats (4 KiB, so a
// 16-byte aligned slab keeps float4 alignment in every bucket); spans are never shorter than 1024 floats unless the
// slab ends. Returns the number of spans; off[i], cnt[i] describe span i. n == 0 gives 0 spans.
inline int bucket_spans(int64_t n, int64_t* off, int64_t* cnt) {
  if (n <= 0) return 0;
  int64_t per = ((n + kMaxBuckets - 1) / kMaxBuckets + 1023) / 1024 * 1024;       // ceil(n / buckets), rounded up to 1024
  if (per < 1024) per = 1024;
  int used = 0;
  for (int b = 0; b < kMaxBuckets; ++b) {
    const int64_t o = (int64_t)b * per;
    if (o >= n) break;
    off[used] = o;
    cnt[used] = n - o < per ? n - o : per;
    ++used;
  }
  return used;
}

}  // namespace ltb
