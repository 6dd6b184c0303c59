// Schedules that define results, shared by the host algorithms and the device kernels.
//
// The order in which ranks' values are combined decides the bits of a floating-point result,
// so the device kernels replay the order of the host algorithms, which in turn follow the
// reference's (src/chunks.h:11-17, src/algo_ring.cc:12-80, src/algo_rd.cc:7-37,
// src/algo_rooted.cc:25-48, src/select.h:10).
#pragma once
#include <cstddef>
#include <cstdint>

#if defined(__CUDACC__)
#define HX_SCHED_HD __host__ __device__ __forceinline__
#else
#define HX_SCHED_HD inline
#endif

namespace hx {

// AllReduce result orders
enum : int { kOrderRing = 0, kOrderDoubling = 1 };

constexpr size_t kDoublingMaxBytes = 64 * 1024;   // below: recursive doubling, else ring
constexpr size_t kTreeMaxBytes = 512 * 1024;      // Broadcast/Reduce: below tree, else chain
constexpr size_t kChainPiece = 512 * 1024;        // chain segment

struct Span {
  size_t off, len;
};

// Block i of `count` elements split n ways: the first count % n blocks are one longer.
HX_SCHED_HD Span ring_block(size_t count, int n, int i) {
  const size_t base = count / static_cast<size_t>(n), extra = count % static_cast<size_t>(n);
  const size_t k = static_cast<size_t>(i);
  return Span{k * base + (k < extra ? k : extra), base + (k < extra ? 1u : 0u)};
}

HX_SCHED_HD int wrap(int a, int n) {
  const int m = a % n;
  return m < 0 ? m + n : m;
}

}  // namespace hx
