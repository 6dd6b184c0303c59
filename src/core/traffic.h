// Bytes and messages a rank sends under the host schedule of each collective. The device
// path moves data differently (direct stores into peer windows), but hxcclCommGetStats reports
// the same figures for the same call on either path, as the reference does
// (tests/gpu_allreduce.cc:52-65); the device path therefore books these values.
#pragma once
#include <cstddef>
#include <cstdint>

#include "core/schedule.h"

namespace hx {

struct Traffic {
  uint64_t bytes = 0, msgs = 0;
  void add(uint64_t b) {
    bytes += b;
    ++msgs;
  }
};

inline Traffic traffic_allreduce(int order, int rank, int n, size_t count, size_t es) {
  Traffic t;
  if (n == 1 || count == 0) return t;
  if (order == kOrderRing) {
    for (int hop = 0; hop < n - 1; ++hop) t.add(ring_block(count, n, wrap(rank - hop, n)).len * es);
    for (int hop = 0; hop < n - 1; ++hop)
      t.add(ring_block(count, n, wrap(rank + 1 - hop, n)).len * es);
    return t;
  }
  int p = 1, levels = 0;
  while (2 * p <= n) p *= 2, ++levels;
  const int spare = n - p;
  const bool paired = rank < 2 * spare;
  if (paired && rank % 2 == 0) {
    t.add(count * es);
    return t;
  }
  for (int i = 0; i < levels; ++i) t.add(count * es);
  if (paired) t.add(count * es);
  return t;
}

inline Traffic traffic_ring_blocks(int n, size_t block_bytes) {  // AllGather, ReduceScatter
  Traffic t;
  if (n == 1 || block_bytes == 0) return t;
  for (int hop = 0; hop < n - 1; ++hop) t.add(block_bytes);
  return t;
}

inline Traffic traffic_broadcast(int rank, int n, size_t bytes, int root) {
  Traffic t;
  if (n == 1 || bytes == 0) return t;
  const int pos = wrap(rank - root, n);
  if (bytes < kTreeMaxBytes) {
    int bit = 1;
    for (; bit < n; bit <<= 1)
      if (pos & bit) break;
    for (bit >>= 1; bit > 0; bit >>= 1)
      if (pos + bit < n) t.add(bytes);
    return t;
  }
  if (pos < n - 1)
    for (size_t off = 0; off < bytes; off += kChainPiece)
      t.add(bytes - off < kChainPiece ? bytes - off : kChainPiece);
  return t;
}

inline Traffic traffic_reduce(int rank, int n, size_t bytes, int root) {
  Traffic t;
  if (n == 1 || bytes == 0) return t;
  const int pos = wrap(rank - root, n);
  if (pos == 0) return t;
  if (bytes < kTreeMaxBytes) {
    t.add(bytes);
    return t;
  }
  for (size_t off = 0; off < bytes; off += kChainPiece)
    t.add(bytes - off < kChainPiece ? bytes - off : kChainPiece);
  return t;
}

inline Traffic traffic_gather(int rank, int n, size_t block, int root) {
  Traffic t;
  (void)n;
  if (block && rank != root) t.add(block);
  return t;
}
inline Traffic traffic_scatter(int rank, int n, size_t block, int root) {
  Traffic t;
  if (block && rank == root)
    for (int i = 0; i < n - 1; ++i) t.add(block);
  return t;
}
inline Traffic traffic_alltoallv(int rank, int n, const size_t* sbytes) {
  Traffic t;
  for (int k = 1; k < n; ++k) t.add(sbytes[(rank + k) % n]);
  return t;
}

}  // namespace hx
