#include "algos.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <vector>

#include "math/reduce_host.h"

namespace hx {
namespace {
// Working memory whose first use is a write: not cleared (clearing 64 MiB costs as much as
// sending it once).
class Scratch {
 public:
  explicit Scratch(size_t bytes) : mem_(bytes ? new char[bytes] : nullptr) {}
  char* data() { return mem_.get(); }

 private:
  std::unique_ptr<char[]> mem_;
};

// A ring over large blocks moves them in rounds of at most ring_slice() bytes per block, so that
// what a hop receives is still in the cache when it is combined or sent on. Every round cuts all
// blocks at the same offsets: which rank's value meets which, and in what order, does not
// change. The pieces of one block count as one message.
size_t ring_slice() {  // HXCCL_RING_SLICE_KB, 16 KiB .. 1 GiB, default 1 MiB
  static const size_t bytes = [] {
    const char* e = std::getenv("HXCCL_RING_SLICE_KB");
    const long kb = e ? std::atol(e) : 0;
    return kb >= 16 && kb <= (1 << 20) ? size_t(kb) << 10 : size_t(1) << 20;
  }();
  return bytes;
}

// Elements [first, first + len) of a block, clipped to the block.
Span slice_of(Span whole, size_t first, size_t len) {
  if (first >= whole.len) return Span{whole.off + whole.len, 0};
  return Span{whole.off + first, std::min(len, whole.len - first)};
}

char* at(void* p, size_t off) { return static_cast<char*>(p) + off; }
const char* at(const void* p, size_t off) { return static_cast<const char*>(p) + off; }
#define HX_TRY(expr)                                  \
  do {                                                \
    const hxcclResult_t hx_rc_ = (expr);              \
    if (hx_rc_ != hxcclSuccess) return hx_rc_;        \
  } while (0)
}  // namespace

// Reduce-scatter around the ring, then all-gather around the ring: 2(n-1) messages of about
// count/n elements per rank. Block c starts at rank c and gathers one rank per hop; the
// receiver's own value is the left operand of each combine.
hxcclResult_t host_allreduce_ring(HostCtx c, const void* send, void* recv, size_t count, int dt,
                                  int op) {
  const size_t es = dtype_size(dt);
  if (c.n == 1 || count == 0) {
    if (send != recv && count) std::memmove(recv, send, count * es);
    return hxcclSuccess;
  }
  // Out of place the input is read where it lies: every block of recv is written by a combine
  // or by the all-gather. Buffers that overlap without being equal are first made one.
  const char* lo = static_cast<const char*>(send);
  char* res = static_cast<char*>(recv);
  if (lo != res && lo < res + count * es && res < lo + count * es) {
    std::memmove(res, lo, count * es);
    lo = res;
  }
  const int next = wrap(c.rank + 1, c.n), prev = wrap(c.rank - 1, c.n);
  const size_t widest = ring_block(count, c.n, 0).len;  // block 0 is never the shorter one
  const size_t per = std::max<size_t>(1, ring_slice() / es);
  Scratch inbox(std::min(widest, per) * es);
  for (size_t first = 0; first < widest; first += per) {
    const bool more = first > 0;
    auto blk = [&](int i) { return slice_of(ring_block(count, c.n, wrap(i, c.n)), first, per); };
    for (int hop = 0; hop < c.n - 1; ++hop) {
      const Span out = blk(c.rank - hop), in = blk(c.rank - hop - 1);
      const char* leaving = (hop == 0 ? lo : res) + out.off * es;
      HX_TRY(c.wire.exchange(next, leaving, out.len * es, prev, inbox.data(), in.len * es, more));
      combine(res + in.off * es, lo + in.off * es, inbox.data(), in.len, dt, op);
    }
    for (int hop = 0; hop < c.n - 1; ++hop) {
      const Span out = blk(c.rank + 1 - hop), in = blk(c.rank - hop);
      HX_TRY(c.wire.exchange(next, res + out.off * es, out.len * es, prev, res + in.off * es,
                             in.len * es, more));
    }
  }
  return hxcclSuccess;
}

// Recursive doubling over the largest power of two p <= n. The first 2(n-p) ranks pair up:
// the even one lends its data to its odd neighbour and later gets the finished result back.
hxcclResult_t host_allreduce_doubling(HostCtx c, const void* send, void* recv, size_t count,
                                      int dt, int op) {
  const size_t bytes = count * dtype_size(dt);
  if (send != recv) std::memmove(recv, send, bytes);
  if (c.n == 1 || count == 0) return hxcclSuccess;
  int p = 1;
  while (2 * p <= c.n) p *= 2;
  const int spare = c.n - p;
  Scratch inbox(bytes);
  const bool paired = c.rank < 2 * spare;
  if (paired && c.rank % 2 == 0) {
    HX_TRY(c.wire.send(c.rank + 1, recv, bytes));
    return c.wire.recv(c.rank + 1, recv, bytes);
  }
  if (paired) {
    HX_TRY(c.wire.recv(c.rank - 1, inbox.data(), bytes));
    reduce_into(recv, inbox.data(), count, dt, op);
  }
  const int me = paired ? c.rank / 2 : c.rank - spare;  // index among the p active ranks
  for (int bit = 1; bit < p; bit <<= 1) {
    const int q = me ^ bit;
    const int peer = q < spare ? 2 * q + 1 : q + spare;
    HX_TRY(c.wire.exchange(peer, recv, bytes, peer, inbox.data(), bytes));
    reduce_into(recv, inbox.data(), count, dt, op);
  }
  if (paired) return c.wire.send(c.rank - 1, recv, bytes);
  return hxcclSuccess;
}

hxcclResult_t host_allgather(HostCtx c, const void* send, void* recv, size_t block) {
  if (send != at(recv, c.rank * block)) std::memmove(at(recv, c.rank * block), send, block);
  if (c.n == 1 || block == 0) return hxcclSuccess;
  const int next = wrap(c.rank + 1, c.n), prev = wrap(c.rank - 1, c.n);
  for (size_t first = 0; first < block; first += ring_slice()) {
    const size_t len = std::min(ring_slice(), block - first);
    for (int hop = 0; hop < c.n - 1; ++hop) {
      const int out = wrap(c.rank - hop, c.n), in = wrap(c.rank - hop - 1, c.n);
      HX_TRY(c.wire.exchange(next, at(recv, out * block + first), len, prev,
                             at(recv, in * block + first), len, first > 0));
    }
  }
  return hxcclSuccess;
}

// Ring reduce-scatter. The input is never written (recv may point into send): a hop sends
// either an untouched input block or the block combined after the previous hop, and combines
// the arriving block with the input's next block into the buffer it arrived in. The hops are
// one block ahead of the AllReduce schedule so that rank r finishes with block r.
hxcclResult_t host_reducescatter(HostCtx c, const void* send, void* recv, size_t per, int dt,
                                 int op) {
  const size_t es = dtype_size(dt), block = per * es;
  if (per == 0) return hxcclSuccess;
  const char* mine = at(send, size_t(c.rank) * block);
  if (c.n == 1) {
    if (recv != mine) std::memmove(recv, mine, block);
    return hxcclSuccess;
  }
  // the result goes straight into recv when recv is apart from the input or exactly this
  // rank's block of it (the in-place form); any other overlap gets a private result
  char* out = static_cast<char*>(recv);
  const char* in_lo = at(send, 0);
  const bool apart = out + block <= in_lo || in_lo + block * c.n <= out;
  Scratch detour(apart || out == mine ? 0 : block);
  char* result = detour.data() ? detour.data() : out;
  const size_t slice = std::max<size_t>(1, ring_slice() / es);  // elements per round
  Scratch two(2 * std::min(per, slice) * es);
  const int next = wrap(c.rank + 1, c.n), prev = wrap(c.rank - 1, c.n);
  for (size_t first = 0; first < per; first += slice) {
    const size_t len = std::min(slice, per - first), bytes = len * es;
    auto part = [&](int b) { return at(send, size_t(wrap(b, c.n)) * block + first * es); };
    const char* leaving = part(c.rank - 1);
    for (int hop = 0; hop < c.n - 1; ++hop) {
      char* inbox = two.data() + (hop & 1) * bytes;
      HX_TRY(c.wire.exchange(next, leaving, bytes, prev, inbox, bytes, first > 0));
      const char* local = part(c.rank - hop - 2);
      char* into = hop < c.n - 2 ? inbox : result + first * es;
      combine(into, local, inbox, len, dt, op);
      leaving = inbox;
    }
  }
  if (result != out) std::memmove(out, result, block);
  return hxcclSuccess;
}

// Small: binomial tree rooted at `root`. Large: a chain root -> root+1 -> ... in pieces.
hxcclResult_t host_broadcast(HostCtx c, const void* send, void* recv, size_t bytes, int root) {
  if (c.rank == root && send != recv) std::memmove(recv, send, bytes);
  if (c.n == 1 || bytes == 0) return hxcclSuccess;
  const int pos = wrap(c.rank - root, c.n);
  auto rank_at = [&](int v) { return (v + root) % c.n; };
  if (bytes < kTreeMaxBytes) {
    int bit = 1;
    for (; bit < c.n; bit <<= 1)
      if (pos & bit) {
        HX_TRY(c.wire.recv(rank_at(pos - bit), recv, bytes));
        break;
      }
    // the sends to all children leave together (farthest child first, as in the tree's order)
    for (bit >>= 1; bit > 0; bit >>= 1)
      if (pos + bit < c.n) {
        if (hxcclResult_t r = c.wire.post_send(rank_at(pos + bit), recv, bytes, kTagColl)) {
          c.wire.cancel_all();
          return r;
        }
      }
    return c.wire.finish_all();
  }
  // A rank in the middle takes in piece k+1 while piece k leaves for its successor.
  auto piece = [&](size_t off) { return std::min(kChainPiece, bytes - off); };
  if (pos > 0) HX_TRY(c.wire.recv(rank_at(pos - 1), recv, piece(0)));
  for (size_t off = 0; off < bytes; off += kChainPiece) {
    const size_t nxt = off + kChainPiece;
    if (pos > 0 && nxt < bytes)
      c.wire.post_recv(rank_at(pos - 1), at(recv, nxt), piece(nxt), kTagColl);
    if (pos < c.n - 1) {
      if (hxcclResult_t r = c.wire.post_send(rank_at(pos + 1), at(recv, off), piece(off), kTagColl)) {
        c.wire.cancel_all();
        return r;
      }
    }
    HX_TRY(c.wire.finish_all());
  }
  return hxcclSuccess;
}

// Mirror image of the broadcast: partial results flow toward the root. Non-root ranks may
// have no recv buffer, so they work in a private copy.
hxcclResult_t host_reduce(HostCtx c, const void* send, void* recv, size_t count, int dt, int op,
                          int root) {
  const size_t es = dtype_size(dt), bytes = count * es;
  std::vector<char> own;
  char* acc;
  if (c.rank == root) {
    acc = static_cast<char*>(recv);
    if (send != recv) std::memmove(acc, send, bytes);
  } else {
    own.assign(at(send, 0), at(send, bytes));
    acc = own.data();
  }
  if (c.n == 1 || count == 0) return hxcclSuccess;
  const int pos = wrap(c.rank - root, c.n);
  auto rank_at = [&](int v) { return (v + root) % c.n; };
  if (bytes < kTreeMaxBytes) {
    Scratch inbox(bytes);
    for (int bit = 1; bit < c.n; bit <<= 1) {
      if (pos & bit) return c.wire.send(rank_at(pos - bit), acc, bytes);
      if (pos + bit < c.n) {
        HX_TRY(c.wire.recv(rank_at(pos + bit), inbox.data(), bytes));
        reduce_into(acc, inbox.data(), count, dt, op);
      }
    }
    return hxcclSuccess;
  }
  // Two inboxes of one piece each (a multiple of every element size): while the combined piece
  // k leaves for the predecessor, piece k+1 of the successor arrives in the other inbox.
  Scratch inbox(pos < c.n - 1 ? 2 * kChainPiece : 0);
  auto piece = [&](size_t off) { return std::min(kChainPiece, bytes - off); };
  if (pos < c.n - 1) HX_TRY(c.wire.recv(rank_at(pos + 1), inbox.data(), piece(0)));
  for (size_t off = 0, k = 0; off < bytes; off += kChainPiece, ++k) {
    const size_t nxt = off + kChainPiece;
    if (pos < c.n - 1) {
      reduce_into(acc + off, inbox.data() + (k & 1) * kChainPiece, piece(off) / es, dt, op);
      if (nxt < bytes)
        c.wire.post_recv(rank_at(pos + 1), inbox.data() + ((k + 1) & 1) * kChainPiece, piece(nxt),
                         kTagColl);
    }
    if (pos > 0) {
      if (hxcclResult_t r = c.wire.post_send(rank_at(pos - 1), acc + off, piece(off), kTagColl)) {
        c.wire.cancel_all();
        return r;
      }
    }
    HX_TRY(c.wire.finish_all());
  }
  return hxcclSuccess;
}

hxcclResult_t host_gather(HostCtx c, const void* send, void* recv, size_t block, int root) {
  if (block == 0) return hxcclSuccess;
  if (c.rank != root) return c.wire.send(root, send, block);
  if (send != at(recv, root * block)) std::memmove(at(recv, root * block), send, block);
  for (int i = 0; i < c.n; ++i)
    if (i != root) c.wire.post_recv(i, at(recv, i * block), block, kTagColl);
  return c.wire.finish_all();
}

hxcclResult_t host_scatter(HostCtx c, const void* send, void* recv, size_t block, int root) {
  if (block == 0) return hxcclSuccess;
  if (c.rank != root) return c.wire.recv(root, recv, block);
  for (int i = 0; i < c.n; ++i)
    if (i != root)
      if (hxcclResult_t r = c.wire.post_send(i, at(send, i * block), block, kTagColl)) {
        c.wire.cancel_all();
        return r;
      }
  if (recv != at(send, root * block)) std::memmove(recv, at(send, root * block), block);
  return c.wire.finish_all();
}

// Pairwise exchange: in round k a rank sends to rank+k and receives from rank-k.
hxcclResult_t host_alltoallv(HostCtx c, const char* send, const size_t* sbytes,
                             const size_t* soff, char* recv, const size_t* rbytes,
                             const size_t* roff) {
  // every receive is posted before the first send, then all pairs move at once: one message
  // per pair and direction, so nothing can be mismatched
  for (int k = 1; k < c.n; ++k) {
    const int from = wrap(c.rank - k, c.n);
    c.wire.post_recv(from, recv + roff[from], rbytes[from], kTagColl);
  }
  for (int k = 1; k < c.n; ++k) {
    const int to = (c.rank + k) % c.n;
    if (hxcclResult_t r = c.wire.post_send(to, send + soff[to], sbytes[to], kTagColl)) {
      c.wire.cancel_all();
      return r;
    }
  }
  if (rbytes[c.rank]) std::memmove(recv + roff[c.rank], send + soff[c.rank], rbytes[c.rank]);
  return c.wire.finish_all();
}

}  // namespace hx
