// Send/Recv as peer-copy lanes. Every Send and Recv of a group on one communicator runs in a
// single launch: the operations toward one peer in one direction form a lane, a lane is split
// over kP2pWorkers CTAs, and each (lane, worker) streams its share of every message through a
// ring of kP2pDepth slots in the receiver's window, so the sender runs up to that many pieces
// ahead of the receiver:
//   sender    wait until the slot's previous occupant was taken (done flag in MY window),
//             store the bytes and the message length, then raise the receiver's ready flag;
//   receiver  wait for ready, read the length, copy min(sent, wanted) bytes out, raise the
//             sender's done flag.
// Counters only grow; both sides keep theirs in their own window between launches. A message
// longer than the receive buffer delivers the leading bytes and reports truncation on the
// receiver only (reference behaviour: src/transport_ipc.cc:424-429); the sender succeeds and
// later transfers are unaffected. This replaces the reference's host-driven READY/DONE chunk
// protocol (src/transport_ipc.cc:358-432).
#pragma once
#include "kernels/prims.cuh"

namespace hx {

__device__ __forceinline__ unsigned long long* p2p_word(char* win, size_t base, int peer, int worker) {
  return reinterpret_cast<unsigned long long*>(win + base) + size_t(peer) * kP2pWorkers + worker;
}
__device__ __forceinline__ char* p2p_slot(char* win, size_t slot_bytes, int sender, int worker, unsigned idx) {
  return win + kOffP2pSlots + ((size_t(sender) * kP2pWorkers + worker) * kP2pDepth + idx) * slot_bytes;
}
__device__ __forceinline__ unsigned long long* p2p_hdr(char* win, int sender, int worker, unsigned idx) {
  return reinterpret_cast<unsigned long long*>(win + kOffP2pHdr) +
         (size_t(sender) * kP2pWorkers + worker) * kP2pDepth + idx;
}

// A message is cut into pieces of at most a slot; one that would not fill a slot per worker is
// cut into kP2pWorkers equal pieces instead, so that every worker of the lane carries part of it
// (both ends compute this from the message length, which travels in the slot header).
__device__ __forceinline__ size_t p2p_piece(size_t total, size_t slot_bytes) {
  const size_t even = ((total + kP2pWorkers - 1) / kP2pWorkers + 15) & ~size_t(15);
  return even < 16 ? 16 : (even < slot_bytes ? even : slot_bytes);
}
// bytes of `total` that worker `wk` moves in round q (rounds advance by kP2pWorkers pieces)
__device__ __forceinline__ void p2p_share(size_t total, size_t slot_bytes, unsigned long long q, int wk, size_t* off,
                                          size_t* len) {
  const size_t piece = p2p_piece(total, slot_bytes);
  const size_t o = (q * kP2pWorkers + wk) * piece;
  *off = o;
  *len = o >= total ? 0 : (total - o < piece ? total - o : piece);
}
__device__ __forceinline__ unsigned long long p2p_rounds(size_t total, size_t slot_bytes) {
  const size_t per = size_t(kP2pWorkers) * p2p_piece(total, slot_bytes);
  const unsigned long long r = (total + per - 1) / per;
  return r ? r : 1;  // an empty message still takes one hand-shake
}

// One worker's share of every operation of a lane. False when a wait gave up.
__device__ inline bool p2p_body(const P2pArgs& a, int lane_idx, int wk, int* sh_fail, unsigned long long* sh_word,
                                BulkPipe* pipe = nullptr) {
  const WinView& w = a.w;
  const P2pLane& lane = a.lanes[lane_idx];
  const int me = w.rank, peer = lane.peer;
  char* mine = w.win[me];
  char* theirs = w.win[peer];
  if (threadIdx.x == 0) *sh_fail = 0;
  __syncthreads();
  if (lane.is_send) {
    unsigned long long* tx_state = p2p_word(mine, kOffP2pTx, peer, wk);
    unsigned long long tx = *tx_state;
    const unsigned long long* done = p2p_word(mine, kOffP2pDone, peer, wk);
    unsigned long long* ready = p2p_word(theirs, kOffP2pReady, me, wk);
    for (int k = 0; k < lane.nops; ++k) {
      const size_t total = lane.ops[k].bytes;
      const unsigned long long rounds = p2p_rounds(total, w.p2p_slot);
      for (unsigned long long q = 0; q < rounds; ++q, ++tx) {
        if (threadIdx.x == 0 && tx >= kP2pDepth && !wait_flag(w, done, tx - kP2pDepth + 1, peer)) *sh_fail = 1;
        __syncthreads();
        if (*sh_fail) return false;
        size_t off, len;
        p2p_share(total, w.p2p_slot, q, wk, &off, &len);
        if (len) {
          char* to = p2p_slot(theirs, w.p2p_slot, me, wk, unsigned(tx % kP2pDepth));
          const char* from = lane.ops[k].buf + off;
          if (pipe && ((reinterpret_cast<uintptr_t>(to) | reinterpret_cast<uintptr_t>(from) | len) & 15u) == 0) {
            // the copy unit moves the piece; one thread drives it, the others meet it at the barrier
            if (threadIdx.x == 0 && !bulk_copy_by_one_thread(*pipe, to, from, len)) {
              raise_failure(w, kStatTimeout, unsigned(peer));
              *sh_fail = 1;
            }
          } else {
            cta_copy(to, from, len);
          }
        }
        __syncthreads();
        if (*sh_fail) return false;
        if (threadIdx.x == 0) {
          st_relaxed_sys(p2p_hdr(theirs, me, wk, unsigned(tx % kP2pDepth)), total);
          st_release_sys(ready, tx + 1);
        }
      }
    }
    if (threadIdx.x == 0) *tx_state = tx;
  } else {
    unsigned long long* rx_state = p2p_word(mine, kOffP2pRx, peer, wk);
    unsigned long long rx = *rx_state;
    const unsigned long long* ready = p2p_word(mine, kOffP2pReady, peer, wk);
    unsigned long long* done = p2p_word(theirs, kOffP2pDone, me, wk);
    for (int k = 0; k < lane.nops; ++k) {
      const size_t room = lane.ops[k].bytes;
      unsigned long long rounds = 1;
      for (unsigned long long q = 0; q < rounds; ++q, ++rx) {
        if (threadIdx.x == 0) {
          if (!wait_flag(w, ready, rx + 1, peer)) *sh_fail = 1;
          *sh_word = ld_relaxed_sys(p2p_hdr(mine, peer, wk, unsigned(rx % kP2pDepth)));
        }
        __syncthreads();
        if (*sh_fail) return false;
        const size_t total = *sh_word;
        if (q == 0) rounds = p2p_rounds(total, w.p2p_slot);
        size_t off, len;
        p2p_share(total, w.p2p_slot, q, wk, &off, &len);
        if (off < room && len) {
          const size_t take = room - off < len ? room - off : len;
          cta_copy(lane.ops[k].buf + off, p2p_slot(mine, w.p2p_slot, peer, wk, unsigned(rx % kP2pDepth)), take);
        }
        if (q == 0 && wk == 0 && threadIdx.x == 0 && total > room)
          st_relaxed_sys(w.soft, (static_cast<unsigned long long>(kStatTruncated) << 56) | unsigned(peer));
        __syncthreads();
        if (threadIdx.x == 0) st_release_sys(done, rx + 1);
      }
    }
    if (threadIdx.x == 0) *rx_state = rx;
  }
  return true;
}

}  // namespace hx
