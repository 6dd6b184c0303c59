// Collective algorithms for host buffers. They are also the statement of record for message
// schedules (what hxcclCommGetStats counts) and for reduction orders (schedule.h).
#pragma once
#include <cstddef>

#include "core/schedule.h"
#include "host/wire.h"

namespace hx {

struct HostCtx {
  HostWire& wire;
  int rank, n;
};

hxcclResult_t host_allreduce_ring(HostCtx c, const void* send, void* recv, size_t count, int dt,
                                  int op);
hxcclResult_t host_allreduce_doubling(HostCtx c, const void* send, void* recv, size_t count,
                                      int dt, int op);
hxcclResult_t host_allgather(HostCtx c, const void* send, void* recv, size_t block_bytes);
hxcclResult_t host_reducescatter(HostCtx c, const void* send, void* recv, size_t per, int dt,
                                 int op);
hxcclResult_t host_broadcast(HostCtx c, const void* send, void* recv, size_t bytes, int root);
hxcclResult_t host_reduce(HostCtx c, const void* send, void* recv, size_t count, int dt, int op,
                          int root);
hxcclResult_t host_gather(HostCtx c, const void* send, void* recv, size_t block_bytes, int root);
hxcclResult_t host_scatter(HostCtx c, const void* send, void* recv, size_t block_bytes, int root);
// byte counts and byte offsets per peer
hxcclResult_t host_alltoallv(HostCtx c, const char* send, const size_t* sbytes,
                             const size_t* soff, char* recv, const size_t* rbytes,
                             const size_t* roff);

}  // namespace hx
