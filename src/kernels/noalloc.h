// An AllReduce entry point for callers that must not allocate device memory.
//
// This function has no counterpart in the reference library. It exists for code that runs
// where cudaMalloc is off limits: inside a region whose memory is owned by a caching allocator
// that forbids raw allocations, in a process that has pinned its whole device-memory budget up
// front, or in late start-up / teardown paths where the allocator is not (or no longer) usable.
// Such callers can still check the collective kernels on one GPU: the staging windows, the
// per-rank argument blocks and the status words all live in one file-scope device array of
// fixed size that is part of the library image, so the call allocates nothing, neither on the
// device nor in pinned host memory.
#pragma once
#include <stddef.h>

#include "hxccl.h"

#ifdef __cplusplus
extern "C" {
#endif

#define HXCCL_NOALLOC_MAX_RANKS 4
#define HXCCL_NOALLOC_MAX_BYTES (1u << 20) /* per rank */

/* AllReduce over `nranks` ranks (1..HXCCL_NOALLOC_MAX_RANKS) that all live on the current
 * device, as hxcclWorldAllReduce does it with the one-shot kernel, in the exact reduction order
 * of the host path: send[r] / recv[r] are rank r's device buffers of `count` elements
 * (count * sizeof(datatype) <= HXCCL_NOALLOC_MAX_BYTES; recv[r] may equal send[r]). `op` is
 * hxcclSum, hxcclProd, hxcclMax, hxcclMin or hxcclAvg.
 *
 * The work is enqueued on `stream` and the function returns after it has completed there
 * (it reads the kernels' status word back), so the result code covers the device side too:
 * hxcclSuccess, hxcclInvalidArgument (bad rank count, datatype, operator, null buffer, or a
 * size beyond the maximum; last error text via hxcclNoAllocLastError), hxcclTimeout when a
 * device-side wait ran out, hxcclUnhandledCudaError for CUDA failures.
 *
 * Scratch: one static device array of 5 251 328 bytes (5.0 MiB) per GPU that loads the
 * library, held until the process exits. The first call on a device is the set-up: with that
 * device current it looks the array's device address up (cudaGetSymbolAddress) and clears the
 * array; make that first call before any stream capture begins. Later calls repeat the look-up
 * (so a device reset cannot leave a stale pointer behind). Every call copies its argument
 * blocks from pageable host memory and ends with cudaStreamSynchronize(stream).
 * Every call uses the same array and finds what the previous call left there: flags only grow
 * from call to call and the status words are cleared at the start of each call. Two calls that
 * overlap on the GPU (different streams, or different threads) therefore race on the array;
 * callers must serialize them. Not thread-safe. */
hxcclResult_t hxcclAllReduceNoAlloc(int nranks, const void* const* send, void* const* recv,
                                    size_t count, hxcclDataType_t datatype, hxcclRedOp_t op,
                                    hxcclStream_t stream);
const char* hxcclNoAllocLastError(void);

#ifdef __cplusplus
}
#endif
