/*
 * Additions of this library that the hxccl 0.2 header does not have: diagnostics of the device
 * path, the standalone elementwise kernels, host versions of the element rules (the oracle the
 * device results are compared with), fault-injection hooks for tests, and a "world on one GPU"
 * harness that runs the collective kernels for every rank of a small communicator inside one
 * cooperative launch, for machines with a single GPU.
 */
#ifndef HXCCL_EXT_H_
#define HXCCL_EXT_H_

#include "hxccl.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- diagnostics -------------------------------------------------------------------------- */
/* kind: "none", "staged", "window" or "window+nvls". variant: what the latest AllReduce used
 * (1 one-shot, 2 two-shot, 3 NVLS). launches: kernels launched by this communicator so far. */
hxcclResult_t hxcclCommDeviceInfo(hxcclComm_t comm, char* kind, size_t kind_len, int* variant,
                                  unsigned long long* launches);
/* Forces the AllReduce variant of later calls (0 auto, 1 one-shot, 2 two-shot, 3 NVLS,
 * 6 neighbour ring, 7 flag-in-data lines for small messages), the
 * exactness mode (1 = floats match the host path bit for bit) and the largest grid (0 keeps it).
 * Every rank must make the same call. */
hxcclResult_t hxcclCommTune(hxcclComm_t comm, int variant, int exact, int max_ctas);

/* Sets one tuning knob of the device path by name (see src/device/planner.h: set_knob), e.g.
 * "roles_min" (bytes from which AllReduce runs as a three-role pipeline). Same call on every
 * rank. hxcclInvalidArgument for an unknown name. */
hxcclResult_t hxcclCommTuneKnob(hxcclComm_t comm, const char* name, long value);

/* AllReduce of fp32 device buffers with a 16-bit float type on the wire (hxcclFloat16 or
 * hxcclBfloat16): every value is rounded to wire_dt, the ranks' values are combined under
 * wire_dt's rules in the ring order (op as for hxcclAllReduce, hxcclAvg and PreMulSum operators
 * created for wire_dt included), and the result is widened back to fp32 - bit for bit what
 * "cast, hxcclAllReduce in wire_dt, cast back" gives, in one kernel and with half the bytes on
 * the links (a gradient bucket of a data-parallel step). count * 2 must be at least 64 KiB
 * (the size from which hxcclAllReduce takes the ring order) and the communicator needs two or
 * more ranks on the window device path; otherwise hxcclInvalidUsage, and nothing was done. */
hxcclResult_t hxcclAllReduceCast(const void* send, void* recv, size_t count, hxcclDataType_t wire_dt,
                                 hxcclRedOp_t op, hxcclComm_t comm, hxcclStream_t stream);

/* Phase timers of the collective kernels (communicators created with HXCCL_TRACE=1): 16
 * nanosecond sums per CTA since the previous read (staging in, first flag, first wait,
 * combining, second flag, second wait, staging out, whole kernel, rest unused). Waits for the
 * enqueued work first. Returns the number of CTA rows written to `out` (0 when tracing is off). */
int hxcclCommReadTrace(hxcclComm_t comm, unsigned long long* out, int max_ctas);

/* ---- elementwise kernels on device buffers (any stream, no communicator) ------------------- */
hxcclResult_t hxcclDevReduce(void* dst, const void* src, size_t count, hxcclDataType_t dt,
                             hxcclRedOp_t op, hxcclStream_t stream); /* dst = dst op src */
hxcclResult_t hxcclDevScale(void* dst, const void* src, size_t count, hxcclDataType_t dt,
                            const void* scalar_host, hxcclStream_t stream);
hxcclResult_t hxcclDevDivide(void* buf, size_t count, hxcclDataType_t dt, int divisor,
                             hxcclStream_t stream);

/* ---- the same rules on host buffers ---------------------------------------------------------- */
hxcclResult_t hxcclHostReduce(void* dst, const void* src, size_t count, hxcclDataType_t dt,
                              hxcclRedOp_t op);
hxcclResult_t hxcclHostScale(void* dst, const void* src, size_t count, hxcclDataType_t dt,
                             const void* scalar);
hxcclResult_t hxcclHostDivide(void* buf, size_t count, hxcclDataType_t dt, int divisor);
/* float -> narrow type bits and back (Float16, Bfloat16, Float8e4m3, Float8e5m2) */
unsigned hxcclHostEncode(hxcclDataType_t dt, float value);
float hxcclHostDecode(hxcclDataType_t dt, unsigned bits);
/* the ring block of `count` elements over n ranks: offset and length of block i */
void hxcclRingBlock(size_t count, int n, int i, size_t* off, size_t* len);

/* Device self-check: runs the device's float -> dt encoder over all 2^32 float bit patterns and
 * its decoder over all codes of dt (Float16, Bfloat16, Float8e4m3, Float8e5m2) and counts the
 * inputs where it differs from the host rules; *first_bad_bits is the smallest such float. */
hxcclResult_t hxcclTestNarrowConvert(hxcclDataType_t dt, unsigned long long* mismatches,
                                     unsigned int* first_bad_bits);

/* Plans one launch without a device: kind 0 generic exchange (amount = largest block of a pair),
 * 1 two-shot / NVLS AllReduce (amount = message bytes), 2 the same as three-role pipeline,
 * 3 neighbour ring (amount = largest ring block), 4 the same for ReduceScatter, for `nranks` ranks whose staging halves hold
 * `half_bytes` each, with the default tuning, then HXCCL_TUNE_FILE when set, then `max_ctas` (0 keeps it) and one optional
 * knob (`knob` may be NULL). shape = {ctas, threads, steps, epochs, sub_bytes}. Returns
 * hxcclSuccess when the shape fits the window layout the kernels assume and covers `amount`,
 * hxcclInternalError otherwise (`why`, when given, receives the reason). */
hxcclResult_t hxcclTestPlan(int kind, size_t amount, int nranks, size_t half_bytes, int max_ctas,
                            const char* knob, long knob_value, size_t shape[5], char* why, size_t why_len);

/* Which AllReduce variant the tuner picks for `bytes` of `dt` on `nranks` ranks in exact (1) or
 * fast (0) mode, with (1) or without (0) NVSwitch multicast, from the compiled-in table, then
 * HXCCL_TUNE_FILE when set. *from_table: 1 when a table row decided, 0 when the fixed thresholds
 * did. shape = {grid limit, CTA width (0 = by size), per-step share} after the row was applied. */
hxcclResult_t hxcclTestChooseVariant(size_t bytes, hxcclDataType_t dt, int nranks, int exact, int nvls,
                                     int* variant, int* from_table, size_t shape[3]);

/* Rows of the compiled-in tuning table that parsed. */
int hxcclTestTableRows(void);

/* ---- fault injection (host side only) ---------------------------------------------------------- */
/* The (after+1)-th host-path send from now fails with hxcclSystemError; after < 0 disarms. */
hxcclResult_t hxcclTestFailSends(hxcclComm_t comm, long after);
/* Closes the control connection to `peer` as if that process had died. */
hxcclResult_t hxcclTestSeverPeer(hxcclComm_t comm, int peer);

/* ---- a whole communicator on one GPU ------------------------------------------------------------ */
typedef struct hxcclWorld* hxcclWorld_t;
/* n ranks (1..16) on the current device, each with a window of window_mb MiB of staging.
 * wait_ms bounds every device-side wait. */
hxcclResult_t hxcclWorldCreate(hxcclWorld_t* world, int n, int window_mb, int wait_ms);
hxcclResult_t hxcclWorldDestroy(hxcclWorld_t world);
/* variant/exact/max_ctas as in hxcclCommTune */
hxcclResult_t hxcclWorldTune(hxcclWorld_t world, int variant, int exact, int max_ctas);
hxcclResult_t hxcclWorldTuneKnob(hxcclWorld_t world, const char* name, long value);
/* send[r] / recv[r] are rank r's device buffers. op is hxcclSum..hxcclAvg; a non-null scalar
 * (host memory, one element of dt) makes it PreMulSum. order: 0 ring, 1 recursive doubling,
 * -1 by message size as the API does. */
hxcclResult_t hxcclWorldAllReduce(hxcclWorld_t world, const void* const* send, void* const* recv,
                                  size_t count, hxcclDataType_t dt, hxcclRedOp_t op,
                                  const void* scalar, int order, hxcclStream_t stream);
/* hxcclAllReduceCast in the world: send[r] / recv[r] hold fp32, wire_dt travels */
hxcclResult_t hxcclWorldAllReduceCast(hxcclWorld_t world, const void* const* send, void* const* recv,
                                      size_t count, hxcclDataType_t wire_dt, hxcclRedOp_t op,
                                      hxcclStream_t stream);
hxcclResult_t hxcclWorldReduceScatter(hxcclWorld_t world, const void* const* send,
                                      void* const* recv, size_t recvcount, hxcclDataType_t dt,
                                      hxcclRedOp_t op, const void* scalar, hxcclStream_t stream);
hxcclResult_t hxcclWorldReduce(hxcclWorld_t world, const void* const* send, void* const* recv,
                               size_t count, hxcclDataType_t dt, hxcclRedOp_t op,
                               const void* scalar, int root, hxcclStream_t stream);
hxcclResult_t hxcclWorldAllGather(hxcclWorld_t world, const void* const* send, void* const* recv,
                                  size_t bytes_per_rank, hxcclStream_t stream);
hxcclResult_t hxcclWorldBroadcast(hxcclWorld_t world, const void* const* send, void* const* recv,
                                  size_t bytes, int root, hxcclStream_t stream);
hxcclResult_t hxcclWorldGather(hxcclWorld_t world, const void* const* send, void* const* recv,
                               size_t bytes_per_rank, int root, hxcclStream_t stream);
hxcclResult_t hxcclWorldScatter(hxcclWorld_t world, const void* const* send, void* const* recv,
                                size_t bytes_per_rank, int root, hxcclStream_t stream);
/* bytes[r*n + j]: bytes rank r sends to rank j; soff / roff likewise (byte offsets; roff[r*n+i]
 * is where rank r puts what rank i sent). */
hxcclResult_t hxcclWorldAllToAllv(hxcclWorld_t world, const void* const* send, void* const* recv,
                                  const size_t* bytes, const size_t* soff, const size_t* roff,
                                  hxcclStream_t stream);
/* nops transfers: transfer k sends sbytes[k] bytes from src[k] on rank from[k] into dst[k]
 * (room rbytes[k]) on rank to[k]; all in one group. */
hxcclResult_t hxcclWorldSendRecv(hxcclWorld_t world, int nops, const int* from, const int* to,
                                 const void* const* src, const size_t* sbytes, void* const* dst,
                                 const size_t* rbytes, hxcclStream_t stream);
/* status words of rank r after the stream is synchronized: sticky (0 = fine; code in the top
 * byte: 1 timeout, 2 remote) and soft (3 in the top byte = a receive was truncated; cleared) */
hxcclResult_t hxcclWorldStatus(hxcclWorld_t world, int rank, unsigned long long* sticky,
                               unsigned long long* soft);
hxcclResult_t hxcclWorldInfo(hxcclWorld_t world, int* variant, unsigned long long* launches);
/* text of the CUDA error behind the latest hxcclUnhandledCudaError of a world call */
const char* hxcclWorldLastError(void);
/* Test hook: from now on rank r's stores and flags go to a private dummy window, so that its
 * peers wait for flags that nothing sets; their bounded waits then run out and report it. */
hxcclResult_t hxcclWorldMute(hxcclWorld_t world, int rank);

#ifdef __cplusplus
}
#endif
#endif /* HXCCL_EXT_H_ */
