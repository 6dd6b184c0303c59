/*
 * hxccl (B200 build): collective communication for NVLink 5 / NVSwitch nodes.
 *
 * The function names, argument order and every numeric value below follow the hxccl 0.2
 * public header (reference: include/hxccl.h:14-155), whose numbering is NCCL v2.32.3's.
 * Device buffers are moved by sm_100a kernels over peer-mapped windows (and NVSwitch
 * multicast where the node offers it); calls on device buffers enqueue on `stream` and
 * return before the work is done. Calls on host buffers run to completion over the
 * socket mesh that hxcclGetUniqueId / hxcclCommInitRank build.
 *
 * MPI is optional: define HXCCL_HAVE_MPI before including this header (and link an MPI
 * build of the library) to get hxcclCommInitMPI.
 */
#ifndef HXCCL_H_
#define HXCCL_H_

#include <limits.h>
#include <stddef.h>
#include <stdint.h>
#ifdef HXCCL_HAVE_MPI
#include <mpi.h>
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- opaque handles ---------------------------------------------------------------- */
typedef struct hxcclComm* hxcclComm_t;
typedef struct { char internal[128]; } hxcclUniqueId;
typedef void* hxcclStream_t; /* a cudaStream_t for device buffers; ignored for host buffers */

/* ---- result codes (NCCL numbering) ------------------------------------------------- */
typedef enum {
  hxcclSuccess            = 0,
  hxcclUnhandledCudaError = 1,
  hxcclSystemError        = 2,
  hxcclInternalError      = 3,
  hxcclInvalidArgument    = 4,
  hxcclInvalidUsage       = 5,
  hxcclRemoteError        = 6,
  hxcclInProgress         = 7,
  hxcclTimeout            = 8,
  hxcclNumResults         = 9
} hxcclResult_t;

/* ---- element types (NCCL numbering) ------------------------------------------------ */
typedef enum {
  hxcclInt8       = 0,  hxcclChar   = 0,
  hxcclUint8      = 1,
  hxcclInt32      = 2,  hxcclInt    = 2,
  hxcclUint32     = 3,
  hxcclInt64      = 4,
  hxcclUint64     = 5,
  hxcclFloat16    = 6,  hxcclHalf   = 6,
  hxcclFloat32    = 7,  hxcclFloat  = 7,
  hxcclFloat64    = 8,  hxcclDouble = 8,
  hxcclBfloat16   = 9,
  hxcclFloat8e4m3 = 10,
  hxcclFloat8e5m2 = 11,
  hxcclNumTypes   = 12
} hxcclDataType_t;

/* ---- reduction operators ----------------------------------------------------------- */
typedef enum {
  hxcclSum      = 0,
  hxcclProd     = 1,
  hxcclMax      = 2,
  hxcclMin      = 3,
  hxcclAvg      = 4,
  hxcclNumOps   = 5,          /* handles from hxcclRedOpCreatePreMulSum start here */
  hxcclMaxRedOp = 0x7fffffff
} hxcclRedOp_t;

typedef enum {
  hxcclScalarDevice        = 0, /* pointer kept; dereferenced when the collective is called */
  hxcclScalarHostImmediate = 1  /* value copied when the op is created */
} hxcclScalarResidence_t;

#define HXCCL_SPLIT_NOCOLOR (-1)
#define HXCCL_VERSION(X, Y, Z) \
  (((X) <= 2 && (Y) <= 8) ? (X) * 1000 + (Y) * 100 + (Z) : (X) * 10000 + (Y) * 100 + (Z))
#define HXCCL_VERSION_CODE HXCCL_VERSION(0, 2, 0)

/* ---- communicator configuration ---------------------------------------------------- */
#define HXCCL_CONFIG_UNDEF_INT INT_MIN
#define HXCCL_CONFIG_MAGIC 0x6878636cu
typedef struct {
  size_t size;
  unsigned int magic;
  unsigned int version;
  int blocking;         /* 1 or HXCCL_CONFIG_UNDEF_INT; 0 is rejected */
  const char* commName; /* kept for NCCL source compatibility; unused */
} hxcclConfig_t;
#define HXCCL_CONFIG_INITIALIZER \
  { sizeof(hxcclConfig_t), HXCCL_CONFIG_MAGIC, HXCCL_VERSION_CODE, HXCCL_CONFIG_UNDEF_INT, NULL }

/* ---- library / communicator lifecycle ---------------------------------------------- */
hxcclResult_t hxcclGetVersion(int* version);
/* The process that creates the id must itself call hxcclCommInitRank with it. */
hxcclResult_t hxcclGetUniqueId(hxcclUniqueId* id);
hxcclResult_t hxcclCommInitRank(hxcclComm_t* comm, int nranks, hxcclUniqueId id, int rank);
#ifdef HXCCL_HAVE_MPI
hxcclResult_t hxcclCommInitMPI(hxcclComm_t* comm, MPI_Comm mpi);
#endif
hxcclResult_t hxcclCommInitRankConfig(hxcclComm_t* comm, int nranks, hxcclUniqueId id,
                                      int rank, hxcclConfig_t* config);
hxcclResult_t hxcclCommDestroy(hxcclComm_t comm);
/* color == HXCCL_SPLIT_NOCOLOR: the caller takes part but gets *newcomm == NULL. */
hxcclResult_t hxcclCommSplit(hxcclComm_t comm, int color, int key, hxcclComm_t* newcomm,
                             hxcclConfig_t* config);
/* Called by the surviving ranks only, all with the same exclude list; shrinkFlags must be 0. */
hxcclResult_t hxcclCommShrink(hxcclComm_t comm, int* excludeRanksList, int excludeRanksCount,
                              hxcclComm_t* newcomm, hxcclConfig_t* config, int shrinkFlags);
hxcclResult_t hxcclCommAbort(hxcclComm_t comm); /* local teardown, contacts no peer */
hxcclResult_t hxcclCommFinalize(hxcclComm_t comm);
hxcclResult_t hxcclCommGetAsyncError(hxcclComm_t comm, hxcclResult_t* asyncError);
hxcclResult_t hxcclCommCount(hxcclComm_t comm, int* count);
hxcclResult_t hxcclCommUserRank(hxcclComm_t comm, int* rank);

/* ---- collectives -------------------------------------------------------------------- */
hxcclResult_t hxcclAllReduce(const void* sendbuff, void* recvbuff, size_t count,
                             hxcclDataType_t datatype, hxcclRedOp_t op, hxcclComm_t comm,
                             hxcclStream_t stream);
hxcclResult_t hxcclAllGather(const void* sendbuff, void* recvbuff, size_t sendcount,
                             hxcclDataType_t datatype, hxcclComm_t comm,
                             hxcclStream_t stream);
hxcclResult_t hxcclReduceScatter(const void* sendbuff, void* recvbuff, size_t recvcount,
                                 hxcclDataType_t datatype, hxcclRedOp_t op,
                                 hxcclComm_t comm, hxcclStream_t stream);
hxcclResult_t hxcclBroadcast(const void* sendbuff, void* recvbuff, size_t count,
                             hxcclDataType_t datatype, int root, hxcclComm_t comm,
                             hxcclStream_t stream);

/* Rooted forms. On non-root ranks recvbuff (Reduce, Gather) and sendbuff (Scatter) may be NULL. */
hxcclResult_t hxcclReduce(const void* sendbuff, void* recvbuff, size_t count,
                          hxcclDataType_t datatype, hxcclRedOp_t op, int root, hxcclComm_t comm,
                          hxcclStream_t stream);
hxcclResult_t hxcclBcast(void* buff, size_t count, hxcclDataType_t datatype, int root,
                         hxcclComm_t comm, hxcclStream_t stream);
hxcclResult_t hxcclGather(const void* sendbuff, void* recvbuff, size_t count,
                          hxcclDataType_t datatype, int root, hxcclComm_t comm,
                          hxcclStream_t stream);
hxcclResult_t hxcclScatter(const void* sendbuff, void* recvbuff, size_t count,
                           hxcclDataType_t datatype, int root, hxcclComm_t comm,
                           hxcclStream_t stream);

/* Block j of sendbuff (count elements) goes to rank j; rank i's block lands at recvbuff + i*count. */
hxcclResult_t hxcclAlltoAll(const void* sendbuff, void* recvbuff, size_t count,
                            hxcclDataType_t datatype, hxcclComm_t comm, hxcclStream_t stream);
/* RCCL spellings. Counts and displacements of AllToAllv are in elements; its arguments are
 * agreed on over the control mesh at call time (also inside a group), so that one rank's bad
 * argument is rejected by every rank instead of stalling the others. */
hxcclResult_t hxcclAllToAll(const void* sendbuff, void* recvbuff, size_t count,
                            hxcclDataType_t datatype, hxcclComm_t comm, hxcclStream_t stream);
hxcclResult_t hxcclAllToAllv(const void* sendbuff, const size_t sendcounts[],
                             const size_t sdispls[], void* recvbuff, const size_t recvcounts[],
                             const size_t rdispls[], hxcclDataType_t datatype,
                             hxcclComm_t comm, hxcclStream_t stream);

/* ---- point to point and groups ------------------------------------------------------ */
hxcclResult_t hxcclSend(const void* sendbuff, size_t count, hxcclDataType_t datatype, int peer,
                        hxcclComm_t comm, hxcclStream_t stream);
hxcclResult_t hxcclRecv(void* recvbuff, size_t count, hxcclDataType_t datatype, int peer,
                        hxcclComm_t comm, hxcclStream_t stream);
/* Calls made between GroupStart and the outermost GroupEnd are issued at that GroupEnd:
 * collectives first, in call order, then every Send/Recv of the group together. */
hxcclResult_t hxcclGroupStart(void);
hxcclResult_t hxcclGroupEnd(void);

/* ---- user reduction operators -------------------------------------------------------- */
/* Sum of (input * scalar). The handle is valid only on `comm` and with `datatype`. */
hxcclResult_t hxcclRedOpCreatePreMulSum(hxcclRedOp_t* op, void* scalar,
                                        hxcclDataType_t datatype,
                                        hxcclScalarResidence_t residence, hxcclComm_t comm);
hxcclResult_t hxcclRedOpDestroy(hxcclRedOp_t op, hxcclComm_t comm);

/* ---- diagnostics ---------------------------------------------------------------------- */
const char* hxcclGetErrorString(hxcclResult_t result);
const char* hxcclGetLastError(hxcclComm_t comm);
/* User payload bytes/messages this rank sent under the reference schedule of each call. */
hxcclResult_t hxcclCommGetStats(hxcclComm_t comm, uint64_t* bytes_sent, uint64_t* msgs_sent);
hxcclResult_t hxcclCommResetStats(hxcclComm_t comm);

#ifdef __cplusplus
}
#endif
#endif /* HXCCL_H_ */
