/* A stand-in for <mpi.h>, just enough to compile the reference library's sources where no MPI
 * is installed. Every function fails (returns MPI_ERR_OTHER); nothing here communicates. The
 * reference arm of bench.py builds the reference's communicators with hxcclGetUniqueId /
 * hxcclCommInitRank (its socket bootstrap), a path on which the reference never calls MPI. */
#ifndef HX_MPI_STUB_H_
#define HX_MPI_STUB_H_
#ifdef __cplusplus
extern "C" {
#endif
typedef int MPI_Comm;
typedef int MPI_Datatype;
typedef int MPI_Op;
typedef int MPI_Request;
typedef int MPI_Group;
typedef int MPI_Errhandler;
typedef struct { int MPI_SOURCE, MPI_TAG, MPI_ERROR; } MPI_Status;
#define MPI_SUCCESS 0
#define MPI_ERR_OTHER 15
#define MPI_ERR_IN_STATUS 17
#define MPI_COMM_NULL 0
#define MPI_COMM_WORLD 1
#define MPI_REQUEST_NULL 0
#define MPI_UNDEFINED (-32766)
#define MPI_BYTE 1
#define MPI_INT 2
#define MPI_MAX 1
#define MPI_IN_PLACE ((void*)1)
#define MPI_STATUS_IGNORE ((MPI_Status*)0)
#define MPI_STATUSES_IGNORE ((MPI_Status*)0)
#define MPI_ERRORS_RETURN 1
#define MPI_MAX_ERROR_STRING 256
#define MPI_ANY_SOURCE (-1)
#define MPI_ANY_TAG (-1)
int MPI_Init(int*, char***);
int MPI_Comm_size(MPI_Comm, int*);
int MPI_Comm_rank(MPI_Comm, int*);
int MPI_Comm_dup(MPI_Comm, MPI_Comm*);
int MPI_Comm_split(MPI_Comm, int, int, MPI_Comm*);
int MPI_Comm_free(MPI_Comm*);
int MPI_Comm_group(MPI_Comm, MPI_Group*);
int MPI_Comm_create_group(MPI_Comm, MPI_Group, int, MPI_Comm*);
int MPI_Comm_set_errhandler(MPI_Comm, MPI_Errhandler);
int MPI_Group_excl(MPI_Group, int, const int*, MPI_Group*);
int MPI_Group_free(MPI_Group*);
int MPI_Send(const void*, int, MPI_Datatype, int, int, MPI_Comm);
int MPI_Recv(void*, int, MPI_Datatype, int, int, MPI_Comm, MPI_Status*);
int MPI_Sendrecv(const void*, int, MPI_Datatype, int, int, void*, int, MPI_Datatype, int, int, MPI_Comm, MPI_Status*);
int MPI_Isend(const void*, int, MPI_Datatype, int, int, MPI_Comm, MPI_Request*);
int MPI_Irecv(void*, int, MPI_Datatype, int, int, MPI_Comm, MPI_Request*);
int MPI_Waitall(int, MPI_Request*, MPI_Status*);
int MPI_Test(MPI_Request*, int*, MPI_Status*);
int MPI_Cancel(MPI_Request*);
int MPI_Request_free(MPI_Request*);
int MPI_Bcast(void*, int, MPI_Datatype, int, MPI_Comm);
int MPI_Allgather(const void*, int, MPI_Datatype, void*, int, MPI_Datatype, MPI_Comm);
int MPI_Allreduce(const void*, void*, int, MPI_Datatype, MPI_Op, MPI_Comm);
int MPI_Error_string(int, char*, int*);
int MPI_Iprobe(int, int, MPI_Comm, int*, MPI_Status*);
int MPI_Testall(int, MPI_Request*, int*, MPI_Status*);
int MPI_Wait(MPI_Request*, MPI_Status*);
#ifdef __cplusplus
}
#endif
#endif
