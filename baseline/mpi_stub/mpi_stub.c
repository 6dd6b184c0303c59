/* Definitions for mpi_stub/mpi.h: every call reports failure. */
#include <string.h>

#include "mpi.h"
#define FAIL { return MPI_ERR_OTHER; }
int MPI_Init(int* a, char*** b) { (void)a; (void)b; return MPI_ERR_OTHER; }
int MPI_Comm_size(MPI_Comm c, int* n) { (void)c; *n = 1; return MPI_ERR_OTHER; }
int MPI_Comm_rank(MPI_Comm c, int* r) { (void)c; *r = 0; return MPI_ERR_OTHER; }
int MPI_Comm_dup(MPI_Comm c, MPI_Comm* o) { (void)c; *o = MPI_COMM_NULL; return MPI_ERR_OTHER; }
int MPI_Comm_split(MPI_Comm c, int a, int b, MPI_Comm* o) { (void)c; (void)a; (void)b; *o = MPI_COMM_NULL; return MPI_ERR_OTHER; }
int MPI_Comm_free(MPI_Comm* c) { (void)c; return MPI_ERR_OTHER; }
int MPI_Comm_group(MPI_Comm c, MPI_Group* g) { (void)c; *g = 0; return MPI_ERR_OTHER; }
int MPI_Comm_create_group(MPI_Comm c, MPI_Group g, int t, MPI_Comm* o) { (void)c; (void)g; (void)t; *o = MPI_COMM_NULL; return MPI_ERR_OTHER; }
int MPI_Comm_set_errhandler(MPI_Comm c, MPI_Errhandler e) { (void)c; (void)e; return MPI_ERR_OTHER; }
int MPI_Group_excl(MPI_Group g, int n, const int* r, MPI_Group* o) { (void)g; (void)n; (void)r; *o = 0; return MPI_ERR_OTHER; }
int MPI_Group_free(MPI_Group* g) { (void)g; return MPI_ERR_OTHER; }
int MPI_Send(const void* b, int n, MPI_Datatype d, int p, int t, MPI_Comm c) { (void)b; (void)n; (void)d; (void)p; (void)t; (void)c; FAIL }
int MPI_Recv(void* b, int n, MPI_Datatype d, int p, int t, MPI_Comm c, MPI_Status* s) { (void)b; (void)n; (void)d; (void)p; (void)t; (void)c; (void)s; FAIL }
int MPI_Sendrecv(const void* a, int b, MPI_Datatype c, int d, int e, void* f, int g, MPI_Datatype h, int i, int j, MPI_Comm k, MPI_Status* l) { (void)a; (void)b; (void)c; (void)d; (void)e; (void)f; (void)g; (void)h; (void)i; (void)j; (void)k; (void)l; FAIL }
int MPI_Isend(const void* b, int n, MPI_Datatype d, int p, int t, MPI_Comm c, MPI_Request* r) { (void)b; (void)n; (void)d; (void)p; (void)t; (void)c; *r = MPI_REQUEST_NULL; FAIL }
int MPI_Irecv(void* b, int n, MPI_Datatype d, int p, int t, MPI_Comm c, MPI_Request* r) { (void)b; (void)n; (void)d; (void)p; (void)t; (void)c; *r = MPI_REQUEST_NULL; FAIL }
int MPI_Waitall(int n, MPI_Request* r, MPI_Status* s) { (void)n; (void)r; (void)s; FAIL }
int MPI_Test(MPI_Request* r, int* f, MPI_Status* s) { (void)r; (void)s; *f = 1; FAIL }
int MPI_Cancel(MPI_Request* r) { (void)r; FAIL }
int MPI_Request_free(MPI_Request* r) { (void)r; FAIL }
int MPI_Bcast(void* b, int n, MPI_Datatype d, int r, MPI_Comm c) { (void)b; (void)n; (void)d; (void)r; (void)c; FAIL }
int MPI_Allgather(const void* a, int b, MPI_Datatype c, void* d, int e, MPI_Datatype f, MPI_Comm g) { (void)a; (void)b; (void)c; (void)d; (void)e; (void)f; (void)g; FAIL }
int MPI_Allreduce(const void* a, void* b, int c, MPI_Datatype d, MPI_Op e, MPI_Comm f) { (void)a; (void)b; (void)c; (void)d; (void)e; (void)f; FAIL }
int MPI_Error_string(int e, char* s, int* n) { (void)e; strcpy(s, "MPI stand-in: no MPI on this machine"); *n = (int)strlen(s); return MPI_SUCCESS; }
int MPI_Iprobe(int p, int t, MPI_Comm c, int* f, MPI_Status* s) { (void)p; (void)t; (void)c; (void)s; *f = 0; FAIL }
int MPI_Testall(int n, MPI_Request* r, int* f, MPI_Status* s) { (void)n; (void)r; (void)s; *f = 1; FAIL }
int MPI_Wait(MPI_Request* r, MPI_Status* s) { (void)r; (void)s; FAIL }
