// hxcclCommInitMPI, compiled only where an MPI installation exists (-DHXCCL_HAVE_MPI). MPI is
// used for nothing but handing the unique id around: rank 0 makes it, MPI_Bcast carries it,
// and every rank then joins through the socket bootstrap, which is what the reference does
// under HXCCL_BOOTSTRAP=socket (src/comm.cc:89-103). Host payload therefore travels over this
// library's own mesh and device payload over the windows; there is no MPI transport here.
#ifdef HXCCL_HAVE_MPI
#include <mpi.h>

#include "hxccl.h"

extern "C" hxcclResult_t hxcclCommInitMPI(hxcclComm_t* comm, MPI_Comm mpi) {
  if (!comm || mpi == MPI_COMM_NULL) return hxcclInvalidArgument;
  int rank = 0, size = 0;
  MPI_Comm_rank(mpi, &rank);
  MPI_Comm_size(mpi, &size);
  hxcclUniqueId id;
  int ok = 1;
  if (rank == 0) ok = hxcclGetUniqueId(&id) == hxcclSuccess;
  MPI_Bcast(&ok, 1, MPI_INT, 0, mpi);
  if (!ok) return hxcclSystemError;
  MPI_Bcast(&id, sizeof id, MPI_BYTE, 0, mpi);
  return hxcclCommInitRank(comm, size, id, rank);
}
#endif
