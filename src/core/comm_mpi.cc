// hxcclCommInitMPI, compiled only where an MPI installation exists (-DHXCCL_HAVE_MPI).
// By default the communicator's control messages and host payload travel over MPI itself
// (ctrl/mpi_carrier.cc), as in the reference, whose MPI communicators use MpiNet and
// MpiTransport (src/comm.cc:21-34). With HXCCL_BOOTSTRAP=socket MPI only hands the unique id
// around and every rank then joins through the socket bootstrap (the reference's switch of the
// same name, src/comm.cc:89-103). Device payload goes through the windows either way.
#ifdef HXCCL_HAVE_MPI
#include <mpi.h>

#include <cstdlib>
#include <cstring>
#include <numeric>

#include "core/comm.h"
#include "ctrl/mpi_carrier.h"

extern "C" hxcclResult_t hxcclCommInitMPI(hxcclComm_t* comm, MPI_Comm mpi) {
  if (!comm || mpi == MPI_COMM_NULL) return hxcclInvalidArgument;
  int rank = 0, size = 0;
  MPI_Comm_rank(mpi, &rank);
  MPI_Comm_size(mpi, &size);
  const char* boot = std::getenv("HXCCL_BOOTSTRAP");
  if (boot && std::strcmp(boot, "socket") == 0) {
    hxcclUniqueId id;
    int ok = 1;
    if (rank == 0) ok = hxcclGetUniqueId(&id) == hxcclSuccess;
    MPI_Bcast(&ok, 1, MPI_INT, 0, mpi);
    if (!ok) return hxcclSystemError;
    MPI_Bcast(&id, sizeof id, MPI_BYTE, 0, mpi);
    return hxcclCommInitRank(comm, size, id, rank);
  }
  auto carrier = std::make_shared<hx::MpiCarrier>(mpi);
  if (!carrier->ok()) return hxcclSystemError;
  // Every communicator made from MPI gets a channel id of its own, agreed by the ranks: rank 0
  // draws it. (Children made by Split / Shrink derive theirs from it as always.)
  uint64_t id = 0;
  if (rank == 0) {
    static uint64_t made = 0;
    id = hx::mix_id(0x6d7069ull, ++made, uint64_t(size));
  }
  if (MPI_Bcast(&id, int(sizeof id), MPI_BYTE, 0, mpi) != MPI_SUCCESS) return hxcclSystemError;
  std::vector<int> members(static_cast<size_t>(size));
  std::iota(members.begin(), members.end(), 0);
  return hx::comm_from_channel(comm, std::make_shared<hx::Channel>(carrier, id, members, rank));
}
#endif
