// Optional MPI entry point: builds a communicator whose control plane is an MPI communicator.
// Declared always; defined only in builds configured with B200CCL_ENABLE_MPI=ON.
//
// Parity: nano-nccl include/nano_nccl/mpi.h:11-12 (create_communicator_from_mpi) and
// src/collective/all_reduce/mpi_communicator.cc:112-253. The adapter wraps the MPI communicator
// in the Bootstrap interface (all-gather → MPI_Allgather, barrier → MPI_Barrier, error consensus
// → MPI_Allreduce(MIN) + gather of messages) and then follows the same path as the TCP rendezvous.
#pragma once

#include "b200ccl/bootstrap.h"
#include "b200ccl/communicator.h"

#if defined(B200CCL_ENABLE_MPI)
#include <mpi.h>

namespace b200ccl {

// The MPI library must be initialised and not finalised. Ranks are laid out in MPI rank order.
std::unique_ptr<Communicator> create_communicator_from_mpi(MPI_Comm control_comm, const CommunicatorConfig& config);
// The MPI communicator as a Bootstrap (descriptor passing still uses AF_UNIX sockets between the
// processes of one host).
std::unique_ptr<Bootstrap> create_mpi_bootstrap(MPI_Comm control_comm);

}  // namespace b200ccl
#endif
