// Source-compatibility header for nano-nccl's include/nano_nccl/mpi.h. The MPI adapter is
// optional (configure with B200CCL_ENABLE_MPI=ON where an MPI C library exists); without it
// multi-process communicators are created from the TCP rendezvous of b200ccl/bootstrap.h.
#pragma once

#include "b200ccl/mpi.h"

namespace nano_nccl = b200ccl;
