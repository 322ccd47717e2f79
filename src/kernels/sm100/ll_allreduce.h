// Host entry point of the low-latency (flag-in-data) AllReduce kernel.
#pragma once

#include "b200ccl/types.h"
#include "kernels/sm100/dev_types.h"

#include <cuda_runtime.h>

namespace b200ccl::kernels {

// Bytes of one rank's receive area for an `nranks` communicator (it must start zeroed).
std::size_t ll_area_bytes(int nranks);
// Message: args->nwords 4-byte words (≤ dev::kLlMaxWords); input and output 4-byte aligned.
// loop_ranks > 0: one cooperative launch plays that many ranks (args[0..loop_ranks)).
cudaError_t launch_ll_all_reduce(DType dtype, RedOp op, const dev::LlArgs* args, int loop_ranks, cudaStream_t stream);

}  // namespace b200ccl::kernels
