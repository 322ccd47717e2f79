// A collective over ONE rank is a copy of the caller's buffer (sum, max and min of one operand
// are the operand; avg scales by 1/1). It is moved by TMA bulk copies through shared memory.
#pragma once

#include "kernels/sm100/dev_types.h"

#include <cuda_runtime.h>

namespace b200ccl::kernels {

// src, dst: this GPU's own memory, 16-byte aligned, not overlapping; bytes: a positive multiple of 16.
// max_ctas <= 0: one CTA per SM. A wait that runs out is recorded in *status (may be null).
cudaError_t launch_local_copy(const void* src, void* dst, unsigned long long bytes, int max_ctas, dev::Status* status,
                              cudaStream_t stream);

}  // namespace b200ccl::kernels
