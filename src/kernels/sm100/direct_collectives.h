// Host-side entry points of the direct (peer load/store and NVLS) kernels.
#pragma once

#include "b200ccl/types.h"
#include "kernels/sm100/dev_types.h"

#include <cuda_runtime.h>

namespace b200ccl::kernels {

struct LaunchConfig {
    int grid = 1;    // CTAs per rank (≤ dev::kMaxCtas)
    int block = dev::kBlockThreads;
    cudaStream_t stream = nullptr;
    // Loopback emulation: one cooperative launch plays `loop_ranks` ranks (blockIdx.y = rank)
    // and `args` points to that many argument structs. 0 → normal launch of args[0].
    int loop_ranks = 0;
    int nvls_unroll = 2;  // multimem loads in flight per thread (1, 2, 4 or 8)
};

// pack_bytes: what one thread moves per access and the unit of every length in `args`: 32 (256-bit
// accesses; every peer-visible pointer 32-byte aligned, the caller's own staged buffers 16-byte
// aligned), 16, or the element size (fallback for odd counts and unaligned buffers).
// nvls: multimem kernels (sum/avg, 16-byte packs only).
cudaError_t launch_reduce(DType dtype, RedOp op, int pack_bytes, bool nvls, const dev::CollArgs* args,
                          const LaunchConfig& cfg);
cudaError_t launch_gather(const dev::GatherArgs* args, const LaunchConfig& cfg);

}  // namespace b200ccl::kernels
