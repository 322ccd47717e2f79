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
    int nvls_unroll = 4;  // multimem loads in flight per thread (2, 4 or 8)
};

// wide: 16-byte packs (all pointers 16-byte aligned, lengths in 16-byte units); else one element
// per access. nvls: multimem kernels (sum/avg, wide only).
cudaError_t launch_reduce(DType dtype, RedOp op, bool wide, bool nvls, const dev::CollArgs* args,
                          const LaunchConfig& cfg);
cudaError_t launch_gather(const dev::GatherArgs* args, const LaunchConfig& cfg);

}  // namespace b200ccl::kernels
