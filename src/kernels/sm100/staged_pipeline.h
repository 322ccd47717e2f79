// AllReduce of buffers that peers cannot address, as a tile pipeline inside one kernel.
#pragma once

#include "b200ccl/types.h"
#include "kernels/sm100/dev_types.h"

#include <cuda_runtime.h>

namespace b200ccl::dev {

// Per-rank flags of the pipeline, in symmetric memory. Row [cta][src] of rank dst is written by
// CTA `cta` of rank `src` (release, system scope) and polled by CTA `cta` of rank dst (acquire).
// Every counter is the number of tiles that CTA index has taken through that stage since the
// communicator was created; it only grows, so nothing is ever reset between calls.
struct PipeFlags {
    unsigned long long in_ready[kMaxCtas][kMaxRanks];  // tiles copied into src's arena
    unsigned long long reduced[kMaxCtas][kMaxRanks];   // tiles whose shard src reduced and stored into every arena
    unsigned long long drained[kMaxCtas][kMaxRanks];   // tiles src copied out of its arena
    unsigned long long base[kMaxCtas];                 // local: tiles this CTA index finished in earlier calls
};

// Where the pipeline's time goes, summed over CTAs and calls by the leading lane of every stage,
// in SM clock cycles (despite the field names). Filled only when a pointer is passed
// (B200CCL_PIPELINE_STATS=1).
struct PipeStats {
    unsigned long long in_wait_slot_ns;   // copy-in: waiting for the arena slot to be free
    unsigned long long in_copy_ns;        // copy-in: moving the tile
    unsigned long long red_wait_ns;       // reduce: waiting for every rank's tile (and a free output slot)
    unsigned long long red_work_ns;       // reduce: loads, arithmetic, stores
    unsigned long long out_wait_ns;       // copy-out: waiting for every rank's shard
    unsigned long long out_copy_ns;       // copy-out: moving the tile
    unsigned long long tiles;             // tiles counted (per CTA and call)
    unsigned long long calls;             // CTAs x calls
    unsigned long long kernel_ns;         // whole kernel, CTA 0 only, summed over calls
};

struct PipeArgs {
    const void* user_in;   // this rank's input (its own memory, 16-byte aligned)
    void* user_out;        // this rank's output
    void* arena_in[kMaxRanks];    // every rank's input half of the staging arena
    void* arena_out[kMaxRanks];   // every rank's output half
    const void* mc_in;     // multicast alias of the input halves (switch variant), else null
    void* mc_out;          // multicast alias of the output halves
    ControlBlock* ctrl[kMaxRanks];
    PipeFlags* flags[kMaxRanks];
    Status* status;
    PipeStats* stats;      // optional
    unsigned long long bytes;       // message size, a multiple of 16
    unsigned long long tile_bytes;  // a multiple of 16; CTA b owns tiles b, b + grid, ...
    unsigned long long timeout_ns;
    unsigned long long plan_hash;
    float scale;
    int rank;
    int nranks;
    int slots;  // arena slots per CTA and half; slot s of CTA b starts at (b * slots + s) * tile_bytes
};

}  // namespace b200ccl::dev

namespace b200ccl::kernels {

struct PipeLaunch {
    int grid = 1;
    cudaStream_t stream = nullptr;
    int loop_ranks = 0;   // >0: one cooperative launch plays that many ranks (args[0..loop_ranks))
    bool nvls = false;    // reduce with multimem.ld_reduce / multimem.st (sum and avg only)
    int nvls_unroll = 2;
};

// Dynamic shared memory one CTA of the pipeline kernel needs.
std::size_t pipeline_smem_bytes();

cudaError_t launch_staged_pipeline(DType dtype, RedOp op, const dev::PipeArgs* args, const PipeLaunch& cfg);

}  // namespace b200ccl::kernels
