// Ring + Simple-protocol kernels (AllReduce, ReduceScatter, AllGather) and their argument types.
#pragma once

#include "b200ccl/types.h"
#include "kernels/sm100/dev_types.h"

#include <cuda_runtime.h>

namespace b200ccl::dev {

// Per rank and channel: time spent in each part of a slice, in ns of %globaltimer, summed by
// thread 0. Filled only when a stats pointer is passed (B200CCL_RING_TURNAROUND=1).
// Parity: nano-nccl src/collective/all_reduce/ring_turnaround.h:10-39.
struct RingTurnaroundStats {
    unsigned long long wait_recv_ns;
    unsigned long long wait_send_ns;
    unsigned long long compute_ns;
    unsigned long long post_ns;
    unsigned long long slices;
    unsigned long long empty_slices;  // elided: no wait, no post, no step
};

// One channel's two edges as seen from one rank. The pointers are fixed for the lifetime of the
// communicator. Ownership follows nano-nccl src/transport/p2p/p2p_step_counters.h:32-35: a rank
// polls words in its own memory (send_head, recv_tail) and publishes into its neighbours'
// (send_tail → next rank's recv_tail word, recv_head → previous rank's send_head word). For
// SHM and network edges all four words live in mapped host memory.
struct RingChannel {
    void* send_fifo;         // next rank's FIFO for this channel (or host FIFO of the outgoing edge)
    const void* recv_fifo;   // this rank's FIFO for this channel (or host FIFO of the incoming edge)
    unsigned long long* send_tail;  // publish: "slice written up to this step"
    unsigned long long* send_head;  // poll:    "next rank consumed up to this step" (credit)
    unsigned long long* recv_tail;  // poll:    "previous rank wrote up to this step"
    unsigned long long* recv_head;  // publish: "I consumed up to this step" (credit)
    unsigned long long* send_base;  // persisted progress of the outgoing edge (local)
    unsigned long long* recv_base;  // persisted progress of the incoming edge (local)
    unsigned int* send_sizes;       // network edges: payload bytes per FIFO step slot, else null
    const unsigned int* abort_word; // network edges: host word set by a failed proxy, else null
    RingTurnaroundStats* stats;     // optional
};

// The addresses of one channel's eight words and FIFOs, for inspection by tests.
struct RingChannelView {
    const void* send_fifo;
    const void* recv_fifo;
    const void* send_tail;
    const void* send_head;
    const void* recv_tail;
    const void* recv_head;
    const void* send_base;
    const void* recv_base;
};

struct RingArgs {
    const void* input;
    void* output;
    const RingChannel* channels;  // [nchannels], device-visible
    ControlBlock* own_ctrl;       // this rank's control block (abort flag, failure latch)
    Status* status;
    unsigned long long count;       // the API's count
    unsigned long long step_elems;  // elements of this dtype per FIFO step
    unsigned long long timeout_ns;
    float scale;
    int rank;
    int nranks;
    int nchannels;
    int collective;  // b200ccl::Collective
    int wide;        // 1: 16-byte accesses and TMA staging of local input are allowed
};

}  // namespace b200ccl::dev

namespace b200ccl::kernels {

struct RingLaunch {
    cudaStream_t stream = nullptr;
    int loop_ranks = 0;  // >0: one cooperative launch plays that many ranks (args[0..loop_ranks))
};

// Launches one CTA per channel (512 threads). `args` points to one struct, or loop_ranks structs.
cudaError_t launch_ring(DType dtype, RedOp op, const dev::RingArgs* args, const RingLaunch& cfg);
int ring_block_threads();

}  // namespace b200ccl::kernels
