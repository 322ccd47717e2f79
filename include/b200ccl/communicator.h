// Communicator: owns the peer mappings, flag pages, staging arenas and FIFOs of one group
// of GPUs and enqueues AllReduce / ReduceScatter / AllGather on caller-owned streams.
//
// Parity: same shape as nano-nccl include/nano_nccl/communicator.h:17-58
// (CommunicatorConfig, CollectiveArgs, move-only Communicator, create_communicator), with
// these differences: the rank count is the size of `devices` (not a build constant);
// reduce_scatter and all_gather are implemented (the reference throws,
// src/collective/all_reduce/communicator.cu:1295-1301); a process may own one GPU of a larger
// group (see bootstrap.h); buffers may be taken from a symmetric heap, which lets every
// peer and the NVSwitch multicast engine address them without staging.
//
// Count semantics: all_reduce — `count` elements in and out on every rank;
// reduce_scatter — recv holds `count`, send holds count*nranks, rank r receives block r;
// all_gather — send holds `count`, recv holds count*nranks (redop ignored).
#pragma once

#include "b200ccl/types.h"

#include <cstddef>
#include <memory>
#include <string>
#include <vector>

#include <cuda_runtime.h>

namespace b200ccl {

class Bootstrap;

struct CommunicatorConfig {
    std::vector<int> devices;                       // CUDA device ids owned by this process
    TransportKind transport = TransportKind::Auto;  // explicit kinds fail instead of falling back
    Algo algo = Algo::Auto;                         // Auto → per-call choice from the tuning table
    int channels = 0;                               // ring channels; 0 → default/env
    std::size_t staging_bytes = 0;                  // per-rank staging arena; 0 → default/env
    double wait_timeout_ms = 0;                     // bound on every device wait; 0 → default/env
    bool loopback = false;  // emulate `loopback_ranks` ranks on devices[0] with one launch per call
    int loopback_ranks = 0;
    bool enable_nvls = true;  // use NVSwitch multicast where the driver exposes it
    // Upper bound on the CTAs one collective occupies per GPU (0 → measured defaults / B200CCL_MAX_CTAS).
    // A small value (16-32) leaves SMs to kernels that run beside the collective, at some bandwidth cost.
    int max_ctas = 0;
};

struct CollectiveArgs {
    std::vector<const void*> send_buffers;  // one entry per LOCAL rank
    std::vector<void*> recv_buffers;
    std::vector<cudaStream_t> streams;
    std::size_t count = 0;
    DType dtype = DType::Float;
    RedOp redop = RedOp::Sum;
    // all_reduce only: accept send == recv. Off by default, like the reference, which rejects
    // in-place calls (communicator.cu:855-857). In-place calls never use the one-shot kernel on
    // buffers that peers read directly.
    bool allow_in_place = false;
};

// What one call resolved to; for logs, tests and the tuner.
struct CallInfo {
    Collective collective = Collective::AllReduce;
    Algo algo = Algo::Auto;
    int grid = 0;
    int block = 0;
    bool staged_in = false;   // input went through the staging arena
    bool staged_out = false;  // output went through the staging arena
    bool vectorized = false;  // 16-byte path (false → scalar fallback for odd sizes/alignments)
    int pack_bytes = 0;       // bytes one thread moves per access: 32, 16 or the element size (0: not applicable)
};

class Communicator {
public:
    Communicator(const Communicator&) = delete;
    Communicator& operator=(const Communicator&) = delete;
    Communicator(Communicator&&) noexcept;
    Communicator& operator=(Communicator&&) noexcept;
    ~Communicator();

    void all_reduce(const CollectiveArgs& args);
    void reduce_scatter(const CollectiveArgs& args);
    void all_gather(const CollectiveArgs& args);

    // Throws the first latched asynchronous failure (device wait timeout, abort, proxy error).
    // After a failure every new collective is rejected.
    void check_async_error() const;

    int local_rank_count() const noexcept;
    int global_rank_count() const noexcept;
    int first_global_rank() const noexcept;
    TransportKind transport() const noexcept;
    bool nvls_available() const noexcept;

    // Symmetric heap. COLLECTIVE over all processes of the communicator: every process calls
    // with the same size, in the same order. Returns one pointer per local rank. Memory from
    // here is mapped on every peer (and bound to the multicast object when NVLS is available),
    // so collectives on it run without staging. Buffers passed to one call must sit at the
    // same offset of the same allocation on every rank.
    std::vector<void*> alloc_symmetric(std::size_t bytes);
    void free_symmetric(const std::vector<void*>& ptrs);

    // Registration of ordinary device buffers (cudaMalloc memory, e.g. tensors of a framework's
    // caching allocator). COLLECTIVE: every process passes its own buffer(s) of `bytes` bytes, one per
    // local rank, in the same call order. Afterwards collectives on these buffers (or on parts of
    // them at the same offset on every rank) load and store peers' copies directly instead of
    // going through the staging arena. In a single-process communicator this is a no-op, since
    // every device buffer is already peer-addressable. Unregister before freeing the memory.
    void register_buffers(const std::vector<void*>& ptrs, std::size_t bytes);
    void unregister_buffers(const std::vector<void*>& ptrs);

    CallInfo last_call() const noexcept;
    // Addresses that one local rank's ring channel is wired to, in the order send_fifo, recv_fifo,
    // send_tail, send_head, recv_tail, recv_head, send_base, recv_base (for tests that check which
    // GPU, or the host, owns each of them). Throws until a ring collective has run.
    std::vector<const void*> ring_channel_pointers(int local_rank, int channel) const;
    std::string describe() const;  // topology + per-edge transport report, one line per item

private:
    class Impl;
    explicit Communicator(std::unique_ptr<Impl> impl);
    std::unique_ptr<Impl> impl_;
    friend std::unique_ptr<Communicator> create_communicator(const CommunicatorConfig&);
    friend std::unique_ptr<Communicator> create_communicator_from_bootstrap(
        Bootstrap&, const CommunicatorConfig&);
};

// Single process owning every GPU of the group (devices.size() ranks, rank i = devices[i]).
std::unique_ptr<Communicator> create_communicator(const CommunicatorConfig& config);

// One process of a multi-process group: `devices` are this process's GPUs; global ranks are
// assigned in bootstrap-rank order. Peer memory is shared through exported allocation handles.
std::unique_ptr<Communicator> create_communicator_from_bootstrap(
    Bootstrap& bootstrap, const CommunicatorConfig& config);

}  // namespace b200ccl
