// Out-of-band control plane for multi-process communicators: a small rendezvous that can
// all-gather byte blobs, run a barrier and pass file descriptors between the processes of one
// host. It stands where nano-nccl uses the MPI C API (src/collective/all_reduce/
// mpi_communicator.cc:112-253: MPI_Allgather of GPU counts and socket addresses, error
// consensus); MPI is optional here and this TCP rendezvous is the default.
#pragma once

#include <cstddef>
#include <memory>
#include <string>
#include <vector>

namespace b200ccl {

class Bootstrap {
public:
    virtual ~Bootstrap() = default;
    virtual int rank() const = 0;
    virtual int size() const = 0;
    // `out` receives size()*bytes, ordered by rank.
    virtual void allgather(const void* in, void* out, std::size_t bytes) = 0;
    virtual void barrier() = 0;
    // Every process contributes `fds` (same length everywhere); returns, for each process in
    // rank order, duplicates of its descriptors usable in the caller (own entries are dup()s).
    // The caller closes what it receives. Same-host only (SCM_RIGHTS over AF_UNIX).
    virtual std::vector<std::vector<int>> exchange_fds(const std::vector<int>& fds) = 0;
    // All processes agree on success: returns "" if every process passed an empty string,
    // else the first non-empty message prefixed by its rank (the MPI_Allreduce(MIN) + gather of
    // error strings of mpi_communicator.cc:38-75).
    std::string error_consensus(const std::string& local_error);
};

// Rank 0 listens on addr:port; the others connect (retrying until timeout_ms).
std::unique_ptr<Bootstrap> create_tcp_bootstrap(const std::string& addr, int port, int rank,
                                                int size, int timeout_ms = 60000);

}  // namespace b200ccl
