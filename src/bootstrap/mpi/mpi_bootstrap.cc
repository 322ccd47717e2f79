// MPI adapter of the control plane. Compiled only with B200CCL_ENABLE_MPI=ON (the image this
// library is developed on has no MPI; the TCP rendezvous is the default and is what the tests use).
// Only the MPI C API is used (no C++ bindings), as in the reference
// (src/collective/all_reduce/mpi_communicator.cc; tests/mpi_c_api_link_static.py).
#include "b200ccl/mpi.h"

#if defined(B200CCL_ENABLE_MPI)

#include <cstring>
#include <stdexcept>
#include <vector>

namespace b200ccl {

namespace {

void mpi_check(int rc, const char* what) {
    if (rc == MPI_SUCCESS) return;
    char text[MPI_MAX_ERROR_STRING] = {0};
    int len = 0;
    MPI_Error_string(rc, text, &len);
    throw std::runtime_error(std::string(what) + " failed: " + std::string(text, len));
}

class MpiBootstrap final : public Bootstrap {
public:
    explicit MpiBootstrap(MPI_Comm comm) : comm_(comm) {
        int initialized = 0, finalized = 0;
        MPI_Initialized(&initialized);
        MPI_Finalized(&finalized);
        if (!initialized || finalized) throw std::runtime_error("MPI must be initialised and not finalised");
        mpi_check(MPI_Comm_rank(comm_, &rank_), "MPI_Comm_rank");
        mpi_check(MPI_Comm_size(comm_, &size_), "MPI_Comm_size");
        // Descriptor passing needs AF_UNIX sockets; reuse the TCP rendezvous for that part, with
        // the address published by rank 0 through MPI.
        int port = 0;
        if (rank_ == 0) port = 20000 + (static_cast<int>(::getpid()) % 20000);
        mpi_check(MPI_Bcast(&port, 1, MPI_INT, 0, comm_), "MPI_Bcast");
        fd_helper_ = create_tcp_bootstrap("127.0.0.1", port, rank_, size_);
    }
    int rank() const override { return rank_; }
    int size() const override { return size_; }
    void allgather(const void* in, void* out, std::size_t bytes) override {
        mpi_check(MPI_Allgather(in, static_cast<int>(bytes), MPI_BYTE, out, static_cast<int>(bytes), MPI_BYTE, comm_), "MPI_Allgather");
    }
    void barrier() override { mpi_check(MPI_Barrier(comm_), "MPI_Barrier"); }
    std::vector<std::vector<int>> exchange_fds(const std::vector<int>& fds) override { return fd_helper_->exchange_fds(fds); }

private:
    MPI_Comm comm_;
    int rank_ = 0, size_ = 1;
    std::unique_ptr<Bootstrap> fd_helper_;
};

}  // namespace

std::unique_ptr<Bootstrap> create_mpi_bootstrap(MPI_Comm control_comm) {
    return std::unique_ptr<Bootstrap>(new MpiBootstrap(control_comm));
}

std::unique_ptr<Communicator> create_communicator_from_mpi(MPI_Comm control_comm, const CommunicatorConfig& config) {
    // The bootstrap must outlive the communicator: it is kept alive for the life of the process.
    static std::vector<std::unique_ptr<Bootstrap>> keep;
    keep.push_back(create_mpi_bootstrap(control_comm));
    return create_communicator_from_bootstrap(*keep.back(), config);
}

}  // namespace b200ccl

#endif  // B200CCL_ENABLE_MPI
