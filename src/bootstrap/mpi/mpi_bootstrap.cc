// MPI adapter of the control plane. Compiled only with B200CCL_ENABLE_MPI=ON (the TCP rendezvous is
// the default). Where no MPI is installed the adapter is still compiled and run by
// tests/cpp/fake_mpi/test_mpi_adapter.cc against an in-process stand-in for the few MPI calls it makes.
// Only the MPI C API is used (no C++ bindings), as in the reference
// (src/collective/all_reduce/mpi_communicator.cc; tests/mpi_c_api_link_static.py).
#include "b200ccl/mpi.h"

#if defined(B200CCL_ENABLE_MPI)

#include "bootstrap/fd_exchange.h"

#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
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
    }
    int rank() const override { return rank_; }
    int size() const override { return size_; }
    void allgather(const void* in, void* out, std::size_t bytes) override {
        if (bytes > static_cast<std::size_t>(INT32_MAX)) throw std::invalid_argument("MPI bootstrap: blob too large");
        mpi_check(MPI_Allgather(in, static_cast<int>(bytes), MPI_BYTE, out, static_cast<int>(bytes), MPI_BYTE, comm_), "MPI_Allgather");
    }
    void barrier() override { mpi_check(MPI_Barrier(comm_), "MPI_Barrier"); }
    // Descriptors cannot travel through MPI: they go over AF_UNIX sockets whose names are agreed
    // through this object's own all-gather.
    std::vector<std::vector<int>> exchange_fds(const std::vector<int>& fds) override {
        if (!fdx_) fdx_.reset(new FdExchange(*this, 60000));
        return fdx_->exchange(fds);
    }

private:
    MPI_Comm comm_;
    int rank_ = 0, size_ = 1;
    std::unique_ptr<FdExchange> fdx_;
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
