#include "transport/rdma/protocol.h"

#include "core/env.h"
#include "transport/rdma/fake_verbs.h"
#include "transport/rdma/verbs_backend.h"

namespace b200ccl::transport::rdma {

DataPlane data_plane_from_env() {
    return env::get_bool("B200CCL_RDMA_USE_WRITE", false, "NANO_NCCL_RDMA_USE_WRITE") ? DataPlane::WriteCts : DataPlane::SendRecv;
}
FifoPlacement fifo_placement_from_env() {
    return env::get_bool("B200CCL_RDMA_GDR", false, "NANO_NCCL_RDMA_GDR") ? FifoPlacement::Gdr : FifoPlacement::HostPinned;
}
bool shared_progress_from_env() {
    return env::get_bool("B200CCL_RDMA_SHARED_PROGRESS", false, "NANO_NCCL_RDMA_SHARED_PROGRESS");
}

#if defined(B200CCL_ENABLE_RDMA_VERBS)
std::shared_ptr<VerbsBackend> create_ibverbs_backend();
#endif

std::shared_ptr<VerbsBackend> create_backend(const std::string& name) {
    std::string which = name.empty() ? env::get_string("B200CCL_RDMA_BACKEND", "") : name;
    if (which.empty()) {
#if defined(B200CCL_ENABLE_RDMA_VERBS)
        which = "ibverbs";
#else
        which = "fake";
#endif
    }
    if (which == "fake") return std::make_shared<FakeVerbs>();
    if (which == "ibverbs") {
#if defined(B200CCL_ENABLE_RDMA_VERBS)
        return create_ibverbs_backend();
#else
        throw std::runtime_error("rdma: this build has no libibverbs backend (configure with B200CCL_ENABLE_RDMA_VERBS=ON)");
#endif
    }
    throw std::invalid_argument("rdma: unknown backend '" + which + "'");
}

}  // namespace b200ccl::transport::rdma
