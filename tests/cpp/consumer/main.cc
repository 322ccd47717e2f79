// A program outside the source tree that uses the installed package through the nano_nccl/
// source-compatibility headers, as a user of the reference library would after switching.
#include "nano_nccl/communicator.h"
#include "nano_nccl/types.h"

#include <cstdio>
#include <stdexcept>

int main() {
    nano_nccl::CommunicatorConfig cfg;
    cfg.devices = {0};
    try {
        auto comm = nano_nccl::create_communicator(cfg);
        std::printf("ranks %d transport %s\n", comm->global_rank_count(), nano_nccl::transport_name(comm->transport()));
    } catch (const std::exception& e) {
        std::printf("no communicator: %s\n", e.what());  // a machine without a GPU ends here
    }
    std::printf("consumer ok %s %s\n", nano_nccl::dtype_name(nano_nccl::DType::BFloat16), nano_nccl::redop_name(nano_nccl::RedOp::Avg));
    return 0;
}
