// Argument checks shared by the three collectives. Kept apart from the communicator so that
// the contract can be tested without a GPU. Messages carry the key words of nano-nccl's
// diagnostics (src/collective/all_reduce/communicator.cu:832-859: "one entry per rank",
// "non-null", "positive", "reduction", "in-place", "unsupported dtype").
#pragma once

#include "b200ccl/communicator.h"

namespace b200ccl {

// Throws std::invalid_argument. `local_ranks` is the number of GPUs this process drives.
void validate_collective_args(Collective collective, const CollectiveArgs& args, int local_ranks,
                              bool allow_in_place);

// Throws std::invalid_argument when `config.devices` is not a non-empty list of distinct
// ordinals below `visible_devices` (or, for loopback, exactly one device and 1..kMaxRanks ranks).
void validate_config(const CommunicatorConfig& config, int visible_devices);

}  // namespace b200ccl
