// Source-compatibility header: code written against nano-nccl's include/nano_nccl/communicator.h can
// include this file and keep using the nano_nccl:: names, which are aliases of b200ccl::.
// Not carried over: the compile-time rank/channel/block constants (kRanks, kChannels,
// kBlockThreads), which are run-time values in this library.
#pragma once

#include "b200ccl/communicator.h"

namespace nano_nccl = b200ccl;
