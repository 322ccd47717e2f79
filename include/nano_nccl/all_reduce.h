// Source-compatibility header for nano-nccl's include/nano_nccl/all_reduce.h
// (run_all_reduce_bench(BenchConfig, std::vector<BenchResult>*)).
#pragma once

#include "b200ccl/bench.h"

namespace nano_nccl = b200ccl;
