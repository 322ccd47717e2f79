// NVTX ranges and a profiler capture window for the benchmark. Everything here compiles to nothing
// unless the build is configured with B200CCL_ENABLE_BENCH_PROFILING=ON, so that numbers are never
// taken from an instrumented binary. Warm-up stays outside the capture window.
// Parity: nano-nccl src/collective/all_reduce/bench_profiling.h:16-50 (NvtxRange, ProfilerSession;
// range text "all_reduce size=<B>B [iteration=<i>]").
#pragma once

#include <cstddef>
#include <string>

#if defined(B200CCL_ENABLE_BENCH_PROFILING)
#include <cuda_profiler_api.h>
#include <nvtx3/nvToolsExt.h>
#endif

namespace b200ccl {

inline std::string bench_range_name(const char* collective, std::size_t bytes, int iteration = -1) {
    std::string s = std::string(collective) + " size=" + std::to_string(bytes) + "B";
    if (iteration >= 0) s += " iteration=" + std::to_string(iteration);
    return s;
}

class NvtxRange {
public:
    explicit NvtxRange(const std::string& name) {
#if defined(B200CCL_ENABLE_BENCH_PROFILING)
        nvtxRangePushA(name.c_str());
#else
        (void)name;
#endif
    }
    ~NvtxRange() {
#if defined(B200CCL_ENABLE_BENCH_PROFILING)
        nvtxRangePop();
#endif
    }
    NvtxRange(const NvtxRange&) = delete;
    NvtxRange& operator=(const NvtxRange&) = delete;
};

class ProfilerSession {
public:
    ProfilerSession() {
#if defined(B200CCL_ENABLE_BENCH_PROFILING)
        cudaProfilerStart();
#endif
    }
    ~ProfilerSession() {
#if defined(B200CCL_ENABLE_BENCH_PROFILING)
        cudaProfilerStop();
#endif
    }
    ProfilerSession(const ProfilerSession&) = delete;
    ProfilerSession& operator=(const ProfilerSession&) = delete;
};

constexpr bool bench_profiling_enabled() {
#if defined(B200CCL_ENABLE_BENCH_PROFILING)
    return true;
#else
    return false;
#endif
}

}  // namespace b200ccl
