// Deterministic test data: element i of rank r is a pure function of (seed, r, i), so the
// expected result of a collective can be recomputed anywhere (host or device) without reading
// the inputs back. uniform[-1,1) or N(0,1), rounded to the element type before it is used.
//
// nano-nccl fills inputs with a fixed arithmetic pattern and sums them on the host
// (src/collective/all_reduce/ring_simple.cu:33-70); this generator gives the seeded random data
// asked for by the benchmark configurations and keeps verification off the host for GiB sizes.
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define B2_HD __host__ __device__ inline
#else
#define B2_HD inline
#endif

namespace b200ccl::datagen {

B2_HD std::uint64_t mix64(std::uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

B2_HD float uniform_pm1(std::uint64_t seed, int rank, std::uint64_t index) {
    const std::uint64_t h = mix64(mix64(seed * 1000003ull + static_cast<std::uint64_t>(rank)) ^ index);
    // 24 random bits → [0,1) → [-1,1)
    return static_cast<float>(h >> 40) * (1.0f / 8388608.0f) - 1.0f;
}

B2_HD float normal01(std::uint64_t seed, int rank, std::uint64_t index) {
    const std::uint64_t h1 = mix64(mix64(seed * 1000003ull + static_cast<std::uint64_t>(rank)) ^ (2 * index));
    const std::uint64_t h2 = mix64(mix64(seed * 1000003ull + static_cast<std::uint64_t>(rank)) ^ (2 * index + 1));
    const float u1 = (static_cast<float>(h1 >> 40) + 1.0f) * (1.0f / 16777217.0f);  // (0,1)
    const float u2 = static_cast<float>(h2 >> 40) * (1.0f / 16777216.0f);
#if defined(__CUDA_ARCH__)
    return sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
#else
    return __builtin_sqrtf(-2.0f * __builtin_logf(u1)) * __builtin_cosf(6.28318530717958647692f * u2);
#endif
}

B2_HD float value(bool uniform, std::uint64_t seed, int rank, std::uint64_t index) {
    return uniform ? uniform_pm1(seed, rank, index) : normal01(seed, rank, index);
}

}  // namespace b200ccl::datagen
