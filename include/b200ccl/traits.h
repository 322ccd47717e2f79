// Compile-time description of the element types and reduction operators.
//
// Parity: nano-nccl include/nano_nccl/traits.h:13-73. Two deliberate differences:
// 16-bit types are always widened to fp32 before they are combined (the reference adds in
// half/bf16 at every ring hop, src/kernels/ring_simple_kernel.cuh:166-219), and Max/Min
// return NaN when either operand is NaN for every dtype.
#pragma once

#include "b200ccl/types.h"

#include <cstddef>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace b200ccl {

template <DType>
struct DTypeTraits;

template <>
struct DTypeTraits<DType::Float> {
    using type = float;
    static constexpr std::size_t kSize = 4;
    static constexpr float kDefaultEpsilon = 1e-5f;
    static __host__ __device__ type from_float(float v) { return v; }
    static __host__ __device__ float to_float(type v) { return v; }
};

template <>
struct DTypeTraits<DType::Float16> {
    using type = __half;
    static constexpr std::size_t kSize = 2;
    static constexpr float kDefaultEpsilon = 1e-2f;
    static __host__ __device__ type from_float(float v) { return __float2half(v); }
    static __host__ __device__ float to_float(type v) { return __half2float(v); }
};

template <>
struct DTypeTraits<DType::BFloat16> {
    using type = __nv_bfloat16;
    static constexpr std::size_t kSize = 2;
    static constexpr float kDefaultEpsilon = 1e-1f;
    static __host__ __device__ type from_float(float v) { return __float2bfloat16(v); }
    static __host__ __device__ float to_float(type v) { return __bfloat162float(v); }
};

// Operators act on fp32 accumulators. Avg combines like Sum; the 1/N factor is applied once,
// by the thread that writes the final value.
template <RedOp>
struct RedOpTraits;

template <>
struct RedOpTraits<RedOp::Sum> {
    static __host__ __device__ __forceinline__ float apply(float a, float b) { return a + b; }
};
template <>
struct RedOpTraits<RedOp::Avg> {
    static __host__ __device__ __forceinline__ float apply(float a, float b) { return a + b; }
};
template <>
struct RedOpTraits<RedOp::Max> {
    static __host__ __device__ __forceinline__ float apply(float a, float b) {
        return (a != a) ? a : ((b != b) ? b : (a > b ? a : b));
    }
};
template <>
struct RedOpTraits<RedOp::Min> {
    static __host__ __device__ __forceinline__ float apply(float a, float b) {
        return (a != a) ? a : ((b != b) ? b : (a < b ? a : b));
    }
};

}  // namespace b200ccl
