// Packs: the unit a thread moves per access. Wide = 16 bytes (4 floats or 8 halves/bf16),
// Narrow = one element (fallback for odd counts and unaligned buffers). Every pack is widened
// to fp32 before it is combined and rounded once when it is written.
//
// Parity: nano-nccl's vector/scalar workers (src/kernels/ring_simple_kernel.cuh:58-92 16-byte
// volatile loads, 166-219 reduce in native 16-bit, 335-364 scalar fallback). Here 16-bit
// inputs accumulate in fp32, and max/min return NaN if any input is NaN for every dtype.
#pragma once

#include "b200ccl/types.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace b200ccl::dev {

// ---- reduction operators on fp32 -------------------------------------------------------
struct OpAdd {
    static __device__ __forceinline__ float apply(float a, float b) { return a + b; }
};
struct OpMax {
    static __device__ __forceinline__ float apply(float a, float b) {
        float r;
        asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
        return r;
    }
};
struct OpMin {
    static __device__ __forceinline__ float apply(float a, float b) {
        float r;
        asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
        return r;
    }
};

// ---- raw 16-byte accesses --------------------------------------------------------------
// Data that a peer wrote during this kernel is read after an acquire; it is streamed once, so
// it is kept out of L1.
__device__ __forceinline__ uint4 ld16_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}
__device__ __forceinline__ void st16(uint4* p, uint4 v) {
    asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// ---- element conversion ----------------------------------------------------------------
template <typename T>
struct Elem;
template <>
struct Elem<float> {
    static __device__ __forceinline__ float to_f(float v) { return v; }
    static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <>
struct Elem<__half> {
    static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <>
struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// ---- Wide pack: 16 bytes ----------------------------------------------------------------
template <typename T>
struct Wide {
    static constexpr int kElems = 16 / sizeof(T);
    static constexpr int kBytes = 16;
    using Raw = uint4;
    static __device__ __forceinline__ Raw load(const void* base, unsigned long long i) {
        return ld16_stream(static_cast<const uint4*>(base) + i);
    }
    static __device__ __forceinline__ void store(void* base, unsigned long long i, Raw v) {
        st16(static_cast<uint4*>(base) + i, v);
    }
    static __device__ __forceinline__ Raw load_user(const void* base, unsigned long long i) { return load(base, i); }
    static __device__ __forceinline__ void store_user(void* base, unsigned long long i, Raw v) { store(base, i, v); }
    static __device__ __forceinline__ void unpack(const Raw& r, float (&f)[kElems]);
    static __device__ __forceinline__ Raw pack(const float (&f)[kElems]);
};

template <>
__device__ __forceinline__ void Wide<float>::unpack(const uint4& r, float (&f)[4]) {
    f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y);
    f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
}
template <>
__device__ __forceinline__ uint4 Wide<float>::pack(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
}

__device__ __forceinline__ float2 h2_to_f2(unsigned int w) {
    __half2 h = *reinterpret_cast<__half2*>(&w);
    return __half22float2(h);
}
__device__ __forceinline__ unsigned int f2_to_h2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<unsigned int*>(&h);
}
__device__ __forceinline__ float2 b2_to_f2(unsigned int w) {
    // bf16 → fp32 is a 16-bit shift; keeps NaN payloads and needs no conversion unit
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
__device__ __forceinline__ unsigned int f2_to_b2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<unsigned int*>(&h);
}

template <>
__device__ __forceinline__ void Wide<__half>::unpack(const uint4& r, float (&f)[8]) {
    float2 a = h2_to_f2(r.x), b = h2_to_f2(r.y), c = h2_to_f2(r.z), d = h2_to_f2(r.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
template <>
__device__ __forceinline__ uint4 Wide<__half>::pack(const float (&f)[8]) {
    return make_uint4(f2_to_h2(f[0], f[1]), f2_to_h2(f[2], f[3]), f2_to_h2(f[4], f[5]), f2_to_h2(f[6], f[7]));
}
template <>
__device__ __forceinline__ void Wide<__nv_bfloat16>::unpack(const uint4& r, float (&f)[8]) {
    float2 a = b2_to_f2(r.x), b = b2_to_f2(r.y), c = b2_to_f2(r.z), d = b2_to_f2(r.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
template <>
__device__ __forceinline__ uint4 Wide<__nv_bfloat16>::pack(const float (&f)[8]) {
    return make_uint4(f2_to_b2(f[0], f[1]), f2_to_b2(f[2], f[3]), f2_to_b2(f[4], f[5]), f2_to_b2(f[6], f[7]));
}

// ---- Wide32 pack: 32 bytes, one 256-bit access (sm_100) on the peer-visible side ----------------
struct Raw32 {
    uint4 lo, hi;
};
__device__ __forceinline__ Raw32 ld32_stream(const void* p) {
    Raw32 v;
    asm volatile("ld.global.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v.lo.x), "=r"(v.lo.y), "=r"(v.lo.z), "=r"(v.lo.w), "=r"(v.hi.x), "=r"(v.hi.y), "=r"(v.hi.z), "=r"(v.hi.w)
                 : "l"(p)
                 : "memory");
    return v;
}
__device__ __forceinline__ void st32(void* p, const Raw32& v) {
    asm volatile("st.global.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v.lo.x), "r"(v.lo.y), "r"(v.lo.z),
                 "r"(v.lo.w), "r"(v.hi.x), "r"(v.hi.y), "r"(v.hi.z), "r"(v.hi.w)
                 : "memory");
}

template <typename T>
struct Wide32 {
    static constexpr int kElems = 32 / sizeof(T);
    static constexpr int kBytes = 32;
    using Raw = Raw32;
    // Peer-visible buffers (32-byte aligned by contract): one 256-bit access.
    static __device__ __forceinline__ Raw load(const void* base, unsigned long long i) {
        return ld32_stream(static_cast<const char*>(base) + i * 32ull);
    }
    static __device__ __forceinline__ void store(void* base, unsigned long long i, const Raw& v) {
        st32(static_cast<char*>(base) + i * 32ull, v);
    }
    // The caller's own buffers in the staging copies need only 16-byte alignment: two 128-bit accesses.
    static __device__ __forceinline__ Raw load_user(const void* base, unsigned long long i) {
        const uint4* q = static_cast<const uint4*>(base) + 2ull * i;
        Raw v;
        v.lo = ld16_stream(q);
        v.hi = ld16_stream(q + 1);
        return v;
    }
    static __device__ __forceinline__ void store_user(void* base, unsigned long long i, const Raw& v) {
        uint4* q = static_cast<uint4*>(base) + 2ull * i;
        st16(q, v.lo);
        st16(q + 1, v.hi);
    }
    static __device__ __forceinline__ void unpack(const Raw& r, float (&f)[kElems]) {
        constexpr int h = kElems / 2;
        float a[h], b[h];
        Wide<T>::unpack(r.lo, a);
        Wide<T>::unpack(r.hi, b);
#pragma unroll
        for (int e = 0; e < h; ++e) {
            f[e] = a[e];
            f[h + e] = b[e];
        }
    }
    static __device__ __forceinline__ Raw pack(const float (&f)[kElems]) {
        constexpr int h = kElems / 2;
        float a[h], b[h];
#pragma unroll
        for (int e = 0; e < h; ++e) {
            a[e] = f[e];
            b[e] = f[h + e];
        }
        Raw v;
        v.lo = Wide<T>::pack(a);
        v.hi = Wide<T>::pack(b);
        return v;
    }
};

// ---- Narrow pack: one element -------------------------------------------------------------
template <typename T>
struct Narrow {
    static constexpr int kElems = 1;
    static constexpr int kBytes = sizeof(T);
    using Raw = T;
    static __device__ __forceinline__ Raw load(const void* base, unsigned long long i) {
        return *(static_cast<const volatile T*>(base) + i);
    }
    static __device__ __forceinline__ void store(void* base, unsigned long long i, Raw v) {
        static_cast<T*>(base)[i] = v;
    }
    static __device__ __forceinline__ Raw load_user(const void* base, unsigned long long i) { return load(base, i); }
    static __device__ __forceinline__ void store_user(void* base, unsigned long long i, Raw v) { store(base, i, v); }
    static __device__ __forceinline__ void unpack(const Raw& r, float (&f)[1]) { f[0] = Elem<T>::to_f(r); }
    static __device__ __forceinline__ Raw pack(const float (&f)[1]) { return Elem<T>::from_f(f[0]); }
};
template <>
__device__ __forceinline__ __half Narrow<__half>::load(const void* base, unsigned long long i) {
    unsigned short v = *(static_cast<const volatile unsigned short*>(base) + i);
    return __ushort_as_half(v);
}
template <>
__device__ __forceinline__ __nv_bfloat16 Narrow<__nv_bfloat16>::load(const void* base, unsigned long long i) {
    unsigned short v = *(static_cast<const volatile unsigned short*>(base) + i);
    return __ushort_as_bfloat16(v);
}

// ---- NVSwitch multicast accesses (sum only; the switch accumulates 16-bit inputs in fp32) ----
template <typename T>
__device__ __forceinline__ uint4 multimem_ld_reduce_add(const uint4* mc);
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce_add<float>(const uint4* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
}
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce_add<__half>(const uint4* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
}
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce_add<__nv_bfloat16>(const uint4* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
}
__device__ __forceinline__ void multimem_st16(uint4* mc, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w)
                 : "memory");
}

}  // namespace b200ccl::dev
