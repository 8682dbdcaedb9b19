// 16-byte vector <-> fp32 lane conversions and the epilogue functors that are
// fused into every collective kernel.
//
// Parity: the reference's ValueOps/SlotOps (src/kernels/type_ops.cuh:21-58,
// 142-288) add fp16/bf16 in the storage type and reduce fp32 one scalar at a
// time.  Here every dtype is moved as 16-byte vectors and accumulated in fp32 in
// rank order 0..N-1, so all ranks obtain bit-identical sums.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../comm/layout.h"
#include "../core/ptx.cuh"

namespace yali {

template <typename T>
struct TypeTraits;
template <>
struct TypeTraits<float> {
    static constexpr int kVec = 4;  // elements per 16 bytes
    static constexpr Dtype kDtype = Dtype::FP32;
};
template <>
struct TypeTraits<__half> {
    static constexpr int kVec = 8;
    static constexpr Dtype kDtype = Dtype::FP16;
};
template <>
struct TypeTraits<__nv_bfloat16> {
    static constexpr int kVec = 8;
    static constexpr Dtype kDtype = Dtype::BF16;
};

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) {
    return v;
}
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) {
    return __half2float(v);
}
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) {
    return v;
}
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) {
    return __float2half_rn(v);
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// acc[0..kVec) += lanes of the 16-byte vector v interpreted as T.
template <typename T>
__device__ __forceinline__ void accumulate(float* acc, const uint4& v);
template <>
__device__ __forceinline__ void accumulate<float>(float* acc, const uint4& v) {
    acc[0] += __uint_as_float(v.x);
    acc[1] += __uint_as_float(v.y);
    acc[2] += __uint_as_float(v.z);
    acc[3] += __uint_as_float(v.w);
}
template <>
__device__ __forceinline__ void accumulate<__half>(float* acc, const uint4& v) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __half22float2(h[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
    }
}
template <>
__device__ __forceinline__ void accumulate<__nv_bfloat16>(float* acc, const uint4& v) {
    // bf16 -> fp32 is a 16-bit shift; do it on the integer pipe.
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        acc[2 * i] += __uint_as_float(w[i] << 16);
        acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
    }
}

// Packs n = 16/sizeof(T) fp32 lanes into one 16-byte vector of T.
template <typename T>
__device__ __forceinline__ uint4 pack16(const float* f);
template <>
__device__ __forceinline__ uint4 pack16<float>(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
}
template <>
__device__ __forceinline__ uint4 pack16<__half>(const float* f) {
    uint4 r;
    __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return r;
}
template <>
__device__ __forceinline__ uint4 pack16<__nv_bfloat16>(const float* f) {
    uint4 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return r;
}

// Stores N fp32 lanes as N consecutive Tout at `p` (local or peer memory).
// N*sizeof(Tout) is 16 when input and output types have equal width, 8 for
// fp32 -> 16-bit and 32 for 16-bit -> fp32; `p` is aligned to that size.
template <typename Tout, int N>
__device__ __forceinline__ void store_lanes(Tout* p, const float* f) {
    if constexpr (N * sizeof(Tout) == 16) {
        ptx::st_v4(p, pack16<Tout>(f));
    } else if constexpr (N * sizeof(Tout) == 8) {
        static_assert(N * sizeof(Tout) != 8 || sizeof(Tout) == 2, "8-byte store packs four 16-bit values");
        Tout t[4] = {from_f32<Tout>(f[0]), from_f32<Tout>(f[1]), from_f32<Tout>(f[2]), from_f32<Tout>(f[3])};
        uint2 v = *reinterpret_cast<uint2*>(t);
        asm volatile("st.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
    } else {
        static_assert(N * sizeof(Tout) == 16 || N * sizeof(Tout) == 8 || N * sizeof(Tout) == 32, "unsupported width");
        ptx::st_v4(p, pack16<Tout>(f));
        ptx::st_v4(p + 4, pack16<Tout>(f + 4));
    }
}

// 16 bytes at p + 16*v of a buffer that is only aligned to its element type T: assembled from
// element loads / written with element stores.  The slow path of ranks whose buffers are not
// 16-byte aligned; their peers never notice, because the data on the wire is laid out the same.
template <typename T>
__device__ __forceinline__ uint4 load16_elems(const void* base, uint64_t v) {
    constexpr int VEC = 16 / sizeof(T);
    const T* p = static_cast<const T*>(base) + v * VEC;
    uint4 r;
    T* o = reinterpret_cast<T*>(&r);
#pragma unroll
    for (int i = 0; i < VEC; ++i) o[i] = p[i];
    return r;
}
template <typename T>
__device__ __forceinline__ void store16_elems(void* base, uint64_t v, const uint4& x) {
    constexpr int VEC = 16 / sizeof(T);
    T* p = static_cast<T*>(base) + v * VEC;
    const T* i_ = reinterpret_cast<const T*>(&x);
#pragma unroll
    for (int i = 0; i < VEC; ++i) p[i] = i_[i];
}

// ---- epilogue functors: applied to the fp32 sum before it is stored ----
struct EpiIdentity {
    static constexpr int kKind = kEpiIdentity;
    __device__ __forceinline__ explicit EpiIdentity(const EpilogueParams&) {}
    __device__ __forceinline__ float operator()(float x) const { return x; }
};
struct EpiScale {
    static constexpr int kKind = kEpiScaleCast;
    float s;
    __device__ __forceinline__ explicit EpiScale(const EpilogueParams& p) : s(p.scale) {}
    __device__ __forceinline__ float operator()(float x) const { return x * s; }
};

}  // namespace yali
