// Shared host-side helpers for the C-ABI translation units.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tb200.h"

namespace tb200 {

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int dtype_size(int dtype) {
    switch (dtype) {
        case TB200_F32: return 4;
        case TB200_F16: return 2;
        case TB200_BF16: return 2;
        default: return 0;
    }
}

// Launch errors are returned as positive cudaError_t values.
inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? TB200_OK : static_cast<int>(e);
}

struct DeviceInfo {
    int index = 0;
    int sm_count = 0;
    int cc_major = 0;
    int cc_minor = 0;
    int max_smem_optin = 0;
    bool valid = false;
};

// Cached per device; the first call on a device queries the runtime.
const DeviceInfo& device_info();

// 8 packed 16-bit values or 4 packed fp32 <-> float registers -----------------
template <typename T>
struct Vec16;  // one 16-byte chunk

template <>
struct Vec16<float> {
    static constexpr int N = 4;
    __device__ static void unpack(const uint4& v, float (&f)[4]) {
        f[0] = __uint_as_float(v.x);
        f[1] = __uint_as_float(v.y);
        f[2] = __uint_as_float(v.z);
        f[3] = __uint_as_float(v.w);
    }
    __device__ static uint4 pack(const float (&f)[4]) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
    }
    __device__ static void unpack2(const uint4& v, float2 (&f)[2]) {
        f[0] = make_float2(__uint_as_float(v.x), __uint_as_float(v.y));
        f[1] = make_float2(__uint_as_float(v.z), __uint_as_float(v.w));
    }
    __device__ static uint4 pack2(const float2 (&f)[2]) {
        return make_uint4(__float_as_uint(f[0].x), __float_as_uint(f[0].y), __float_as_uint(f[1].x),
                          __float_as_uint(f[1].y));
    }
    // element-wise a + b, rounded to the element type
    __device__ static uint4 add_rn(const uint4& a, const uint4& b) {
        return make_uint4(__float_as_uint(__fadd_rn(__uint_as_float(a.x), __uint_as_float(b.x))),
                          __float_as_uint(__fadd_rn(__uint_as_float(a.y), __uint_as_float(b.y))),
                          __float_as_uint(__fadd_rn(__uint_as_float(a.z), __uint_as_float(b.z))),
                          __float_as_uint(__fadd_rn(__uint_as_float(a.w), __uint_as_float(b.w))));
    }
};

template <>
struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void unpack(const uint4& v, float (&f)[8]) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            // bf16 -> fp32 is a 16-bit shift
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
    __device__ static uint4 pack(const float (&f)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ static void unpack2(const uint4& v, float2 (&f)[4]) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xFFFF0000u));
    }
    __device__ static uint4 pack2(const float2 (&f)[4]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __float22bfloat162_rn(f[i]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ static uint4 add_rn(const uint4& a, const uint4& b) {
        const uint32_t x[4] = {a.x, a.y, a.z, a.w}, y[4] = {b.x, b.y, b.z, b.w};
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = __hadd2_rn(*reinterpret_cast<const __nv_bfloat162*>(&x[i]),
                                                *reinterpret_cast<const __nv_bfloat162*>(&y[i]));
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};

template <>
struct Vec16<__half> {
    static constexpr int N = 8;
    __device__ static void unpack(const uint4& v, float (&f)[8]) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
            float2 p = __half22float2(h);
            f[2 * i] = p.x;
            f[2 * i + 1] = p.y;
        }
    }
    __device__ static uint4 pack(const float (&f)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ static void unpack2(const uint4& v, float2 (&f)[4]) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    }
    __device__ static uint4 pack2(const float2 (&f)[4]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h = __float22half2_rn(f[i]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ static uint4 add_rn(const uint4& a, const uint4& b) {
        const uint32_t x[4] = {a.x, a.y, a.z, a.w}, y[4] = {b.x, b.y, b.z, b.w};
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 h = __hadd2_rn(*reinterpret_cast<const __half2*>(&x[i]), *reinterpret_cast<const __half2*>(&y[i]));
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }

}  // namespace tb200
