// shared by the kernels of libb200mixers.so: type conversion, warp reductions, dtype dispatch
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include "b200_mixers.h"

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
// log(sigmoid(z)) without cancellation on either side
__device__ __forceinline__ float log_sigmoid_f(float z) { return z >= 0.0f ? -log1pf(expf(-z)) : z - log1pf(expf(z)); }

// q (32-bit, e.g. staged in shared memory) . one row of keys; 16-byte loads when the rows allow them
template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ qs, const T* __restrict__ kr, int dim) {
    float s = 0.0f;
    if constexpr (sizeof(T) == 2) {
        if ((dim & 7) == 0) {                                // rows start on 16-byte boundaries: eight elements a load
            const uint4* k4 = reinterpret_cast<const uint4*>(kr);
            const float4* q4 = reinterpret_cast<const float4*>(qs);
            float s0 = 0.0f, s1 = 0.0f;
            for (int d = 0; d < dim; d += 8) {
                uint4 v = k4[d >> 3];
                const T* e = reinterpret_cast<const T*>(&v);
                float4 qa = q4[d >> 2], qb = q4[(d >> 2) + 1];
                s0 += qa.x * to_f(e[0]) + qa.y * to_f(e[1]) + qa.z * to_f(e[2]) + qa.w * to_f(e[3]);
                s1 += qb.x * to_f(e[4]) + qb.y * to_f(e[5]) + qb.z * to_f(e[6]) + qb.w * to_f(e[7]);
            }
            return s0 + s1;
        }
    }
    for (int d = 0; d < dim; ++d) s += qs[d] * to_f(kr[d]);
    return s;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
    return v;
}

// the oldest storage index that a query at storage index c may see.  window > 0: itself and the window - 1 positions before it;
// chunk > 0: only positions of its own chunk, chunks of `chunk` positions counted from the row's first token (storage index
// first_real, which is negative once the row's first positions have left the storage); never anything before first_real.
// Non-decreasing in c, so the first row of a tile bounds the tile.
__device__ __forceinline__ int visible_from(int c, int first_real, int window, int chunk) {
    int lo = window > 0 ? c - window + 1 : 0;
    if (chunk > 0 && c >= first_real) {
        const int start = first_real + (c - first_real) / chunk * chunk;
        if (start > lo) lo = start;
    }
    if (lo < first_real) lo = first_real;
    return lo < 0 ? 0 : lo;
}

#define MIXERS_DISPATCH(dtype, ...)                                                              \
    do {                                                                                         \
        if ((dtype) == 0) { using T = float; __VA_ARGS__; }                                      \
        else if ((dtype) == 1) { using T = __nv_bfloat16; __VA_ARGS__; }                         \
        else if ((dtype) == 2) { using T = __half; __VA_ARGS__; }                                \
        else return (int)cudaErrorInvalidValue;                                                  \
    } while (0)

static inline int mixers_status() { return (int)cudaGetLastError(); }
