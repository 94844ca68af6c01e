// common.cuh — element-type traits, small device helpers and host-side error plumbing shared by the
// SAPA kernels.  Everything computes in an accumulation type (float for f32/f16/bf16, double for f64).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/sapa_b200.h"

namespace sapa {

// ---------------------------------------------------------------------------------- type traits
template <typename T> struct AccOf { using type = float; };
template <> struct AccOf<double> { using type = double; };

__device__ __forceinline__ float to_acc(float x) { return x; }
__device__ __forceinline__ float to_acc(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_acc(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ double to_acc(double x) { return x; }

template <typename T> __device__ __forceinline__ T from_acc(typename AccOf<T>::type x);
template <> __device__ __forceinline__ float from_acc<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_acc<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ double from_acc<double>(double x) { return x; }

// A pair of adjacent elements (the two high-res columns of one low-res parent when s == 2).
template <typename T> struct Pair;
template <> struct Pair<float> { using type = float2; };
template <> struct Pair<__half> { using type = __half2; };
template <> struct Pair<__nv_bfloat16> { using type = __nv_bfloat162; };

__device__ __forceinline__ float2 pair_to_float2(float2 p) { return p; }
__device__ __forceinline__ float2 pair_to_float2(__half2 p) { return __half22float2(p); }
__device__ __forceinline__ float2 pair_to_float2(__nv_bfloat162 p) { return __bfloat1622float2(p); }

template <typename T> __device__ __forceinline__ typename Pair<T>::type float2_to_pair(float a, float b);
template <> __device__ __forceinline__ float2 float2_to_pair<float>(float a, float b) { return make_float2(a, b); }
template <> __device__ __forceinline__ __half2 float2_to_pair<__half>(float a, float b) { return __floats2half2_rn(a, b); }
template <> __device__ __forceinline__ __nv_bfloat162 float2_to_pair<__nv_bfloat16>(float a, float b) {
    return __floats2bfloat162_rn(a, b);
}

// Read-only load that bypasses L1 allocation (streamed once) and a streaming store.
template <typename V> __device__ __forceinline__ V ld_stream(const V *p) { return __ldcs(p); }
template <typename V> __device__ __forceinline__ void st_stream(V *p, V v) { __stcs(p, v); }

__device__ __forceinline__ void atomic_add(float *p, float v) { atomicAdd(p, v); }
__device__ __forceinline__ void atomic_add(double *p, double v) { atomicAdd(p, v); }

// ---------------------------------------------------------------------------------- host helpers
void set_error(const char *fmt, ...);   // stores a thread-local message, see api.cu
int check_launch(const char *what);     // cudaGetLastError() -> SAPA_OK / SAPA_ERR_LAUNCH

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline size_t dtype_size(int dtype) {
    switch (dtype) {
        case SAPA_F32: return 4;
        case SAPA_F16: return 2;
        case SAPA_BF16: return 2;
        case SAPA_F64: return 8;
        default: return 0;
    }
}

inline int ceil_div(long long a, long long b) { return static_cast<int>((a + b - 1) / b); }

#define SAPA_REQUIRE(cond, code, ...)      \
    do {                                   \
        if (!(cond)) {                     \
            ::sapa::set_error(__VA_ARGS__); \
            return (code);                 \
        }                                  \
    } while (0)

#define SAPA_CHECK_PTR(fn, p)                                                                      \
    do {                                                                                           \
        SAPA_REQUIRE((p) != nullptr, SAPA_ERR_ARGUMENT, "%s: %s is NULL", fn, #p);                  \
        SAPA_REQUIRE(::sapa::aligned16(p), SAPA_ERR_ALIGNMENT, "%s: %s is not 16-byte aligned", fn, #p); \
    } while (0)

// Runs the lambda body with `scalar_t` bound to the element type named by the dtype code.
// SAPA_DISPATCH_FAST: f32 / f16 / bf16 (tiled kernels).  SAPA_DISPATCH_ALL adds f64 (generic kernels).
#define SAPA_DISPATCH_CASE_(code, type, ...) \
    case code: {                             \
        using scalar_t = type;               \
        return __VA_ARGS__();                \
    }
#define SAPA_DISPATCH_FAST(dtype, ...)                                           \
    [&]() -> int {                                                               \
        switch (dtype) {                                                         \
            SAPA_DISPATCH_CASE_(SAPA_F32, float, __VA_ARGS__)                    \
            SAPA_DISPATCH_CASE_(SAPA_F16, __half, __VA_ARGS__)                   \
            SAPA_DISPATCH_CASE_(SAPA_BF16, __nv_bfloat16, __VA_ARGS__)           \
            default:                                                             \
                ::sapa::set_error("dtype code %d has no tiled kernel", (int)(dtype)); \
                return SAPA_ERR_DTYPE;                                           \
        }                                                                        \
    }()
#define SAPA_DISPATCH_ALL(dtype, ...)                                            \
    [&]() -> int {                                                               \
        switch (dtype) {                                                         \
            SAPA_DISPATCH_CASE_(SAPA_F32, float, __VA_ARGS__)                    \
            SAPA_DISPATCH_CASE_(SAPA_F16, __half, __VA_ARGS__)                   \
            SAPA_DISPATCH_CASE_(SAPA_BF16, __nv_bfloat16, __VA_ARGS__)           \
            SAPA_DISPATCH_CASE_(SAPA_F64, double, __VA_ARGS__)                   \
            default:                                                             \
                ::sapa::set_error("unknown dtype code %d", (int)(dtype));        \
                return SAPA_ERR_DTYPE;                                           \
        }                                                                        \
    }()

}  // namespace sapa
