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

// Streaming (evict-first) load / store of two adjacent elements (the two high-res columns of one low-res
// parent when s == 2) as one 64-bit or 32-bit access.  The 16-bit types go through `unsigned int` builtins:
// the toolkit's own __stcs overloads for __half2 / __nv_bfloat162 are inline asm with a "memory" clobber,
// which pins every shared-memory load behind the previous store and serialises the aggregation loop.
template <typename T> __device__ __forceinline__ float2 load_pair(const T *p);
template <> __device__ __forceinline__ float2 load_pair<float>(const float *p) {
    return __ldcs(reinterpret_cast<const float2 *>(p));
}
template <> __device__ __forceinline__ float2 load_pair<__half>(const __half *p) {
    const unsigned int raw = __ldcs(reinterpret_cast<const unsigned int *>(p));
    return __half22float2(*reinterpret_cast<const __half2 *>(&raw));
}
template <> __device__ __forceinline__ float2 load_pair<__nv_bfloat16>(const __nv_bfloat16 *p) {
    const unsigned int raw = __ldcs(reinterpret_cast<const unsigned int *>(p));
    return make_float2(__uint_as_float(raw << 16), __uint_as_float(raw & 0xffff0000u));
}

template <typename T> __device__ __forceinline__ void store_pair(T *p, float a, float b);
template <> __device__ __forceinline__ void store_pair<float>(float *p, float a, float b) {
    __stcs(reinterpret_cast<float2 *>(p), make_float2(a, b));
}
template <> __device__ __forceinline__ void store_pair<__half>(__half *p, float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    __stcs(reinterpret_cast<unsigned int *>(p), *reinterpret_cast<const unsigned int *>(&h));
}
template <> __device__ __forceinline__ void store_pair<__nv_bfloat16>(__nv_bfloat16 *p, float a, float b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    __stcs(reinterpret_cast<unsigned int *>(p), *reinterpret_cast<const unsigned int *>(&h));
}

__device__ __forceinline__ void atomic_add(float *p, float v) { atomicAdd(p, v); }
__device__ __forceinline__ void atomic_add(double *p, double v) { atomicAdd(p, v); }

// ---------------------------------------------------------------------------------- host helpers
void set_error(const char *fmt, ...);   // stores a thread-local message, see api.cu
int check_launch(const char *what);     // cudaGetLastError() -> SAPA_OK (and records `what`) / SAPA_ERR_LAUNCH
void trace_reset();                     // start of an entry point: forget the kernels of the previous call
void trace_kernel(const char *name);    // appended by check_launch: read back through sapa_last_kernels()

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

// every tensor pointer must be non-null and aligned to its element size; 16-byte alignment is only needed by the
// vectorised / tiled / tensor-map kernels and is checked where those are chosen (all_aligned16)
// (uses the entry point's `dtype` argument)
#define SAPA_CHECK_PTR(fn, p)                                                                                  \
    do {                                                                                                       \
        SAPA_REQUIRE((p) != nullptr, SAPA_ERR_ARGUMENT, "%s: %s is NULL", fn, #p);                              \
        SAPA_REQUIRE(::sapa::dtype_size(dtype) != 0 && reinterpret_cast<uintptr_t>(p) % ::sapa::dtype_size(dtype) == 0, \
                     SAPA_ERR_ALIGNMENT, "%s: %s is not aligned to the element size", fn, #p);                  \
    } while (0)

template <typename... P> inline bool all_aligned16(const P *...p) { return (aligned16(p) && ...); }

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
