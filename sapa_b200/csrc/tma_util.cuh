// tma_util.cuh — PTX wrappers shared by the TMA kernels (sapa_tma.cu, sapa_gath_mma.cu): mbarriers with bounded
// waits, tensor-map tile loads / stores, warp-level MMA, and the host-side lookup of cuTensorMapEncodeTiled.
#pragma once

#include "common.cuh"

#include <cuda.h>

#include <atomic>

namespace sapa {
namespace tmau {

constexpr unsigned TF32_MASK = 0xffffe000u;
constexpr int WAIT_LIMIT = 1 << 22;        // bounded mbarrier wait (each try suspends for a while in hardware)
constexpr int SCHED_SLOTS = 256;           // scheduler counter pairs per translation unit (one per launch in flight)
constexpr int SCHED_EAGER = 192;           // pairs [0, SCHED_EAGER) serve ordinary launches, the rest launches under stream capture

__device__ __forceinline__ void mbar_init(unsigned bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity) {      // may suspend for a bounded time
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait(unsigned bar, unsigned parity) {     // never suspends
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// returns false when the limit was reached (the caller raises its error flag and leaves)
__device__ __forceinline__ bool mbar_wait_bounded(unsigned bar, unsigned parity) {
    for (int i = 0; i < WAIT_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// global -> shared tile load, completion counted on an mbarrier; coordinates outside the tensor read zeros
__device__ __forceinline__ void tma_load_4d(unsigned dst, const CUtensorMap *map, unsigned bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];\n"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
// shared -> global tile store; out-of-range parts of the box (tile overhang, channel tail) are clipped
__device__ __forceinline__ void tma_store_4d(const CUtensorMap *map, unsigned src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];\n"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
// 32-bit load from a shared-memory address (state-space address, so the compiler emits LDS with an immediate
// offset instead of a generic load with 64-bit address arithmetic)
__device__ __forceinline__ unsigned lds32(unsigned addr) {
    unsigned v;
    asm("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts64(unsigned addr, float a, float b) {
    asm volatile("st.shared.v2.f32 [%0], {%1, %2};\n" ::"r"(addr), "f"(a), "f"(b) : "memory");
}
// low term of the two-term tf32 split (the high term is the register itself: the tensor core reads its top 19 bits)
__device__ __forceinline__ unsigned tf32_lo(unsigned x) {
    return __float_as_uint(__uint_as_float(x) - __uint_as_float(x & TF32_MASK));
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// two floats rounded to a packed 16-bit pair, `a` in the low half
__device__ __forceinline__ unsigned pack_pair(__half, float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const unsigned *>(&h);
}
__device__ __forceinline__ unsigned pack_pair(__nv_bfloat16, float a, float b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const unsigned *>(&h);
}

// ---------------------------------------------------------------------------------- host side
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled is a driver entry point; it is looked up through the runtime so that the library links
// only against cudart.  nullptr when the driver does not provide it.
inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Scheduler pair for the next launch on `st`.  A launch recorded into a CUDA graph keeps its pair for every replay,
// so captured launches draw from a range of their own that the round-robin of ordinary launches never enters:
// a replay can then never share a pair with an ordinary launch in flight on another stream.  (Two replays of graphs
// that hold the same pair must not overlap on the GPU: replay one graph at a time per device, or on one stream.)
inline int next_sched_slot(std::atomic<unsigned> &eager, std::atomic<unsigned> &captured, cudaStream_t st) {
    cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &status) == cudaSuccess && status != cudaStreamCaptureStatusNone)
        return SCHED_EAGER + (int)(captured.fetch_add(1u) % (unsigned)(SCHED_SLOTS - SCHED_EAGER));
    return (int)(eager.fetch_add(1u) % (unsigned)SCHED_EAGER);
}

// CUresult of the most recent cuTensorMapEncodeTiled call on this thread (for error messages)
inline int &last_encode_result() {
    static thread_local int code = 0;
    return code;
}

// 4-D map over a dense NCHW tensor seen as (x, channel, y, image); box = box_w columns x box_ch channels x box_rows rows
inline bool make_nchw_map(CUtensorMap *map, const void *base, int width, int height, int channels, int images, int box_w,
                          int box_ch, int box_rows, CUtensorMapDataType type, int esize, CUtensorMapSwizzle swizzle,
                          CUtensorMapL2promotion promotion = CU_TENSOR_MAP_L2_PROMOTION_L2_128B) {
    EncodeTiledFn encode = encode_tiled_fn();
    if (encode == nullptr) return false;
    const cuuint64_t dims[4] = {(cuuint64_t)width, (cuuint64_t)channels, (cuuint64_t)height, (cuuint64_t)images};
    const cuuint64_t strides[3] = {(cuuint64_t)height * width * esize, (cuuint64_t)width * esize,
                                   (cuuint64_t)channels * height * width * esize};
    const cuuint32_t box[4] = {(cuuint32_t)box_w, (cuuint32_t)box_ch, (cuuint32_t)box_rows, 1u};
    const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    CUresult r = encode(map, type, 4, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle, promotion, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_ERROR_INVALID_CONTEXT) {
        // The encoder is a driver entry point and wants a current context.  A thread that has made no runtime call
        // yet (PyTorch's autograd worker running a backward is the usual case) has none bound: cudaFree(nullptr) is
        // the runtime's no-op that binds the device's primary context to the calling thread.  Then once more.
        cudaFree(nullptr);
        r = encode(map, type, 4, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                   promotion, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    last_encode_result() = (int)r;
    return r == CUDA_SUCCESS;
}

}  // namespace tmau
}  // namespace sapa
