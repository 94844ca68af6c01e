// sapa_proj.cu — the step in front of the attention: GroupNorm followed by the 1x1 query / key projection
// (reference: sapa_base.py:27-34, sapa_deform.py:35-42), as ONE dense GEMM per image on the 5th-generation tensor cores.
//
// GroupNorm is affine per (image, channel) once the group statistics are known, so it folds into the projection:
//   out[b, j, p] = sum_c W[j, c] * (gamma_c * rstd_bg * (x[b, c, p] - mean_bg) + beta_c) + bias_j
//                = sum_c W'[b, j, c] * x[b, c, p] + bias'[b, j]
//   W'[b, j, c]  = W[j, c] * gamma_c * rstd_bg(c),      bias'[b, j] = bias_j + sum_c W[j, c] * (beta_c - mean_bg(c) * gamma_c * rstd_bg(c))
// Three launches: (1) partial sums of x and x^2 per (image, group) - one pass over x at memory speed, float64 partials;
// (2) the fold above (tiny); (3) a persistent GEMM kernel that reads x exactly once more and writes out.  The normalised
// activation tensor of the unfused sequence (one write + one read of the size of x) never exists.
//
// GEMM kernel (tcgen05 / TMEM; one CTA per SM, 128-pixel tiles):
//   D[128 px x d] (+)= A[128 px x k] * B[k x d],  A = x^T, B = W' (K-major: channels contiguous)
//   * warp 4 (one lane): TMA producer of the activations, warp 6 (one lane): TMA producer of the W' blocks.  A stage =
//     128 px x (128 B / esize) channels of x as boxes of one 128-byte pixel row per channel (128-byte swizzle) plus the
//     matching d x 128 B block of W' (canonical K-major layout).
//   * 16-bit types: the landed boxes ARE the canonical operand layout for an operand whose M dimension is the contiguous
//     one ("MN-major"), and the tensor core reads them in place.
//   * float32, warps 7-14: 3xTF32 split AND transposition.  The tensor core reads tf32 (the upper 19 bits); the product
//     is evaluated as hi*hi + lo*hi + hi*lo with hi = x & 0xffffe000, lo = x - hi (exact): float32 accuracy (1e-6).  The
//     warps read a landed ring slot (lane = channel, 16 bytes = 4 pixels) and write hi and lo into an operand slot as
//     K-major rows (row = pixel, 128 bytes = the stage's 32 channels, 128-byte swizzle): both sides are free of bank
//     conflicts and the ring slot is released at once.  (The landed boxes can also be fed as an MN-major tf32 operand:
//     that needs the 128-byte swizzle of 32-byte chunks - CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, descriptor layout type 1,
//     4-row atoms; with the ordinary swizzle the product is wrong.  That form is as accurate and no faster.)  W' arrives
//     already split.
//   * warp 5 (one lane): issues tcgen05.mma (M = 128, N = d, K = 32 bytes) into one of two TMEM accumulators, frees a
//     stage with tcgen05.commit, signals the epilogue with another commit.  Its own instruction latency is on the
//     critical path (one thread): ring positions and descriptors advance by additions only, and for float32 with
//     d <= 128 the terms x_hi * W'_hi and x_hi * W'_lo are ONE instruction of N = 2d (the two W' blocks are adjacent
//     rows of the operand; the epilogue adds the two halves of the accumulator): 8 instead of 12 MMAs per stage.
//   * warps 0-3: epilogue.  tcgen05.ld (lane = pixel, column = output channel), add bias', store: for a fixed output
//     channel the 32 lanes of a warp write 32 consecutive pixels.  Runs under the MMAs of the next tile.
// Tiles walk the images from the last to the first: the statistics pass has just read them in ascending order, so the
// tail of x is what the L2 still holds.
// Every mbarrier wait is bounded; a wait that gives up raises g_wait_timeout and the CTA drains and frees its TMEM.
#include "tma_util.cuh"

#include <algorithm>
#include <cstdint>
#include <type_traits>

namespace sapa {
namespace proj {

using namespace tmau;

constexpr int TILE_PX = 128;
constexpr int EPI_WARPS = 4, TMA_WARP = 4, MMA_WARP = 5, W_WARP = 6, SPLIT_WARP0 = 7, SPLIT_WARPS = 8;
constexpr int THREADS = (SPLIT_WARP0 + SPLIT_WARPS) * 32;
constexpr int Y_STAGE = 16384;           // bytes of activations per stage: 128 px x (128 B / esize) channels
constexpr int MAX_SLOTS = 8;              // slots per ring
constexpr int OP_SLOTS_F32 = 2, OP_SLOTS_16 = 4;     // operand ring depth (the kernel is not sensitive to it)
constexpr int SMEM_LIMIT = 227 * 1024;
constexpr int STAT_THREADS = 256, MAX_SPLIT = 64, MAX_GROUPS = 256;

__device__ int g_wait_timeout = 0;

struct Args {
    CUtensorMap x_map;              // (pixel, channel, 1, image), box = one 128-byte pixel row x (128 B / esize) channels
    CUtensorMap whi_map, wlo_map;   // (channel, output channel, 1, image), box = 128 bytes of channels x d rows
    const float *bias;              // folded bias [images or 1][d]
    void *out;                      // [B][d][HW]
    int B, C, HW, d, w_per_image, tiles_per_image, total_tiles, kblocks, nx, no, tmem_cols;
    int wide;                       // float32: hi*hi and hi*lo in ONE instruction of N = 2d (W' hi and lo blocks are adjacent rows)
};

// ---------------------------------------------------------------------------------- tcgen05 wrappers
__device__ __forceinline__ void tc_alloc(unsigned smem_slot, unsigned ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_slot), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc(unsigned taddr, unsigned ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// the mbarrier receives one arrival when every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void tc_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
// One tcgen05.mma.  The 64-bit shared-memory descriptors are passed as their low words (start address and leading
// offset; the part that changes from instruction to instruction) plus the high word all operands of this kernel share:
// the issuing thread is a single thread whose own instruction latency bounds the MMA rate, so it must spend only a
// handful of instructions per MMA.
template <bool TF32>
__device__ __forceinline__ void tc_mma(unsigned d_tmem, unsigned a_lo, unsigned b_lo, unsigned desc_hi, unsigned idesc, unsigned accumulate) {
    if (TF32)
        asm volatile("{\n .reg .pred p;\n .reg .b64 da, db;\n setp.ne.b32 p, %5, 0;\n mov.b64 da, {%1, %3};\n mov.b64 db, {%2, %3};\n"
                     " tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %4, p;\n}\n"
                     ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate) : "memory");
    else
        asm volatile("{\n .reg .pred p;\n .reg .b64 da, db;\n setp.ne.b32 p, %5, 0;\n mov.b64 da, {%1, %3};\n mov.b64 db, {%2, %3};\n"
                     " tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n}\n"
                     ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate) : "memory");
}
// 16 consecutive accumulator columns of this thread's lane
__device__ __forceinline__ void tc_ld16(unsigned taddr, unsigned (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// Shared-memory matrix descriptor (64 bits).  Low word: start address (bits 0-13) and leading byte offset (bits 16-29),
// both in 16-byte units.  High word: stride byte offset in 16-byte units (bits 0-13 = descriptor bits 32-45), descriptor
// version 1 (bit 14 = bit 46), layout type 2 = 128-byte swizzle of 16-byte chunks (bits 29-31 = bits 61-63; 8-row atoms
// of 1 KB, aligned to 1 KB).  Every operand of this kernel has a stride of 1 KB between its 8-row atoms, so they all
// share one high word.  (Layout type 1, the 128-byte swizzle of 32-byte chunks with 4-row atoms, is what a tf32 operand
// needs when its M / N dimension is the contiguous one; it is not used any more, see the header.)
constexpr unsigned DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ unsigned desc_lo(unsigned addr, unsigned leading_bytes) {
    return ((addr & 0x3ffffu) >> 4) | ((leading_bytes >> 4) << 16);
}

template <typename T> struct UmmaFormat;
template <> struct UmmaFormat<float> { static constexpr unsigned code = 2; };            // tf32
template <> struct UmmaFormat<__half> { static constexpr unsigned code = 0; };
template <> struct UmmaFormat<__nv_bfloat16> { static constexpr unsigned code = 1; };

__device__ __forceinline__ void store_out(float *p, float v) { __stcs(p, v); }
__device__ __forceinline__ void store_out(__half *p, float v) { *p = __float2half_rn(v); }
__device__ __forceinline__ void store_out(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

// ---------------------------------------------------------------------------------- the GEMM kernel
// Shared memory: an activation ring (NX slots of 16 KB, filled by TMA) and an operand ring (NO slots).  16-bit types:
// the tensor core reads the activations straight from their ring slot and an operand slot holds only the W' block.
// float32: an operand slot holds the split activations (hi, lo) and the W' blocks (hi, lo); the split warps move a
// landed slot into it and hand the ring slot back at once, so the loads in flight do not wait for the MMAs.
template <typename T>
__global__ void __launch_bounds__(THREADS, 1) sapa_proj_umma_kernel(const __grid_constant__ Args a) {
    constexpr bool F32 = sizeof(T) == 4;
    constexpr int KCH = 128 / (int)sizeof(T);        // channels per stage = one 128-byte row of the weight block
    constexpr int PXG = 128 / (int)sizeof(T);        // pixels per activation box = one 128-byte row
    constexpr int NBOX = TILE_PX / PXG;
    constexpr int KSTEPS = 4;                        // one tcgen05.mma covers 32 bytes of channels: 8 (tf32) or 16 (16-bit)
    constexpr unsigned A_BOX = KCH * 128;            // bytes of one activation box = distance between 128-byte pixel groups
    constexpr unsigned A_KSTEP = A_BOX / KSTEPS;     // KCH / 4 channels further down the box
    // activation operand: 16-bit types are read where TMA put them (pixels contiguous, 8-channel atoms, 128-byte swizzle);
    // float32 is rewritten by the split warps as K-major rows (one pixel = 128 bytes of channels, 8-pixel atoms)

    extern __shared__ unsigned char smem_dyn[];
    const unsigned xring = ((unsigned)__cvta_generic_to_shared(smem_dyn) + 1023u) & ~1023u;
    const int d = a.d;
    const unsigned nx = (unsigned)a.nx, no = (unsigned)a.no;
    const unsigned w_bytes = (unsigned)d * 128u;
    const unsigned w_ofs = F32 ? 2u * Y_STAGE : 0u;                       // W' blocks inside an operand slot
    const unsigned op_bytes = w_ofs + (F32 ? 2u : 1u) * w_bytes;
    const unsigned opring = xring + nx * (unsigned)Y_STAGE;
    const unsigned bars = opring + no * op_bytes;
    const unsigned xfull0 = bars, xempty0 = bars + 8 * MAX_SLOTS, ready0 = bars + 16 * MAX_SLOTS, wfull0 = bars + 24 * MAX_SLOTS;
    const unsigned oempty0 = bars + 32 * MAX_SLOTS, tfull0 = bars + 40 * MAX_SLOTS, tempty0 = tfull0 + 16, tmem_slot = tempty0 + 16;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (unsigned i = 0; i < nx; ++i) {
            mbar_init(xfull0 + 8 * i, 1);
            mbar_init(xempty0 + 8 * i, F32 ? SPLIT_WARPS * 32 : 1);
        }
        for (unsigned i = 0; i < no; ++i) {
            mbar_init(ready0 + 8 * i, SPLIT_WARPS * 32);
            mbar_init(wfull0 + 8 * i, 1);
            mbar_init(oempty0 + 8 * i, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(tfull0 + 8 * i, 1);
            mbar_init(tempty0 + 8 * i, EPI_WARPS * 32);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == MMA_WARP) {            // the whole warp allocates the accumulator columns
        tc_alloc(tmem_slot, (unsigned)a.tmem_cols);
        tc_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    unsigned tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");

    const int tpi = a.tiles_per_image, kblocks = a.kblocks;
    const unsigned acc_cols = (unsigned)(a.wide ? 2 * d : d);       // accumulator columns per tile
    bool ok = true;

    if (warp == TMA_WARP) {            // activations: global -> ring
        if (lane == 0) {
            unsigned it = 0;
            for (int tile = blockIdx.x; tile < a.total_tiles && ok; tile += gridDim.x) {
                const int bi = tile / tpi, b = a.B - 1 - bi, px0 = (tile - bi * tpi) * TILE_PX;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const unsigned r = it % nx, rph = (it / nx) & 1u;
                    if (!mbar_wait_bounded(xempty0 + 8 * r, rph ^ 1u)) { ok = false; break; }
                    const unsigned slot = xring + r * (unsigned)Y_STAGE, full = xfull0 + 8 * r;
                    mbar_expect_tx(full, Y_STAGE);
#pragma unroll
                    for (int j = 0; j < NBOX; ++j) tma_load_4d(slot + j * A_BOX, &a.x_map, full, px0 + j * PXG, kb * KCH, 0, b);
                }
            }
        }
    } else if (warp == W_WARP) {       // W' blocks: global (L2 resident) -> operand ring
        if (lane == 0) {
            unsigned it = 0;
            for (int tile = blockIdx.x; tile < a.total_tiles && ok; tile += gridDim.x) {
                const int bi = tile / tpi, b = a.B - 1 - bi, wb = a.w_per_image ? b : 0;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const unsigned o = it % no, oph = (it / no) & 1u;
                    if (!mbar_wait_bounded(oempty0 + 8 * o, oph ^ 1u)) { ok = false; break; }
                    const unsigned slot = opring + o * op_bytes + w_ofs, full = wfull0 + 8 * o;
                    mbar_expect_tx(full, (int)((F32 ? 2u : 1u) * w_bytes));
                    tma_load_4d(slot, &a.whi_map, full, kb * KCH, 0, 0, wb);
                    if (F32) tma_load_4d(slot + w_bytes, &a.wlo_map, full, kb * KCH, 0, 0, wb);
                }
            }
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            const unsigned idesc = (1u << 4) | (UmmaFormat<T>::code << 7) | (UmmaFormat<T>::code << 10) | (F32 ? 0u : (1u << 15)) |
                                   ((unsigned)(d >> 3) << 17) | ((unsigned)(TILE_PX >> 4) << 24);
            const unsigned idesc_wide = (idesc & ~(0x3fu << 17)) | ((unsigned)(2 * d >> 3) << 17);      // the same with N = 2d
            // low descriptor words per ring slot are base + slot * pitch; a K step adds a constant (all in 16-byte units)
            const unsigned a_base = F32 ? desc_lo(opring, 16) : desc_lo(xring, A_BOX);
            const unsigned a_pitch = (F32 ? op_bytes : (unsigned)Y_STAGE) >> 4, a_kstep = (F32 ? 32u : A_KSTEP) >> 4;
            const unsigned b_base = desc_lo(opring + w_ofs, 16), b_pitch = op_bytes >> 4;
            unsigned r = 0, rph = 0, o = 0, oph = 0, ti = 0;
            for (int tile = blockIdx.x; tile < a.total_tiles && ok; tile += gridDim.x, ++ti) {
                const unsigned buf = ti & 1u, tph = (ti >> 1) & 1u;
                if (!mbar_wait_bounded(tempty0 + 8 * buf, tph ^ 1u)) { ok = false; break; }
                tc_fence_after();
                const unsigned d_tmem = tmem_base + buf * acc_cols;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait_bounded((F32 ? ready0 + 8 * o : xfull0 + 8 * r), F32 ? oph : rph) ||
                        !mbar_wait_bounded(wfull0 + 8 * o, oph)) { ok = false; break; }
                    tc_fence_after();
                    const unsigned a0 = a_base + (F32 ? o : r) * a_pitch, b0 = b_base + o * b_pitch;
#pragma unroll
                    for (int ks = 0; ks < KSTEPS; ++ks) {
                        const unsigned first = (ks != 0 || kb != 0) ? 1u : 0u;
                        if (F32 && a.wide) {
                            // x_hi * [W'_hi ; W'_lo] as one instruction of N = 2d (columns [0, d) and [d, 2d) of the
                            // accumulator, added by the epilogue), then x_lo * W'_hi into the first half
                            tc_mma<F32>(d_tmem, a0 + ks * a_kstep, b0 + ks * 2u, DESC_HI, idesc_wide, first);
                            tc_mma<F32>(d_tmem, a0 + (Y_STAGE >> 4) + ks * a_kstep, b0 + ks * 2u, DESC_HI, idesc, 1u);
                        } else {
                            tc_mma<F32>(d_tmem, a0 + ks * a_kstep, b0 + ks * 2u, DESC_HI, idesc, first);
                            if (F32) {
                                tc_mma<F32>(d_tmem, a0 + (Y_STAGE >> 4) + ks * a_kstep, b0 + ks * 2u, DESC_HI, idesc, 1u);      // lo * hi
                                tc_mma<F32>(d_tmem, a0 + ks * a_kstep, b0 + (w_bytes >> 4) + ks * 2u, DESC_HI, idesc, 1u);      // hi * lo
                            }
                        }
                    }
                    if (!F32) tc_commit(xempty0 + 8 * r);   // the activation slot is free once these MMAs have read it
                    tc_commit(oempty0 + 8 * o);             // and so is the operand slot
                    if (++r == nx) { r = 0; rph ^= 1u; }
                    if (++o == no) { o = 0; oph ^= 1u; }
                }
                if (ok) tc_commit(tfull0 + 8 * buf);        // the accumulator is complete once all MMAs so far are done
            }
        }
    } else if (warp >= SPLIT_WARP0) {
        if (F32) {
            const int st = tid - SPLIT_WARP0 * 32;
            unsigned it = 0;
            for (int tile = blockIdx.x; tile < a.total_tiles && ok; tile += gridDim.x) {
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const unsigned r = it % nx, rph = (it / nx) & 1u, o = it % no, oph = (it / no) & 1u;
                    if (!mbar_wait_bounded(xfull0 + 8 * r, rph) || !mbar_wait_bounded(oempty0 + 8 * o, oph ^ 1u)) { ok = false; break; }
                    const unsigned src = xring + r * (unsigned)Y_STAGE, dst = opring + o * op_bytes;
                    // item = (pixel group j, channel c = lane, 16-byte chunk q = 4 pixels): two warps per pixel group
                    const int sw = st >> 5, c = st & 31, j = sw >> 1;
                    unsigned v[4][4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {            // all four loads in flight before the first store
                        const int q = (sw & 1) * 4 + i;
                        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v[i][0]), "=r"(v[i][1]), "=r"(v[i][2]), "=r"(v[i][3])
                                     : "r"(src + (unsigned)j * A_BOX + (unsigned)c * 128u + (unsigned)((q ^ (c & 7)) << 4)) : "memory");
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int q = (sw & 1) * 4 + i;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int p = 32 * j + 4 * q + e;            // pixel = operand row
                            const unsigned at = dst + (unsigned)p * 128u + (unsigned)((((c >> 2) ^ (p & 7)) << 4) | ((c & 3) << 2));
                            asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(at), "r"(v[i][e] & TF32_MASK) : "memory");
                            asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(at + Y_STAGE), "r"(tf32_lo(v[i][e])) : "memory");
                        }
                    }
                    mbar_arrive(xempty0 + 8 * r);                                    // the ring slot can be refilled
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic writes -> tensor-core reads
                    mbar_arrive(ready0 + 8 * o);
                }
            }
        }
    } else {        // epilogue warps: warp w owns accumulator lanes 32w .. 32w+31 = pixels px0 + 32w + lane
        unsigned ti = 0;
        T *out = static_cast<T *>(a.out);
        for (int tile = blockIdx.x; tile < a.total_tiles && ok; tile += gridDim.x, ++ti) {
            const unsigned buf = ti & 1u, tph = (ti >> 1) & 1u;
            const int bi = tile / tpi, b = a.B - 1 - bi, px = (tile - bi * tpi) * TILE_PX + warp * 32 + lane, wb = a.w_per_image ? b : 0;
            if (!mbar_wait_bounded(tfull0 + 8 * buf, tph)) { ok = false; break; }
            tc_fence_after();
            const unsigned taddr = tmem_base + ((unsigned)(warp * 32) << 16) + buf * acc_cols;
            const float *bias = a.bias + (size_t)wb * d;
            T *op = out + (size_t)b * d * a.HW + px;
            for (int c0 = 0; c0 < d; c0 += 16) {
                unsigned r[16];
                tc_ld16(taddr + (unsigned)c0, r);
                tc_wait_ld();
                if (a.wide) {                           // second half of the accumulator: the x_hi * W'_lo term
                    unsigned r2[16];
                    tc_ld16(taddr + (unsigned)(d + c0), r2);
                    tc_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r2[j]));
                }
                if (c0 + 16 >= d) {                     // last read of this accumulator: hand it back to the MMA warp
                    tc_fence_before();
                    mbar_arrive(tempty0 + 8 * buf);
                }
                if (px < a.HW) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) store_out(op + (size_t)(c0 + j) * a.HW, __uint_as_float(r[j]) + __ldg(bias + c0 + j));
                }
            }
        }
    }
    if (!ok) atomicExch(&g_wait_timeout, 1);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == MMA_WARP) tc_dealloc(tmem_base, (unsigned)a.tmem_cols);
}

// ---------------------------------------------------------------------------------- GroupNorm statistics and the fold
// one 16-byte load: 4 float32 or 8 16-bit elements, widened to float
template <typename T> struct Vec16 { static constexpr int N = 16 / (int)sizeof(T); };
__device__ __forceinline__ void load16(const float *p, float (&v)[4]) {
    const float4 t = __ldcs(reinterpret_cast<const float4 *>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load16(const __half *p, float (&v)[8]) {
    const uint4 t = __ldcs(reinterpret_cast<const uint4 *>(p));
    const unsigned w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
        v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void load16(const __nv_bfloat16 *p, float (&v)[8]) {
    const uint4 t = __ldcs(reinterpret_cast<const uint4 *>(p));
    const unsigned w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

__device__ __forceinline__ double block_sum(double v, double *scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    double t = 0;
    if (threadIdx.x == 0)
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += scratch[w];
    return t;       // valid in thread 0
}

// grid (nsplit, B * groups): block (s, bg) sums its slice of the n = (C / groups) * HW contiguous elements of group bg
// (16-byte loads, four in flight per thread; float partial sums of at most 32 elements, float64 beyond)
template <typename T>
__global__ void __launch_bounds__(STAT_THREADS) gn_partial_kernel(const T *__restrict__ x, double2 *__restrict__ partial, long long n, int nsplit) {
    constexpr int VN = Vec16<T>::N;
    __shared__ double scratch[STAT_THREADS / 32];
    const T *base = x + (size_t)blockIdx.y * n;
    const long long vecs = n / VN, per = (vecs + nsplit - 1) / nsplit;
    const long long q0 = blockIdx.x * per, q1 = min(vecs, q0 + per);
    double s = 0, ss = 0;
    for (long long q = q0 + threadIdx.x; q < q1; q += 4 * STAT_THREADS) {
        float v[4][VN];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const long long qq = q + (long long)u * STAT_THREADS;
            if (qq < q1) {
                load16(base + qq * VN, v[u]);
            } else {
#pragma unroll
                for (int i = 0; i < VN; ++i) v[u][i] = 0.f;
            }
        }
        float fs = 0.f, fss = 0.f;
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int i = 0; i < VN; ++i) { fs += v[u][i]; fss += v[u][i] * v[u][i]; }
        s += fs; ss += fss;
    }
    const double ts = block_sum(s, scratch), tss = block_sum(ss, scratch);
    if (threadIdx.x == 0) partial[(size_t)blockIdx.y * nsplit + blockIdx.x] = make_double2(ts, tss);
}

// grid (d, images): block (j, b) writes row j of W'[b] (split in two for float32) and bias'[b, j]
template <typename T>
__global__ void __launch_bounds__(STAT_THREADS) gn_fold_kernel(const double2 *__restrict__ partial, int nsplit, const T *__restrict__ gamma,
                                                              const T *__restrict__ beta, const T *__restrict__ weight,
                                                              const T *__restrict__ bias, T *__restrict__ whi, T *__restrict__ wlo,
                                                              float *__restrict__ bias_out, int C, int groups, int d, long long n, float eps) {
    __shared__ float s_mean[MAX_GROUPS], s_rstd[MAX_GROUPS];
    __shared__ double scratch[STAT_THREADS / 32];
    const int j = blockIdx.x, b = blockIdx.y;
    for (int g = threadIdx.x; g < groups; g += STAT_THREADS) {
        double s = 0, ss = 0;
        for (int i = 0; i < nsplit; ++i) {
            const double2 p = partial[((size_t)b * groups + g) * nsplit + i];
            s += p.x; ss += p.y;
        }
        const double mean = s / (double)n, var = fmax(ss / (double)n - mean * mean, 0.0);
        s_mean[g] = (float)mean;
        s_rstd[g] = (float)(1.0 / sqrt(var + (double)eps));
    }
    __syncthreads();
    const int cpg = groups > 0 ? C / groups : C;
    double acc = 0;
    for (int c = threadIdx.x; c < C; c += STAT_THREADS) {
        float scale = 1.f, shift = 0.f;
        if (groups > 0) {
            const int g = c / cpg;
            scale = to_acc(gamma[c]) * s_rstd[g];
            shift = to_acc(beta[c]) - s_mean[g] * scale;
        }
        const float w = to_acc(weight[(size_t)j * C + c]);
        const float wp = w * scale;
        const size_t at = ((size_t)b * d + j) * C + c;
        if (sizeof(T) == 4) {
            const float hi = __uint_as_float(__float_as_uint(wp) & TF32_MASK);
            whi[at] = from_acc<T>(hi);
            wlo[at] = from_acc<T>(wp - hi);
        } else {
            whi[at] = from_acc<T>(wp);
        }
        acc += (double)w * (double)shift;
    }
    const double t = block_sum(acc, scratch);
    if (threadIdx.x == 0) bias_out[(size_t)b * d + j] = (float)(t + (bias != nullptr ? (double)to_acc(bias[j]) : 0.0));
}

// ---------------------------------------------------------------------------------- host side
struct Plan {
    int esize, nsplit, nimg, nx, no, tmem_cols, wide;
    size_t smem;
    size_t partial_ofs, whi_ofs, wlo_ofs, bias_ofs, total;
};

static size_t round256(size_t v) { return (v + 255) & ~(size_t)255; }

// false when the configuration cannot run on the tensor-map / tcgen05 kernel
static bool make_plan(Plan &p, int B, int C, int HW, int d, int groups, int dtype) {
    if (dtype != SAPA_F32 && dtype != SAPA_F16 && dtype != SAPA_BF16) return false;
    p.esize = (int)dtype_size(dtype);
    if (B <= 0 || C <= 0 || HW <= 0 || d < 16 || d > 256 || d % 16 != 0) return false;
    if (((size_t)HW * p.esize) % 16 != 0 || ((size_t)C * p.esize) % 16 != 0) return false;     // tensor-map strides
    if (groups < 0 || groups > MAX_GROUPS || (groups > 0 && (C % groups != 0 || ((size_t)(C / groups) * HW * p.esize) % 16 != 0))) return false;
    // operand slots: split activations + W' blocks (float32), W' block only (16-bit); the rest goes to the activation ring
    const size_t op = p.esize == 4 ? 2 * (size_t)Y_STAGE + 2 * (size_t)d * 128 : (size_t)d * 128;
    const size_t fixed = 1024 + 64 * 8;      // alignment slack + barriers
    p.no = p.esize == 4 ? OP_SLOTS_F32 : OP_SLOTS_16;
    if (fixed + p.no * op + 2 * (size_t)Y_STAGE > SMEM_LIMIT) return false;
    p.nx = (int)std::min<size_t>(MAX_SLOTS, (SMEM_LIMIT - fixed - p.no * op) / Y_STAGE);
    p.smem = fixed + p.no * op + (size_t)p.nx * Y_STAGE;
    p.wide = p.esize == 4 && 4 * d <= 512 ? 1 : 0;     // two accumulators of 2d columns must fit into TMEM
    p.tmem_cols = 32;
    while (p.tmem_cols < 2 * (p.wide ? 2 * d : d)) p.tmem_cols *= 2;
    p.nimg = groups > 0 ? B : 1;
    p.nsplit = groups > 0 ? std::max(1, std::min(MAX_SPLIT, (148 * 8 + B * groups - 1) / (B * groups))) : 1;
    size_t at = 0;
    p.partial_ofs = at; at = round256(at + (size_t)B * std::max(groups, 1) * p.nsplit * sizeof(double2));
    p.whi_ofs = at; at = round256(at + (size_t)p.nimg * d * C * p.esize);
    p.wlo_ofs = at; at = round256(at + (p.esize == 4 ? (size_t)p.nimg * d * C * p.esize : 0));
    p.bias_ofs = at; at = round256(at + (size_t)p.nimg * d * sizeof(float));
    p.total = at;
    return true;
}

template <typename T>
static int run_project(const Plan &p, const void *x, const void *gamma, const void *beta, const void *weight, const void *bias,
                       void *out, unsigned char *ws, int B, int C, int HW, int d, int groups, float eps, cudaStream_t st) {
    constexpr int KCH = 128 / (int)sizeof(T);
    constexpr CUtensorMapDataType type = sizeof(T) == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                         : std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    double2 *partial = reinterpret_cast<double2 *>(ws + p.partial_ofs);
    T *whi = reinterpret_cast<T *>(ws + p.whi_ofs), *wlo = reinterpret_cast<T *>(ws + p.wlo_ofs);
    float *bias_out = reinterpret_cast<float *>(ws + p.bias_ofs);
    const long long n = groups > 0 ? (long long)(C / groups) * HW : 0;
    if (groups > 0) {
        gn_partial_kernel<T><<<dim3(p.nsplit, B * groups), STAT_THREADS, 0, st>>>(static_cast<const T *>(x), partial, n, p.nsplit);
        if (int e = check_launch("gn_partial_kernel")) return e;
    }
    gn_fold_kernel<T><<<dim3(d, p.nimg), STAT_THREADS, 0, st>>>(partial, p.nsplit, static_cast<const T *>(gamma), static_cast<const T *>(beta),
                                                               static_cast<const T *>(weight), static_cast<const T *>(bias), whi, wlo, bias_out,
                                                               C, groups, d, n, eps);
    if (int e = check_launch("gn_fold_kernel")) return e;

    Args a;
    if (!make_nchw_map(&a.x_map, x, HW, 1, C, B, KCH, KCH, 1, type, (int)sizeof(T),
                       CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_nchw_map(&a.whi_map, whi, C, 1, d, p.nimg, KCH, d, 1, type, (int)sizeof(T), CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_nchw_map(&a.wlo_map, sizeof(T) == 4 ? wlo : whi, C, 1, d, p.nimg, KCH, d, 1, type, (int)sizeof(T), CU_TENSOR_MAP_SWIZZLE_128B)) {
        set_error("sapa_project_forward: tensor map creation failed (CUresult %d)", last_encode_result());
        return SAPA_ERR_UNSUPPORTED;
    }
    a.bias = bias_out; a.out = out;
    a.B = B; a.C = C; a.HW = HW; a.d = d; a.w_per_image = groups > 0 ? 1 : 0;
    a.tiles_per_image = (HW + TILE_PX - 1) / TILE_PX;
    a.total_tiles = a.tiles_per_image * B;
    a.kblocks = (C + KCH - 1) / KCH;
    a.nx = p.nx; a.no = p.no; a.tmem_cols = p.tmem_cols; a.wide = p.wide;
    const size_t smem = p.smem;
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    if (cudaFuncSetAttribute(sapa_proj_umma_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        set_error("sapa_project_forward: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(cudaGetLastError()));
        return SAPA_ERR_LAUNCH;
    }
    sapa_proj_umma_kernel<T><<<std::min(a.total_tiles, sms), THREADS, smem, st>>>(a);
    return check_launch("sapa_proj_umma_kernel");
}

}  // namespace proj

int proj_wait_timeout_flag() {
    int flag = 0;
    if (cudaMemcpyFromSymbol(&flag, proj::g_wait_timeout, sizeof(int)) != cudaSuccess) return -1;
    if (flag != 0) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(proj::g_wait_timeout, &zero, sizeof(int)) != cudaSuccess) return -1;
    }
    return flag;
}

}  // namespace sapa

using namespace sapa;

extern "C" {

size_t sapa_project_workspace(int B, int C, int HW, int d, int groups, int dtype) {
    proj::Plan p;
    return proj::make_plan(p, B, C, HW, d, groups, dtype) ? p.total : 0;
}

int sapa_project_forward(const void *x, const void *gamma, const void *beta, const void *weight, const void *bias, void *out,
                         void *workspace, size_t workspace_bytes, int B, int C, int HW, int d, int groups, float eps, int dtype,
                         void *stream) {
    const char *fn = "sapa_project_forward";
    trace_reset();
    SAPA_REQUIRE(dtype_size(dtype) != 0, SAPA_ERR_DTYPE, "%s: unknown dtype code %d", fn, dtype);
    proj::Plan p;
    SAPA_REQUIRE(proj::make_plan(p, B, C, HW, d, groups, dtype), SAPA_ERR_UNSUPPORTED,
                 "%s: needs float32 / float16 / bfloat16, d a multiple of 16 up to 256, rows of HW and C elements that are "
                 "multiples of 16 bytes and C divisible by groups (got B=%d C=%d HW=%d d=%d groups=%d)", fn, B, C, HW, d, groups);
    SAPA_CHECK_PTR(fn, x); SAPA_CHECK_PTR(fn, weight); SAPA_CHECK_PTR(fn, out);
    if (groups > 0) { SAPA_CHECK_PTR(fn, gamma); SAPA_CHECK_PTR(fn, beta); }
    SAPA_REQUIRE(all_aligned16(x, out), SAPA_ERR_ALIGNMENT, "%s: x and out must be 16-byte aligned", fn);
    SAPA_REQUIRE(workspace != nullptr && workspace_bytes >= p.total && reinterpret_cast<uintptr_t>(workspace) % 256 == 0,
                 SAPA_ERR_WORKSPACE, "%s: a 256-byte aligned workspace of %zu bytes is required, got %zu", fn, p.total, workspace_bytes);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned char *ws = static_cast<unsigned char *>(workspace);
    switch (dtype) {
        case SAPA_F32: return proj::run_project<float>(p, x, gamma, beta, weight, bias, out, ws, B, C, HW, d, groups, eps, st);
        case SAPA_F16: return proj::run_project<__half>(p, x, gamma, beta, weight, bias, out, ws, B, C, HW, d, groups, eps, st);
        default: return proj::run_project<__nv_bfloat16>(p, x, gamma, beta, weight, bias, out, ws, B, C, HW, d, groups, eps, st);
    }
}

}  // extern "C"
