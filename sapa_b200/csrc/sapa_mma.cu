// sapa_mma.cu — fused SAPA-B forward (sim -> softmax -> atn) for K = 5, s = 2 on the warp-level tensor-core
// path, written like a tiny flash-attention: the softmax output never leaves registers and is fed to the
// aggregation MMA as its B operand.
//
// Why tensor cores: with one thread per low-res pixel the aggregation needs one shared-memory load per four
// FMAs, which saturates the LSU and the FP32 pipe together (profiled: FMA pipe 30 % busy, issue-bound, 3.6x
// off the HBM time).  For pixels of one row the aggregation is a banded GEMM over the window cells,
//     Out[16 ch x 8 px] += V[16 ch x cells] * P[cells x 8 px]         (one high-res row, one window row dy)
// which maps to one MMA per window row: m16n8k8 (tf32, 8 cells = the window span of 4 low-res pixels, 5/8 of
// the band non-zero) or m16n8k16 (f16 / bf16, 16 cells = the span of 8 low-res pixels).  float32 inputs are
// split into two tf32 terms (hi = top 19 bits, which is what the tensor core reads of a float32 register;
// lo = x - hi) and use three MMAs (hi*hi + lo*hi + hi*lo), which keeps float32 accuracy.
//
// These kernels stage their tiles with per-lane cp.async copies.  They are the fall-back of the TMA kernels in
// sapa_tma.cu (same mathematics, tensor maps instead of cp.async) for tensors whose rows are not 16-byte aligned
// (float32: W % 4 != 0, 16-bit: W % 8 != 0), and remain selectable with SAPA_FUSED_IMPL=mma.
//
// CTA = 4 low-res rows x 8 columns.  16-bit kernel: 4 warps, a warp owns the 8 low-res pixels (16 x 2 high-res) of
// one row and takes all fragments with ldmatrix.  float32 kernel: 8 warps = (row, 4-pixel half); logits on the
// FP32 pipe with packed FMAs, value fragments with per-lane 32-bit shared loads (the window starts 8 bytes off a
// 16-byte boundary, so ldmatrix cannot be used).  Everything a stage needs arrives by cp.async into a 4-deep ring
// of shared-memory slots: first 16 channels of the key halo tile (8 rows, zero outside the image) together with
// the same 16 channels of the query tile (8 x 16 high-res pixels) per stage, then 32 (f32) or 64 (16-bit) channels
// of the value halo per stage; no thread waits on a global load inside the compute loops.
#include "common.cuh"

#include <type_traits>

namespace sapa {

namespace mma {

constexpr int ROWS = 4;              // low-res rows per CTA (= warps)
constexpr int COLS = 8;              // low-res columns per CTA
constexpr int HH = ROWS + 4;         // halo rows
constexpr int HP = 16;               // halo row pitch in cells (12 or 16 of them are filled)
constexpr int CELLS = HH * HP;       // 128 cells per channel plane
constexpr int QROWS = 2 * ROWS, QCOLS = 2 * COLS;   // high-res query tile 8 x 16
constexpr int KCH = 16;              // key / query channels per stage
constexpr int NSTAGE = 4;
constexpr int NT = ROWS * 32;
constexpr unsigned TF32_MASK = 0xffffe000u;

// Shared-memory geometry per element type.  Plane strides are chosen so that the 8 row addresses of an
// ldmatrix (8 consecutive channels) fall into 8 different 16-byte bank groups (stride == 16 bytes mod 128) and
// so that per-lane 32-bit fragment loads (lane = 4*channel + word) are conflict-free (stride == 4 words mod 32).
template <typename T> struct Geo;
template <> struct Geo<float> {
    static constexpr int PLANE = 132, QPLANE = 132;   // elements per key/value plane, per query plane
    static constexpr int VCH = 32;                    // value channels per stage
    static constexpr int KOX = 4, VOX = 4;            // halo column 0 is image column x0 - 4: 16-byte aligned copies
};
template <typename T16> struct Geo16 {
    static constexpr int PLANE = 136, QPLANE = 136;
    static constexpr int VCH = 64;
    static constexpr int KOX = 2, VOX = 4;            // the value halo starts at x0-4 so that 8-byte copies are aligned
};
template <> struct Geo<__half> : Geo16<__half> {};
template <> struct Geo<__nv_bfloat16> : Geo16<__nv_bfloat16> {};

template <int BYTES>
__device__ __forceinline__ void cp_async(unsigned smem, const void *gmem) {
    if constexpr (BYTES == 16)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem), "l"(gmem));
    else
        asm volatile("cp.async.ca.shared.global [%0], [%1], %2;\n" ::"r"(smem), "l"(gmem), "n"(BYTES));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

template <int BYTES> __device__ __forceinline__ void zero_chunk(unsigned char *p) {
    if constexpr (BYTES == 16) *reinterpret_cast<uint4 *>(p) = make_uint4(0u, 0u, 0u, 0u);
    else if constexpr (BYTES == 8) *reinterpret_cast<uint2 *>(p) = make_uint2(0u, 0u);
    else *reinterpret_cast<unsigned *>(p) = 0u;
}

// four 8x8 (b16) matrices; lane L supplies the row address of matrix L/8, row L%8
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void mma_tf32(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T>
__device__ __forceinline__ void mma_16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    if constexpr (std::is_same<T, __half>::value)
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ unsigned pack2(__half, float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const unsigned *>(&h);
}
__device__ __forceinline__ unsigned pack2(__nv_bfloat16, float a, float b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const unsigned *>(&h);
}

struct Args {
    const void *q, *k, *v;
    void *out, *attn;
    int B, d, C, H, W;     // H, W: low-res rows / cols for which outputs are produced
    int rows, ytop0;       // rows held by k / v (H + halos) and the k / v row of output row 0
    int tiles_x, tiles_y;
};

// ------------------------------------------------------------------------------------------------
// Producer: copies channel planes of a [NROWS x NCOLS] window (row pitch PITCH elements in shared memory) in
// chunks of BYTES.  Chunk i of a stage (i = tid, tid + NT, ...) belongs to channel i / NCHUNK and chunk slot
// i % NCHUNK; because NT * PERIOD is a multiple of NCHUNK a thread only ever sees PERIOD different slots,
// whose global offsets are computed once per kernel.
// ------------------------------------------------------------------------------------------------
constexpr int gcd_c(int a, int b) { return b == 0 ? a : gcd_c(b, a % b); }

template <typename T, int BYTES, int NCOLS, int NROWS, int PITCH, int NTHREADS = NT>
struct TileCopier {
    static constexpr int ES = sizeof(T);
    static constexpr int EPC = BYTES / ES;                        // elements per chunk
    static constexpr int NCHUNK = NROWS * NCOLS / EPC;            // chunks per plane
    static constexpr int PERIOD = NCHUNK / gcd_c(NCHUNK, NTHREADS);
    static constexpr int CADV = NTHREADS * PERIOD / NCHUNK;             // channels advanced per period
    int src[PERIOD];      // element offset of the chunk inside a global plane, -1 = outside the image
    int dst[PERIOD];      // byte offset of the chunk inside a shared-memory plane
    int ch0[PERIOD];      // first channel this thread copies for that slot

    // (gy0, gx0): image position of tile element (0,0); valid region [0,rows) x [0,cols); row length ld
    __device__ __forceinline__ void init(int tid, int gy0, int gx0, int rows, int cols, int ld) {
#pragma unroll
        for (int u = 0; u < PERIOD; ++u) {
            const int i = tid + u * NTHREADS;
            const int slot = i % NCHUNK, e = slot * EPC;
            const int ty = e / NCOLS, tx = e % NCOLS;
            const int gy = gy0 + ty, gx = gx0 + tx;
            ch0[u] = i / NCHUNK;
            dst[u] = (ty * PITCH + tx) * ES;
            src[u] = (gy >= 0 && gy < rows && gx >= 0 && gx < cols) ? gy * ld + gx : -1;
        }
    }
    // copies channels [0, cn) from `g` (plane stride gplane elements) and stores zeros for [cn, nzero)
    __device__ __forceinline__ void run(const T *g, size_t gplane, int cn, int nzero, unsigned char *smem, unsigned smem_addr,
                                        int plane_bytes) const {
#pragma unroll
        for (int u = 0; u < PERIOD; ++u) {
            int c = ch0[u];
            if (src[u] >= 0) {
                const T *p = g + (size_t)c * gplane + src[u];
                unsigned d = smem_addr + c * plane_bytes + dst[u];
                for (; c < cn; c += CADV, p += (size_t)CADV * gplane, d += CADV * plane_bytes) cp_async<BYTES>(d, p);
            } else {
                for (; c < cn; c += CADV) zero_chunk<BYTES>(smem + c * plane_bytes + dst[u]);
            }
            for (; c < nzero; c += CADV) zero_chunk<BYTES>(smem + c * plane_bytes + dst[u]);
        }
    }
};

// Softmax over the 25 window slots of one high-res pixel whose logits are spread over the 4 lanes of a quad;
// `ok[i]` tells which of the lane's values belong to the window.  v: [5 window rows][NV values per row]
template <int NV>
__device__ __forceinline__ void quad_softmax(float (&v)[5][NV], const bool (&ok)[NV]) {
    float m = -INFINITY;
#pragma unroll
    for (int dy = 0; dy < 5; ++dy)
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (ok[i]) m = fmaxf(m, v[dy][i]);
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
    float z = 0.f;
#pragma unroll
    for (int dy = 0; dy < 5; ++dy)
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            v[dy][i] = ok[i] ? expf(v[dy][i] - m) : 0.f;
            z += v[dy][i];
        }
    z += __shfl_xor_sync(0xffffffffu, z, 1);
    z += __shfl_xor_sync(0xffffffffu, z, 2);
    const float inv = 1.f / z;
#pragma unroll
    for (int dy = 0; dy < 5; ++dy)
#pragma unroll
        for (int i = 0; i < NV; ++i) v[dy][i] *= inv;
}

// ================================================================================================
// float32: logits on the FP32 pipe (packed FMA), aggregation with 3 x tf32 m16n8k8
// ================================================================================================
// 8 warps per CTA: warp = (low-res row, 4-pixel half of the 8 columns), so that a lane keeps only 40 registers of
// probabilities and the register budget leaves room to run two m16 blocks and the next fragment loads at once.
// HB / QB: bytes per cp.async of the halo tiles / of the query tile (what the image width's alignment allows)
constexpr int NT32 = 2 * ROWS * 32;

template <int HB, int QB>
__global__ void __launch_bounds__(NT32, 2) sapa_mma_fused_f32_kernel(const Args a) {
    using T = float;
    using G = Geo<float>;
    constexpr int PLANE = G::PLANE, QPLANE = G::QPLANE, VCH = G::VCH, NBLK = VCH / 16;
    constexpr int PLANE_B = PLANE * 4, QPLANE_B = QPLANE * 4;
    constexpr int HALO_BYTES = KCH * PLANE_B;
    constexpr int SLOT_BYTES = (VCH * PLANE_B > HALO_BYTES + KCH * QPLANE_B) ? VCH * PLANE_B : HALO_BYTES + KCH * QPLANE_B;
    extern __shared__ __align__(128) unsigned char smem_raw[];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wrow = warp >> 1, h = warp & 1;         // low-res row of the tile, 4-pixel half
    const int g = lane >> 2, t = lane & 3;
    int bid = blockIdx.x;
    const int bx = bid % a.tiles_x; bid /= a.tiles_x;
    const int by = bid % a.tiles_y; bid /= a.tiles_y;
    const int n = bid;
    const int x0 = bx * COLS, y0 = by * ROWS;
    const int y = y0 + wrow;
    const int sW = 2 * a.W, sH = 2 * a.H;
    const size_t hi_plane = (size_t)sH * sW, lo_plane = (size_t)a.rows * a.W;
    const T *qn = static_cast<const T *>(a.q) + (size_t)n * a.d * hi_plane;
    const T *kn = static_cast<const T *>(a.k) + (size_t)n * a.d * lo_plane;
    const T *vn = static_cast<const T *>(a.v) + (size_t)n * a.C * lo_plane;
    const unsigned smem_base = (unsigned)__cvta_generic_to_shared(smem_raw);

    TileCopier<T, HB, 16, HH, HP, NT32> halo;          // key and value: image columns x0-4 .. x0+11 (window cell j = column j+2)
    TileCopier<T, QB, QCOLS, QROWS, QCOLS, NT32> qcp;
    halo.init(tid, a.ytop0 + y0 - 2, x0 - G::KOX, a.rows, a.W, a.W);
    qcp.init(tid, 2 * y0, 2 * x0, sH, sW, sW);
    const int nk = (a.d + KCH - 1) / KCH, nv = (a.C + VCH - 1) / VCH, total = nk + nv;

    auto issue = [&](int it) {
        if (it < total) {
            unsigned char *slot = smem_raw + (it % NSTAGE) * SLOT_BYTES;
            const unsigned saddr = smem_base + (it % NSTAGE) * SLOT_BYTES;
            if (it < nk) {
                const int c0 = it * KCH, cn = min(KCH, a.d - c0);
                // key planes that do not exist must read as zero: the contraction runs over all 16 planes
                halo.run(kn + (size_t)c0 * lo_plane, lo_plane, cn, KCH, slot, saddr, PLANE_B);
                qcp.run(qn + (size_t)c0 * hi_plane, hi_plane, cn, KCH, slot + HALO_BYTES, saddr + HALO_BYTES, QPLANE_B);
            } else {
                const int c0 = (it - nk) * VCH, cn = min(VCH, a.C - c0);
                halo.run(vn + (size_t)c0 * lo_plane, lo_plane, cn, cn, slot, saddr, PLANE_B);
            }
        }
        cp_async_commit();
    };

    // Lane (g,t) owns high-res pixel 8h+g of the tile's 16 columns (both high-res rows) and the window cells
    // j = 2t, 2t+1 of the 8-cell span of its half (halo columns 4h + j); the parent of pixel g inside the half
    // is l = g/2 and its window is j in [l, l+4].
    const int l = g >> 1;
    const bool ok2[2] = {(2 * t >= l) && (2 * t <= l + 4), (2 * t + 1 >= l) && (2 * t + 1 <= l + 4)};

    // logits, then probabilities: s[row][dy][cell 2t | 2t+1]
    float s[2][5][2];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int dy = 0; dy < 5; ++dy) s[r][dy][0] = s[r][dy][1] = 0.f;
    // B fragments of the aggregation after the softmax: probabilities of cells (t, t+4) as tf32 hi / lo terms
    unsigned phi[2][5][2], plo[2][5][2];

#pragma unroll
    for (int i = 0; i < NSTAGE - 1; ++i) issue(i);

    for (int it = 0; it < total; ++it) {
        cp_async_wait<NSTAGE - 2>();
        __syncthreads();
        issue(it + NSTAGE - 1);
        const unsigned char *stage = smem_raw + (it % NSTAGE) * SLOT_BYTES;

        if (it < nk) {
            // ------------------------------------------------------------- sim: (cell 2t, cell 2t+1) += q * (key 2t, key 2t+1)
            const float *ks = reinterpret_cast<const float *>(stage) + (wrow * HP + 2 + 4 * h + 2 * t);
            const float *qs = reinterpret_cast<const float *>(stage + HALO_BYTES) + (2 * wrow) * QCOLS + 8 * h + g;
#pragma unroll 8
            for (int c = 0; c < KCH; ++c) {
                const float q0 = qs[c * QPLANE], q1 = qs[c * QPLANE + QCOLS];
                const float2 q00 = make_float2(q0, q0), q11 = make_float2(q1, q1);
#pragma unroll
                for (int dy = 0; dy < 5; ++dy) {
                    const float2 kk = *reinterpret_cast<const float2 *>(ks + c * PLANE + dy * HP);
                    const float2 s0 = __ffma2_rn(q00, kk, make_float2(s[0][dy][0], s[0][dy][1]));
                    const float2 s1 = __ffma2_rn(q11, kk, make_float2(s[1][dy][0], s[1][dy][1]));
                    s[0][dy][0] = s0.x; s[0][dy][1] = s0.y;
                    s[1][dy][0] = s1.x; s[1][dy][1] = s1.y;
                }
            }
            if (it == nk - 1) {
#pragma unroll
                for (int r = 0; r < 2; ++r) quad_softmax<2>(s[r], ok2);
                if (a.attn != nullptr && y < a.H && x0 + 4 * h + l < a.W) {
                    T *an = static_cast<T *>(a.attn) + (size_t)n * 25 * hi_plane + (size_t)(2 * y) * sW + 2 * (x0 + 4 * h) + g;
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy)
#pragma unroll
                        for (int r = 0; r < 2; ++r)
#pragma unroll
                            for (int i = 0; i < 2; ++i)
                                if (ok2[i]) an[(size_t)(dy * 5 + 2 * t + i - l) * hi_plane + (size_t)r * sW] = s[r][dy][i];
                }
                // re-distribute inside the quad from cells (2t, 2t+1) to cells (t, t+4), the k order of the
                // ldmatrix'd value fragments, and split into tf32 hi / lo terms
                const int src_a = (lane & ~3) | (t >> 1), src_b = src_a + 2;
                const bool odd = t & 1;
#pragma unroll
                for (int r = 0; r < 2; ++r)
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy) {
                        const float a0 = __shfl_sync(0xffffffffu, s[r][dy][0], src_a), a1 = __shfl_sync(0xffffffffu, s[r][dy][1], src_a);
                        const float b0 = __shfl_sync(0xffffffffu, s[r][dy][0], src_b), b1 = __shfl_sync(0xffffffffu, s[r][dy][1], src_b);
                        const float pa = odd ? a1 : a0, pb = odd ? b1 : b0;        // cell t, cell t+4
                        const unsigned ua = __float_as_uint(pa), ub = __float_as_uint(pb);
                        phi[r][dy][0] = ua;
                        phi[r][dy][1] = ub;
                        plo[r][dy][0] = __float_as_uint(pa - __uint_as_float(ua & TF32_MASK));
                        plo[r][dy][1] = __float_as_uint(pb - __uint_as_float(ub & TF32_MASK));
                    }
            }
        } else {
            // ------------------------------------------------------------- atn: Out[16 ch][8 px] += V[16 ch][8 cells] P[8 cells][8 px]
            const int c0 = (it - nk) * VCH;
            // a0 = V[ch g][cell t], a1 = V[ch g+8][cell t], a2 = V[ch g][cell t+4], a3 = V[ch g+8][cell t+4]; the window
            // starts 8 bytes off a 16-byte boundary (column 2 + 4h), so ldmatrix cannot be used; bank = 4g + t + const
            const unsigned *vs = reinterpret_cast<const unsigned *>(stage) + g * PLANE + wrow * HP + 2 + 4 * h + t;
            float acc[NBLK][2][4];
#pragma unroll
            for (int b = 0; b < NBLK; ++b)
#pragma unroll
                for (int r = 0; r < 2; ++r)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[b][r][i] = 0.f;
#pragma unroll
            for (int dy = 0; dy < 5; ++dy) {
                unsigned ah[NBLK][4], al[NBLK][4];
#pragma unroll
                for (int b = 0; b < NBLK; ++b) {
                    const unsigned *v0 = vs + 16 * b * PLANE + dy * HP;
                    ah[b][0] = v0[0]; ah[b][1] = v0[8 * PLANE]; ah[b][2] = v0[4]; ah[b][3] = v0[8 * PLANE + 4];
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        al[b][i] = __float_as_uint(__uint_as_float(ah[b][i]) - __uint_as_float(ah[b][i] & TF32_MASK));
                }
                // three passes over the independent accumulators: hi*hi, lo*hi, hi*lo
#pragma unroll
                for (int b = 0; b < NBLK; ++b)
#pragma unroll
                    for (int r = 0; r < 2; ++r) mma_tf32(acc[b][r], ah[b], phi[r][dy][0], phi[r][dy][1]);
#pragma unroll
                for (int b = 0; b < NBLK; ++b)
#pragma unroll
                    for (int r = 0; r < 2; ++r) mma_tf32(acc[b][r], al[b], phi[r][dy][0], phi[r][dy][1]);
#pragma unroll
                for (int b = 0; b < NBLK; ++b)
#pragma unroll
                    for (int r = 0; r < 2; ++r) mma_tf32(acc[b][r], ah[b], plo[r][dy][0], plo[r][dy][1]);
            }
            // D fragment: d0,d1 = Out[ch g][px 2t, 2t+1], d2,d3 = Out[ch g+8][px 2t, 2t+1]
            if (y < a.H && x0 + 4 * h + t < a.W) {
                T *o = static_cast<T *>(a.out) + ((size_t)n * a.C + c0 + g) * hi_plane + (size_t)(2 * y) * sW + 2 * (x0 + 4 * h + t);
                const bool full = c0 + VCH <= a.C;
#pragma unroll
                for (int b = 0; b < NBLK; ++b)
#pragma unroll
                    for (int half = 0; half < 2; ++half) {      // channel g, then channel g + 8
                        if (full || c0 + 16 * b + 8 * half + g < a.C) {
                            store_pair<T>(o, acc[b][0][2 * half], acc[b][0][2 * half + 1]);
                            store_pair<T>(o + sW, acc[b][1][2 * half], acc[b][1][2 * half + 1]);
                        }
                        o += 8 * hi_plane;
                    }
            }
        }
    }
    cp_async_wait<0>();
}

// ================================================================================================
// f16 / bf16: logits and aggregation both with m16n8k16 (16 cells = the window span of 8 low-res pixels)
// ================================================================================================
// HBV / QB: bytes per cp.async of the value halo / of the query tile (the key halo always uses 4-byte copies)
template <typename T, int HBV, int QB>
__global__ void __launch_bounds__(NT, 3) sapa_mma_fused_16_kernel(const Args a) {
    using G = Geo<T>;
    constexpr int PLANE = G::PLANE, QPLANE = G::QPLANE, VCH = G::VCH, NBLK = VCH / 16;
    constexpr int PLANE_B = PLANE * 2, QPLANE_B = QPLANE * 2;
    constexpr int HALO_BYTES = KCH * PLANE_B;
    constexpr int SLOT_BYTES = (VCH * PLANE_B > HALO_BYTES + KCH * QPLANE_B) ? VCH * PLANE_B : HALO_BYTES + KCH * QPLANE_B;
    extern __shared__ __align__(128) unsigned char smem_raw[];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    int bid = blockIdx.x;
    const int bx = bid % a.tiles_x; bid /= a.tiles_x;
    const int by = bid % a.tiles_y; bid /= a.tiles_y;
    const int n = bid;
    const int x0 = bx * COLS, y0 = by * ROWS;
    const int y = y0 + warp;
    const int sW = 2 * a.W, sH = 2 * a.H;
    const size_t hi_plane = (size_t)sH * sW, lo_plane = (size_t)a.rows * a.W;
    const T *qn = static_cast<const T *>(a.q) + (size_t)n * a.d * hi_plane;
    const T *kn = static_cast<const T *>(a.k) + (size_t)n * a.d * lo_plane;
    const T *vn = static_cast<const T *>(a.v) + (size_t)n * a.C * lo_plane;
    const unsigned smem_base = (unsigned)__cvta_generic_to_shared(smem_raw);

    // the 8 spare elements at the end of every plane are read (times a zero probability) by the last window row
    for (int i = tid; i < NSTAGE * VCH; i += NT)
        *reinterpret_cast<uint4 *>(smem_raw + (i / VCH) * SLOT_BYTES + (i % VCH) * PLANE_B + CELLS * 2) = make_uint4(0u, 0u, 0u, 0u);

    TileCopier<T, 4, 12, HH, HP> kcp;            // key: image columns x0-2 .. x0+9 (window cell j = halo column j)
    TileCopier<T, HBV, 16, HH, HP> vcp;          // value: image columns x0-4 .. x0+11 (window cell j = halo column j+2)
    TileCopier<T, QB, QCOLS, QROWS, QCOLS> qcp;
    kcp.init(tid, a.ytop0 + y0 - 2, x0 - G::KOX, a.rows, a.W, a.W);
    vcp.init(tid, a.ytop0 + y0 - 2, x0 - G::VOX, a.rows, a.W, a.W);
    qcp.init(tid, 2 * y0, 2 * x0, sH, sW, sW);
    const int nk = (a.d + KCH - 1) / KCH, nv = (a.C + VCH - 1) / VCH, total = nk + nv;
    __syncthreads();

    auto issue = [&](int it) {
        if (it < total) {
            unsigned char *slot = smem_raw + (it % NSTAGE) * SLOT_BYTES;
            const unsigned saddr = smem_base + (it % NSTAGE) * SLOT_BYTES;
            if (it < nk) {
                const int c0 = it * KCH, cn = min(KCH, a.d - c0);
                kcp.run(kn + (size_t)c0 * lo_plane, lo_plane, cn, KCH, slot, saddr, PLANE_B);
                qcp.run(qn + (size_t)c0 * hi_plane, hi_plane, cn, KCH, slot + HALO_BYTES, saddr + HALO_BYTES, QPLANE_B);
            } else {
                const int c0 = (it - nk) * VCH, cn = min(VCH, a.C - c0);
                vcp.run(vn + (size_t)c0 * lo_plane, lo_plane, cn, cn, slot, saddr, PLANE_B);
            }
        }
        cp_async_commit();
    };

    // Lane (g,t) owns high-res pixels g and g+8 of the warp's 16 columns (both rows) and the window cells
    // j = 2t, 2t+1, 8+2t, 9+2t of the 12-cell span (j = 12..15 do not exist: probability 0).  The parent of pixel p
    // is l = p/2 and its window is j in [l, l+4].
    bool okp[2][4];
#pragma unroll
    for (int p = 0; p < 2; ++p) {
        const int l = (g >> 1) + 4 * p;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j = 2 * t + (i & 1) + 8 * (i >> 1);
            okp[p][i] = (j >= l) && (j <= l + 4);
        }
    }
    // logits, then probabilities: s[row][pixel g | g+8][dy][cell 2t, 2t+1, 8+2t, 9+2t]
    float s[2][2][5][4];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int p = 0; p < 2; ++p)
#pragma unroll
            for (int dy = 0; dy < 5; ++dy)
#pragma unroll
                for (int i = 0; i < 4; ++i) s[r][p][dy][i] = 0.f;
    unsigned pb[2][2][5][2];     // packed probabilities: B fragments (b0, b1) of the aggregation

#pragma unroll
    for (int i = 0; i < NSTAGE - 1; ++i) issue(i);

    for (int it = 0; it < total; ++it) {
        cp_async_wait<NSTAGE - 2>();
        __syncthreads();
        issue(it + NSTAGE - 1);
        const unsigned saddr = smem_base + (it % NSTAGE) * SLOT_BYTES;

        if (it < nk) {
            // ------------------------------------------------------------- sim: S[16 px][16 cells] += Qt[16 px][16 ch] K[16 ch][16 cells]
            // A = Qt via ldmatrix.trans of [ch][px]: matrices (ch 0-7, px 0-7), (ch 0-7, px 8-15), (ch 8-15, px 0-7), (ch 8-15, px 8-15)
            const unsigned qaddr = saddr + HALO_BYTES + (((lane & 7) + 8 * (lane >> 4)) * QPLANE + (2 * warp) * QCOLS + 8 * ((lane >> 3) & 1)) * 2;
            // B = K via ldmatrix.trans of [ch][cell]: matrices (ch 0-7, cells 0-7), (ch 8-15, cells 0-7), (ch 0-7, cells 8-15), (ch 8-15, cells 8-15)
            const unsigned kaddr = saddr + (((lane & 7) + 8 * ((lane >> 3) & 1)) * PLANE + warp * HP + 8 * (lane >> 4)) * 2;
            unsigned qa[2][4];
            ldmatrix_x4_trans(qa[0], qaddr);
            ldmatrix_x4_trans(qa[1], qaddr + QCOLS * 2);
#pragma unroll
            for (int dy = 0; dy < 5; ++dy) {
                unsigned kb[4];
                ldmatrix_x4_trans(kb, kaddr + dy * HP * 2);
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    // D rows g -> pixel g, rows g+8 -> pixel g+8; columns 2t, 2t+1 of the 8-cell tile
                    float dA[4] = {s[r][0][dy][0], s[r][0][dy][1], s[r][1][dy][0], s[r][1][dy][1]};
                    float dB[4] = {s[r][0][dy][2], s[r][0][dy][3], s[r][1][dy][2], s[r][1][dy][3]};
                    mma_16<T>(dA, qa[r], kb[0], kb[1]);
                    mma_16<T>(dB, qa[r], kb[2], kb[3]);
                    s[r][0][dy][0] = dA[0]; s[r][0][dy][1] = dA[1]; s[r][1][dy][0] = dA[2]; s[r][1][dy][1] = dA[3];
                    s[r][0][dy][2] = dB[0]; s[r][0][dy][3] = dB[1]; s[r][1][dy][2] = dB[2]; s[r][1][dy][3] = dB[3];
                }
            }
            if (it == nk - 1) {
#pragma unroll
                for (int r = 0; r < 2; ++r)
#pragma unroll
                    for (int p = 0; p < 2; ++p) quad_softmax<4>(s[r][p], okp[p]);
                if (a.attn != nullptr) {
                    T *an = static_cast<T *>(a.attn) + (size_t)n * 25 * hi_plane;
#pragma unroll
                    for (int p = 0; p < 2; ++p) {
                        const int l = (g >> 1) + 4 * p;
                        if (y < a.H && x0 + l < a.W) {
                            const size_t pix = (size_t)(2 * y) * sW + 2 * x0 + 8 * p + g;
#pragma unroll
                            for (int dy = 0; dy < 5; ++dy)
#pragma unroll
                                for (int r = 0; r < 2; ++r)
#pragma unroll
                                    for (int i = 0; i < 4; ++i)
                                        if (okp[p][i])
                                            an[(size_t)(dy * 5 + 2 * t + (i & 1) + 8 * (i >> 1) - l) * hi_plane + pix + (size_t)r * sW] =
                                                from_acc<T>(s[r][p][dy][i]);
                        }
                    }
                }
#pragma unroll
                for (int r = 0; r < 2; ++r)
#pragma unroll
                    for (int p = 0; p < 2; ++p)
#pragma unroll
                        for (int dy = 0; dy < 5; ++dy) {
                            pb[r][p][dy][0] = pack2(T(), s[r][p][dy][0], s[r][p][dy][1]);   // k = 2t, 2t+1   -> cells 2t, 2t+1
                            pb[r][p][dy][1] = pack2(T(), s[r][p][dy][2], s[r][p][dy][3]);   // k = 2t+8, 2t+9 -> cells 8+2t, 9+2t
                        }
            }
        } else {
            // ------------------------------------------------------------- atn: Out[16 ch][8 px] += V[16 ch][16 cells] P[16 cells][8 px]
            const int c0 = (it - nk) * VCH;
            // a0 = V[ch g][cells 2t,2t+1], a1 = V[ch g+8][same], a2 = V[ch g][cells 8+2t, 9+2t], a3 = V[ch g+8][same];
            // window cell j sits in halo column j + 2
            const unsigned *vs = reinterpret_cast<const unsigned *>(smem_raw + (it % NSTAGE) * SLOT_BYTES) + g * (PLANE / 2) + (warp * HP + 2) / 2 + t;
            T *o = static_cast<T *>(a.out) + ((size_t)n * a.C + c0 + g) * hi_plane + (size_t)(2 * y) * sW + 2 * (x0 + t);
            const bool full = c0 + VCH <= a.C;
#pragma unroll
            for (int b = 0; b < NBLK; ++b) {
                float acc[2][2][4];
#pragma unroll
                for (int r = 0; r < 2; ++r)
#pragma unroll
                    for (int p = 0; p < 2; ++p)
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[r][p][i] = 0.f;
#pragma unroll
                for (int dy = 0; dy < 5; ++dy) {
                    const unsigned *v0 = vs + (16 * b) * (PLANE / 2) + dy * (HP / 2);
                    const unsigned av[4] = {v0[0], v0[8 * (PLANE / 2)], v0[4], v0[8 * (PLANE / 2) + 4]};
#pragma unroll
                    for (int r = 0; r < 2; ++r)
#pragma unroll
                        for (int p = 0; p < 2; ++p) mma_16<T>(acc[r][p], av, pb[r][p][dy][0], pb[r][p][dy][1]);
                }
                // D fragment of pixel tile p: d0,d1 = Out[ch g][px 8p + 2t, +1], d2,d3 = Out[ch g+8][same]
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    if (y < a.H && (full || c0 + 16 * b + 8 * half + g < a.C)) {
#pragma unroll
                        for (int p = 0; p < 2; ++p)
                            if (x0 + 4 * p + t < a.W) {
                                store_pair<T>(o + 8 * p, acc[0][p][2 * half], acc[0][p][2 * half + 1]);
                                store_pair<T>(o + 8 * p + sW, acc[1][p][2 * half], acc[1][p][2 * half + 1]);
                            }
                    }
                    o += 8 * hi_plane;
                }
            }
        }
    }
    cp_async_wait<0>();
}

template <typename Kernel>
static int launch_with_smem(Kernel kernel, int threads, int smem, const Args &a, unsigned blocks, cudaStream_t st) {
    // opt in to > 48 KB of dynamic shared memory (a per-function, per-device attribute; cheap to repeat)
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
        set_error("sapa_mma_fused_kernel: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
        return SAPA_ERR_LAUNCH;
    }
    kernel<<<blocks, threads, smem, st>>>(a);
    return check_launch("sapa_mma_fused_kernel");
}

template <typename T> constexpr int slot_bytes() {
    using G = Geo<T>;
    constexpr int v = G::VCH * G::PLANE * (int)sizeof(T);
    constexpr int kq = KCH * (G::PLANE + G::QPLANE) * (int)sizeof(T);
    return v > kq ? v : kq;
}

}  // namespace mma

// True when the tensor-core fused forward can run this problem (K == 5 and s == 2 are the caller's business).
bool fused_mma_supported(int W, int dtype) { return dtype == SAPA_F32 || (dtype != SAPA_F64 && W % 2 == 0); }

int launch_fused_mma(const void *q, const void *k, const void *v, void *out, void *attn, int B, int d, int C, int H, int W,
                     int rows, int ytop0, int dtype, cudaStream_t st) {
    using namespace mma;
    Args a{};
    a.q = q; a.k = k; a.v = v; a.out = out; a.attn = attn;
    a.B = B; a.d = d; a.C = C; a.H = H; a.W = W; a.rows = rows; a.ytop0 = ytop0;
    a.tiles_x = ceil_div(W, COLS);
    a.tiles_y = ceil_div(H, ROWS);
    const long long nblocks = (long long)B * a.tiles_x * a.tiles_y;
    if (nblocks > 0x7fffffffLL) {
        set_error("too many tiles");
        return SAPA_ERR_ARGUMENT;
    }
    const unsigned blocks = (unsigned)nblocks;
    if (dtype == SAPA_F32) {
        constexpr int smem = NSTAGE * slot_bytes<float>();
        // W % 4 == 0: every row of every tensor starts on a 16-byte boundary (the fast copies)
        if (W % 4 == 0) return launch_with_smem(sapa_mma_fused_f32_kernel<16, 16>, NT32, smem, a, blocks, st);
        if (W % 2 == 0) return launch_with_smem(sapa_mma_fused_f32_kernel<8, 16>, NT32, smem, a, blocks, st);
        return launch_with_smem(sapa_mma_fused_f32_kernel<4, 8>, NT32, smem, a, blocks, st);
    }
    if (dtype == SAPA_F16) {
        constexpr int smem = NSTAGE * slot_bytes<__half>();
        return W % 4 == 0 ? launch_with_smem(sapa_mma_fused_16_kernel<__half, 8, 16>, NT, smem, a, blocks, st)
                          : launch_with_smem(sapa_mma_fused_16_kernel<__half, 4, 4>, NT, smem, a, blocks, st);
    }
    if (dtype == SAPA_BF16) {
        constexpr int smem = NSTAGE * slot_bytes<__nv_bfloat16>();
        return W % 4 == 0 ? launch_with_smem(sapa_mma_fused_16_kernel<__nv_bfloat16, 8, 16>, NT, smem, a, blocks, st)
                          : launch_with_smem(sapa_mma_fused_16_kernel<__nv_bfloat16, 4, 4>, NT, smem, a, blocks, st);
    }
    set_error("dtype code %d has no tensor-core kernel", dtype);
    return SAPA_ERR_DTYPE;
}

}  // namespace sapa
