// sapa_cl.cu — float32 fused forward of SAPA-B for K = 5, s = 2: logits on the tensor cores, aggregation on the FP32
// pipe with the softmax weights resident in registers.
//
// Why a second float32 kernel.  The aggregation is 80 % of the arithmetic.  Through 3 x tf32 warp-level MMAs it is
// bound by the MMA issue path (the kernel of sapa_tma.cu spends its whole time there); on the FP32 pipe with one
// thread per low-res pixel it needs one shared-memory word per four FMAs, which saturates the shared-memory return path
// (128 bytes per clock per SM, whatever the access width or broadcast) together with the FMA pipe.  Here a lane owns
// a PAIR of neighbouring low-res pixels (8 high-res pixels): their 2 x 25 x 4 softmax weights stay in 200 registers for
// the whole tile, and every value channel streams through them as five 6-wide window rows (three 64-bit loads each):
// 30 words per 200 FMAs, and 16-byte output stores straight from registers.
//
// Tile = 4 x 8 low-res pixels (8 x 16 high-res).  A CTA is 12 warps:
//   * warps 0-7, consumers (240 registers each after setmaxnreg).  Per tile: (1) logits as 3 x tf32 m16n8k8,
//     S[16 px][8 cells] += Q^T K per window row and 8 channels, warp = (tile row, column half); softmax across the
//     quad; (2) probabilities to shared memory as W[row][slot][pair parity][pair][2 x 2 pixel]; (3) aggregation with
//     warp = (tile row, channel half), lane = (pair, channel c8): the lane loads its pair's weights once and walks
//     through the value boxes of its half, channels c8 + 8i.
//   * warp 8, lane 0: producer.  It claims tiles from a global counter and feeds two rings by TMA: 4 slots of key +
//     query stages (16 channels: boxes [8 rows][16 ch][16 cols], 64-byte swizzle) and 2 x 4 slots of value boxes
//     ([8 rows][32 ch][16 cols]), refilling a slot as soon as its consumers have released it, so the loads of the
//     next tile run under the arithmetic of this one.  Warps 9-11 only give their registers away.
// Values outside the image are zero-filled by the TMA unit (the reference's border rule: logit 0, weight kept, value
// 0).  Every wait on a barrier is bounded and raises a device flag instead of spinning for ever.
#include "tma_util.cuh"

#include <atomic>

namespace sapa {

namespace cl {

using namespace tmau;

constexpr int ROWS = 4, COLS = 8;            // low-res tile of a CTA
constexpr int HH = ROWS + 4;                 // halo rows
constexpr int HC = 16;                       // halo columns x0-4 .. x0+11 = one 64-byte row
constexpr int ROWB = HC * 4;                 // 64 bytes
constexpr int KCH = 16;                      // key / query channels per stage
constexpr int VCH = 32;                      // value channels per box
constexpr int NKQ = 4;                       // ring slots for key / query stages
constexpr int NV = 8;                        // value slots: 4 per channel half
constexpr int NCW = 8;                       // consumer warps
constexpr int NT = 384;                      // 12 warps: 8 consumers, the producer warp, 3 register donors
constexpr int K_BYTES = HH * KCH * ROWB;     // 8192: key box; the query box of the same stage follows it
constexpr int SLOT_BYTES = HH * VCH * ROWB;  // 16384 = key box + query box = one value box
static_assert(2 * K_BYTES == SLOT_BYTES, "a key/query stage and a value box share the slot size");
constexpr int W_FLOATS = ROWS * 25 * 2 * 4 * 4;   // probabilities of one tile
constexpr int SMEM_BYTES = (NKQ + NV) * SLOT_BYTES + W_FLOATS * 4 + 1024;
constexpr int TILE_RING = 8;                 // claimed tiles remembered (the producer runs at most 4 tiles ahead)
constexpr int IDLE_LIMIT = 1 << 22;          // producer polls without progress before it gives up

__device__ int g_wait_timeout = 0;
__device__ unsigned g_next_tile[SCHED_SLOTS];
__device__ unsigned g_ctas_done[SCHED_SLOTS];

#ifdef SAPA_CL_TIMING
__device__ unsigned long long g_prof[8];
#define PROF_DECL long long pt_ = clock64(); unsigned long long pacc_[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#define PROF(i) { const long long now_ = clock64(); pacc_[i] += (unsigned long long)(now_ - pt_); pt_ = now_; }
#define PROF_FLUSH if (lane == 0) { for (int i_ = 0; i_ < 8; ++i_) atomicAdd(&g_prof[i_], pacc_[i_]); }
#else
#define PROF_DECL
#define PROF(i)
#define PROF_FLUSH
#endif

struct Args {
    float *out, *attn;     // attn: optional softmax output [B, 25, 2H, 2W]
    int B, d, C, H, W;
    int rows, ytop0;       // key / value tensors hold `rows` rows; output row 0 reads from row ytop0 - 2 on
    int tiles_x, tiles_y;
    int sched_slot;
};

__device__ __forceinline__ int swz(int col, int channel) { return ((((col >> 2) ^ (channel >> 1)) & 3) << 4) | ((col & 3) << 2); }

// volatile: the addresses repeat from tile to tile while the contents change (a plain asm would be hoisted out of the
// tile loop as a pure function of its address)
__device__ __forceinline__ unsigned lds32v(unsigned addr) {
    unsigned v;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void lds64(unsigned addr, float &a, float &b) {
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];\n" : "=f"(a), "=f"(b) : "r"(addr));
}
__device__ __forceinline__ float4 lds128(unsigned addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(NCW * 32) : "memory"); }

__global__ void __launch_bounds__(NT, 1)
sapa_cl_fused_f32_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                         const __grid_constant__ CUtensorMap vmap, const Args a) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) unsigned long long bars[2 * (NKQ + NV)];   // full_kq, full_v, empty_kq, empty_v
    __shared__ int tile_ids[TILE_RING];     // tile_ids[T % TILE_RING] = the T-th tile of this CTA, -1 = none
    const unsigned ring_addr = ((unsigned)__cvta_generic_to_shared(smem_dyn) + 1023u) & ~1023u;
    const unsigned full_kq = (unsigned)__cvta_generic_to_shared(bars), full_v = full_kq + 8 * NKQ;
    const unsigned empty_kq = full_v + 8 * NV, empty_v = empty_kq + 8 * NKQ;
    const unsigned w_addr = ring_addr + (NKQ + NV) * SLOT_BYTES;
    float *wbuf = reinterpret_cast<float *>(smem_dyn + (ring_addr - (unsigned)__cvta_generic_to_shared(smem_dyn)) +
                                            (NKQ + NV) * SLOT_BYTES);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sW = 2 * a.W;
    const size_t hi_plane = (size_t)(2 * a.H) * sW;
    const int nk = (a.d + KCH - 1) / KCH, nv = (a.C + VCH - 1) / VCH;
    const int ntiles = a.B * a.tiles_x * a.tiles_y;
    // value box u of a tile belongs to channel half (u >> 2) & 1; a half sees nb[h] boxes per tile, in increasing u,
    // and cycles through depth[h] of its 4 slots
    const int nb0 = (nv / 8) * 4 + min(4, nv % 8), nb1 = (nv / 8) * 4 + max(0, nv % 8 - 4);

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < NKQ + NV; ++i) mbar_init(full_kq + 8 * i, 1);
#pragma unroll
        for (int i = 0; i < NKQ; ++i) mbar_init(empty_kq + 8 * i, NCW);
#pragma unroll
        for (int i = 0; i < NV; ++i) mbar_init(empty_v + 8 * i, NCW / 2);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    if (warp >= NCW) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 24;\n");
        if (warp != NCW || lane != 0) return;
        // ------------------------------------------------------------------ producer
        int n_claimed = 0;
        bool no_more = false;
        auto tile_of = [&](int T) {          // claims tiles in order until the T-th is known
            while (n_claimed <= T) {
                int c = -1;
                if (!no_more) {
                    c = n_claimed == 0 ? (int)blockIdx.x : (int)(atomicAdd(&g_next_tile[a.sched_slot], 1u) + gridDim.x);
                    if (c >= ntiles) { c = -1; no_more = true; }
                }
                tile_ids[n_claimed % TILE_RING] = c;
                ++n_claimed;
            }
            return tile_ids[T % TILE_RING];
        };
        int s_kq = 0;                 // next key/query stage of the stream (tile s_kq / nk, stage s_kq % nk)
        int q_v[2] = {0, 0};          // next value box of each half's stream
        bool done_kq = false, done_v[2] = {nb0 == 0, nb1 == 0};
        int idle = 0;
        while (!(done_kq && done_v[0] && done_v[1])) {
            bool progress = false;
            if (!done_kq) {
                const int slot = s_kq % NKQ;
                if (mbar_test_wait(empty_kq + 8 * slot, ((s_kq / NKQ) & 1) ^ 1)) {
                    progress = true;
                    const int T = s_kq / nk, it = s_kq % nk;
                    int tile = tile_of(T);
                    if (tile < 0) {
                        mbar_arrive(full_kq + 8 * slot);     // completes the phase without data: the consumers read -1 and stop
                        done_kq = true;
                    } else {
                        const int x0 = (tile % a.tiles_x) * COLS; tile /= a.tiles_x;
                        const int y0 = (tile % a.tiles_y) * ROWS; tile /= a.tiles_y;
                        const unsigned dst = ring_addr + slot * SLOT_BYTES, bar = full_kq + 8 * slot;
                        mbar_expect_tx(bar, 2 * K_BYTES);
                        tma_load_4d(dst, &kmap, bar, x0 - 4, it * KCH, a.ytop0 + y0 - 2, tile);
                        tma_load_4d(dst + K_BYTES, &qmap, bar, 2 * x0, it * KCH, 2 * y0, tile);
                        ++s_kq;
                    }
                }
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (done_v[h]) continue;
                const int nb = h == 0 ? nb0 : nb1, depth = min(4, nb);
                const int slot = 4 * h + q_v[h] % depth;
                if (!mbar_test_wait(empty_v + 8 * slot, ((q_v[h] / depth) & 1) ^ 1)) continue;
                progress = true;
                const int T = q_v[h] / nb, j = q_v[h] % nb;
                int tile = tile_of(T);
                if (tile < 0) { done_v[h] = true; continue; }
                const int x0 = (tile % a.tiles_x) * COLS; tile /= a.tiles_x;
                const int y0 = (tile % a.tiles_y) * ROWS; tile /= a.tiles_y;
                const int u = (j >> 2) * 8 + 4 * h + (j & 3);
                const unsigned bar = full_v + 8 * slot;
                mbar_expect_tx(bar, SLOT_BYTES);
                tma_load_4d(ring_addr + (NKQ + slot) * SLOT_BYTES, &vmap, bar, x0 - 4, u * VCH, a.ytop0 + y0 - 2, tile);
                ++q_v[h];
            }
            if (progress) {
                idle = 0;
            } else {
                __nanosleep(64);
                if (++idle > IDLE_LIMIT) { atomicExch(&g_wait_timeout, 1); break; }
            }
        }
        if (atomicAdd(&g_ctas_done[a.sched_slot], 1u) == gridDim.x - 1) {   // last CTA out: reset the scheduler pair
            g_next_tile[a.sched_slot] = 0u;
            g_ctas_done[a.sched_slot] = 0u;
        }
        return;
    }
    asm volatile("setmaxnreg.inc.sync.aligned.u32 240;\n");

    // ------------------------------------------------------------------ consumers
    // logit phase: warp = (low-res row, 4-column half); lane (g, t) as in the m16n8k8 fragments
    const int wrow = warp >> 1, h = warp & 1;
    const int g = lane >> 2, t = lane & 3;
    const int l = g >> 1;
    const bool ok0 = (2 * t >= l) && (2 * t <= l + 4), ok1 = (2 * t + 1 >= l) && (2 * t + 1 <= l + 4);
    const int q_off0 = t * ROWB + swz(8 * h + g, t), q_off1 = (t + 4) * ROWB + swz(8 * h + g, t + 4);
    const int k_off0 = t * ROWB + swz(2 + 4 * h + g, t), k_off1 = (t + 4) * ROWB + swz(2 + 4 * h + g, t + 4);
    // where this lane's probabilities go: W[prow][slot][pc & 1][pc >> 1][2r + cx], parent column pc = 4h + l
    const int pc = 4 * h + l;
    const int w_lane = ((pc & 1) * 4 + (pc >> 1)) * 4 + (g & 1);       // + (prow*25 + slot)*32 + 2r
    // aggregation phase: warp = (tile row py, channel half); lane = (pair xb, channel c8)
    const int py = warp & 3, half = warp >> 2;
    const int c8 = lane & 7, xb = lane >> 3;
    int voff[3];
#pragma unroll
    for (int p = 0; p < 3; ++p) voff[p] = swz(2 * xb + 2 + 2 * p, c8);      // (c8 + 8i) >> 1 == c8 >> 1 (mod 4)
    const unsigned w_lane_rd = w_addr + xb * 16;
    const int nb = half == 0 ? nb0 : nb1, depth = min(4, nb);
    constexpr float LOG2E = 1.4426950408889634f;

    int s_kq = 0, q_v = 0;
    PROF_DECL
    for (int T = 0;; ++T) {
        int n = 0, x0 = 0, y0 = 0;
        // ------------------------------------------------------------------ logits
        float s[5][4];
        for (int it = 0; it < nk; ++it, ++s_kq) {
            const int slot = s_kq % NKQ;
            PROF(0)
            if (!mbar_wait_bounded(full_kq + 8 * slot, (s_kq / NKQ) & 1)) {
                atomicExch(&g_wait_timeout, 1);
                return;
            }
            PROF(1)
            if (it == 0) {
                int tile = tile_ids[T % TILE_RING];      // published by the producer before the barrier's phase completed
                if (tile < 0) { PROF_FLUSH return; }
                x0 = (tile % a.tiles_x) * COLS; tile /= a.tiles_x;
                y0 = (tile % a.tiles_y) * ROWS; tile /= a.tiles_y;
                n = tile;
#pragma unroll
                for (int dy = 0; dy < 5; ++dy)
#pragma unroll
                    for (int i = 0; i < 4; ++i) s[dy][i] = 0.f;
            }
            const unsigned stage = ring_addr + slot * SLOT_BYTES;
            const unsigned kb = stage + wrow * (KCH * ROWB);
            const unsigned qb = stage + K_BYTES + (2 * wrow) * (KCH * ROWB);
#pragma unroll
            for (int ks = 0; ks < KCH / 8; ++ks) {
                unsigned ah[4], al[4];
                ah[0] = lds32v(qb + ks * 8 * ROWB + q_off0);
                ah[1] = lds32v(qb + KCH * ROWB + ks * 8 * ROWB + q_off0);
                ah[2] = lds32v(qb + ks * 8 * ROWB + q_off1);
                ah[3] = lds32v(qb + KCH * ROWB + ks * 8 * ROWB + q_off1);
                unsigned b0[5], b1[5];
#pragma unroll
                for (int dy = 0; dy < 5; ++dy) {
                    b0[dy] = lds32v(kb + dy * (KCH * ROWB) + ks * 8 * ROWB + k_off0);
                    b1[dy] = lds32v(kb + dy * (KCH * ROWB) + ks * 8 * ROWB + k_off1);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) al[i] = tf32_lo(ah[i]);
#pragma unroll
                for (int dy = 0; dy < 5; ++dy) mma_tf32(s[dy], ah, b0[dy], b1[dy]);
#pragma unroll
                for (int dy = 0; dy < 5; ++dy) mma_tf32(s[dy], al, b0[dy], b1[dy]);
#pragma unroll
                for (int dy = 0; dy < 5; ++dy) mma_tf32(s[dy], ah, tf32_lo(b0[dy]), tf32_lo(b1[dy]));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_kq + 8 * slot);
            PROF(2)
        }
        const int y = y0 + wrow;
        // softmax over the 25 window slots of each pixel (spread over the 4 lanes of a quad);
        // exp(x - m) = 2^(x log2(e) - m log2(e)): one FMA and one ex2 per element
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float m = -INFINITY;
#pragma unroll
            for (int dy = 0; dy < 5; ++dy) {
                if (ok0) m = fmaxf(m, s[dy][2 * r]);
                if (ok1) m = fmaxf(m, s[dy][2 * r + 1]);
            }
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
            m *= LOG2E;
            float z = 0.f;
#pragma unroll
            for (int dy = 0; dy < 5; ++dy) {
                s[dy][2 * r] = ok0 ? ex2(fmaf(s[dy][2 * r], LOG2E, -m)) : 0.f;
                s[dy][2 * r + 1] = ok1 ? ex2(fmaf(s[dy][2 * r + 1], LOG2E, -m)) : 0.f;
                z += s[dy][2 * r] + s[dy][2 * r + 1];
            }
            z += __shfl_xor_sync(0xffffffffu, z, 1);
            z += __shfl_xor_sync(0xffffffffu, z, 2);
            const float inv = 1.f / z;
#pragma unroll
            for (int dy = 0; dy < 5; ++dy) { s[dy][2 * r] *= inv; s[dy][2 * r + 1] *= inv; }
        }
        if (a.attn != nullptr && y < a.H && x0 + pc < a.W) {
            float *an = a.attn + (size_t)n * 25 * hi_plane + (size_t)(2 * y) * sW + 2 * (x0 + 4 * h) + g;
#pragma unroll
            for (int dy = 0; dy < 5; ++dy)
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    if (ok0) an[(size_t)(dy * 5 + 2 * t - l) * hi_plane + (size_t)r * sW] = s[dy][2 * r];
                    if (ok1) an[(size_t)(dy * 5 + 2 * t + 1 - l) * hi_plane + (size_t)r * sW] = s[dy][2 * r + 1];
                }
        }
        {
            float *wp = wbuf + wrow * (25 * 32) + w_lane;
#pragma unroll
            for (int dy = 0; dy < 5; ++dy)
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    if (ok0) wp[(dy * 5 + 2 * t - l) * 32 + 2 * r] = s[dy][2 * r];
                    if (ok1) wp[(dy * 5 + 2 * t + 1 - l) * 32 + 2 * r] = s[dy][2 * r + 1];
                }
        }
        PROF(3)
        consumer_sync();         // the tile's probabilities are complete in shared memory
        PROF(4)

        // ------------------------------------------------------------------ aggregation
        float wreg[25][2][4];
#pragma unroll
        for (int k = 0; k < 25; ++k)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float4 w = lds128(w_lane_rd + ((py * 25 + k) * 32 + j * 16) * 4);
                wreg[k][j][0] = w.x; wreg[k][j][1] = w.y; wreg[k][j][2] = w.z; wreg[k][j][3] = w.w;
            }
        consumer_sync();         // every warp holds its weights: the next tile's probabilities may overwrite the buffer
        PROF(5)
        const bool px_ok = x0 + 2 * xb < a.W && y0 + py < a.H;
        for (int j = 0; j < nb; ++j, ++q_v) {
            const int slot = 4 * half + q_v % depth;
            if (!mbar_wait_bounded(full_v + 8 * slot, (q_v / depth) & 1)) {
                atomicExch(&g_wait_timeout, 1);
                return;
            }
            PROF(6)
            const int chb = ((j >> 2) * 8 + 4 * half + (j & 3)) * VCH;
            const unsigned vb = ring_addr + (NKQ + slot) * SLOT_BYTES + c8 * ROWB + py * (VCH * ROWB);
            float *op = a.out + ((size_t)n * a.C + chb + c8) * hi_plane + (size_t)(2 * (y0 + py)) * sW + 2 * (x0 + 2 * xb);
            float xc[6], xn[6];
#pragma unroll
            for (int p = 0; p < 3; ++p) lds64(vb + voff[p], xc[2 * p], xc[2 * p + 1]);
#pragma unroll 1
            for (int i = 0; i < 4; ++i) {
                float acc[2][4];
#pragma unroll
                for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[jj][e] = 0.f;
#pragma unroll
                for (int dy = 0; dy < 5; ++dy) {
                    // the next window row (of the next channel after the last row) is in flight during these 40 FMAs
                    if (dy < 4) {
#pragma unroll
                        for (int p = 0; p < 3; ++p)
                            lds64(vb + (dy + 1) * (VCH * ROWB) + i * 8 * ROWB + voff[p], xn[2 * p], xn[2 * p + 1]);
                    } else if (i < 3) {
#pragma unroll
                        for (int p = 0; p < 3; ++p) lds64(vb + (i + 1) * 8 * ROWB + voff[p], xn[2 * p], xn[2 * p + 1]);
                    }
#pragma unroll
                    for (int dx = 0; dx < 5; ++dx)
#pragma unroll
                        for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                            for (int e = 0; e < 4; ++e) acc[jj][e] = fmaf(wreg[dy * 5 + dx][jj][e], xc[jj + dx], acc[jj][e]);
#pragma unroll
                    for (int c = 0; c < 6; ++c) xc[c] = xn[c];
                }
                if (px_ok && chb + c8 + 8 * i < a.C) {
                    float *o = op + (size_t)(8 * i) * hi_plane;
                    __stcs(reinterpret_cast<float4 *>(o), make_float4(acc[0][0], acc[0][1], acc[1][0], acc[1][1]));
                    __stcs(reinterpret_cast<float4 *>(o + sW), make_float4(acc[0][2], acc[0][3], acc[1][2], acc[1][3]));
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_v + 8 * slot);
            PROF(7)
        }
    }
}

static std::atomic<unsigned> g_next_sched_slot{0}, g_next_captured_slot{0};

}  // namespace cl

bool fused_cl_supported(int W, int dtype) { return dtype == SAPA_F32 && W % 4 == 0 && cl::encode_tiled_fn() != nullptr; }

// Fused float32 forward for K = 5, s = 2.  Returns SAPA_ERR_UNSUPPORTED when a tensor map cannot be built (the caller then
// uses another kernel).
int launch_fused_cl(const void *q, const void *k, const void *v, void *out, void *attn, int B, int d, int C, int H, int W,
                    int rows, int ytop0, cudaStream_t st) {
    using namespace cl;
    const char *name = "sapa_cl_fused_f32_kernel";
    CUtensorMap qmap, kmap, vmap;
    const auto ty = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    const auto sw = CU_TENSOR_MAP_SWIZZLE_64B;
    if (!make_nchw_map(&qmap, q, 2 * W, 2 * H, d, B, HC, KCH, HH, ty, 4, sw) ||
        !make_nchw_map(&kmap, k, W, rows, d, B, HC, KCH, HH, ty, 4, sw) ||
        !make_nchw_map(&vmap, v, W, rows, C, B, HC, VCH, HH, ty, 4, sw)) {
        set_error("%s: cuTensorMapEncodeTiled rejected the tensor layout (CUresult %d)", name, last_encode_result());
        return SAPA_ERR_UNSUPPORTED;
    }
    Args a{};
    a.out = static_cast<float *>(out); a.attn = static_cast<float *>(attn);
    a.B = B; a.d = d; a.C = C; a.H = H; a.W = W; a.rows = rows; a.ytop0 = ytop0;
    a.tiles_x = ceil_div(W, COLS);
    a.tiles_y = ceil_div(H, ROWS);
    const long long nblocks = (long long)B * a.tiles_x * a.tiles_y;
    if (nblocks > 0x7fffffffLL) {
        set_error("too many tiles");
        return SAPA_ERR_ARGUMENT;
    }
    const cudaError_t e = cudaFuncSetAttribute(sapa_cl_fused_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) {
        set_error("%s: cudaFuncSetAttribute failed: %s", name, cudaGetErrorString(e));
        return SAPA_ERR_LAUNCH;
    }
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
        set_error("%s: cannot query the SM count", name);
        return SAPA_ERR_LAUNCH;
    }
    const unsigned grid = (unsigned)(nblocks < sms ? nblocks : sms);       // persistent: one CTA per SM
    a.sched_slot = next_sched_slot(g_next_sched_slot, g_next_captured_slot, st);
    sapa_cl_fused_f32_kernel<<<grid, NT, SMEM_BYTES, st>>>(qmap, kmap, vmap, a);
    return check_launch(name);
}

#ifdef SAPA_CL_TIMING
extern "C" int sapa_debug_cl_prof(unsigned long long *out) {
    if (cudaMemcpyFromSymbol(out, cl::g_prof, sizeof(cl::g_prof)) != cudaSuccess) return -1;
    static const unsigned long long zeros[8] = {};
    return cudaMemcpyToSymbol(cl::g_prof, zeros, sizeof(zeros)) == cudaSuccess ? 0 : -1;
}
#endif

int cl_wait_timeout_flag() {
    int flag = 0;
    if (cudaMemcpyFromSymbol(&flag, cl::g_wait_timeout, sizeof(int)) != cudaSuccess) return -1;
    if (flag != 0) {
        static const unsigned zeros[tmau::SCHED_SLOTS] = {};
        const int zero = 0;
        if (cudaMemcpyToSymbol(cl::g_next_tile, zeros, sizeof(zeros)) != cudaSuccess ||
            cudaMemcpyToSymbol(cl::g_ctas_done, zeros, sizeof(zeros)) != cudaSuccess ||
            cudaMemcpyToSymbol(cl::g_wait_timeout, &zero, sizeof(int)) != cudaSuccess)
            return -1;
    }
    return flag;
}

}  // namespace sapa
