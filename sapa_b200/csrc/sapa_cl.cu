// sapa_cl.cu — float32 fused forward of SAPA-B for K = 5, s = 2: logits on the tensor cores, aggregation on the FP32
// pipe with the softmax weights resident in registers.
//
// Why a second float32 kernel.  The aggregation is 80 % of the arithmetic.  Through 3 x tf32 warp-level MMAs it is
// bound by the MMA issue path (the kernel of sapa_tma.cu spends its whole time there); on the FP32 pipe with one
// thread per low-res pixel it needs one shared-memory word per four FMAs, which saturates the shared-memory return path
// (128 bytes per clock per SM, whatever the access width or broadcast) together with the FMA pipe.  Here a lane owns
// a PAIR of neighbouring low-res pixels (8 high-res pixels): their 2 x 25 x 4 softmax weights stay in 200 registers for
// the whole tile, and every value channel streams through them as five 6-wide window rows (three 64-bit loads each):
// 30 words per 200 FMAs.
//
// Tile = 2 x 16 low-res pixels (4 x 32 high-res): 128-byte rows everywhere.  That is what the memory system wants:
// TMA boxes of 128-byte rows that start on a 32-byte boundary (x0 - 8) cost a third of the 64-byte rows at x0 - 4 of
// an 8-wide tile, and the eight lanes of a row write one full 128-byte line per channel and row (half lines cost the
// aggregation a third of its speed).  One persistent CTA of 8 warps per SM (255 registers per thread).  Per tile:
//   1. logits as 3 x tf32 m16n8k8: S[16 px][8 cells] += Q^T K per window row and 8 channels, warp = (tile row, column
//      quarter); softmax across the quad;
//   2. probabilities to shared memory as W[row][slot][pair parity][pair][2 x 2 pixel];
//   3. aggregation: warp = (tile row, channel quarter), lane = (pair xq, channel slot cq); the lane loads its pair's
//      weights once and walks through the value boxes of its quarter, four channels of a box per lane.
// Loads: two TMA rings with the 128-byte swizzle, 4 slots of key + query stages (16 channels: key box [6 rows][16 ch]
// [32 cols], query box [4 rows][16 ch][32 px]) and 4 x 2 slots of value boxes ([6 rows][16 ch][32 cols]).  There is no
// producer warp (it would cost the other warps 15 registers each): lane 0 of the first warp of every tile row, and of
// any warp that has to wait, runs the producer step under a try-lock - claim tiles from the global counter, refill
// every slot whose consumers have released it - so the loads of the next tile are issued under the arithmetic of
// this one.  Values outside the image are zero-filled by the TMA unit (the reference's border rule: logit 0, weight
// kept, value 0).  Every wait on a barrier is bounded and raises a device flag instead of spinning for ever.
#include "tma_util.cuh"

#include <atomic>

namespace sapa {

namespace cl {

using namespace tmau;

constexpr int ROWS = 2, COLS = 16;           // low-res tile of a CTA
constexpr int HH = ROWS + 4;                 // halo rows
constexpr int HC = 32;                       // halo columns x0-8 .. x0+23 = one 128-byte row
constexpr int ROWB = HC * 4;                 // 128 bytes
constexpr int KCH = 16;                      // key / query channels per stage
constexpr int VCH = 16;                      // value channels per box
#ifndef SAPA_CL_NW
#define SAPA_CL_NW 8
#endif
constexpr int NW = SAPA_CL_NW;               // warps per CTA: 8 (one CTA per SM) or 4 (two CTAs per SM)
constexpr int CTAS_PER_SM = 8 / NW;
constexpr int NT = NW * 32;
constexpr int TASKS = 8 / NW;                // (tile row, column quarter) logit tasks per warp
constexpr int NKQ = NW / 2;                  // ring slots for key / query stages
constexpr int NQT = NW / ROWS;               // channel groups of the aggregation: one per pair of warps
constexpr int BPG = 16 / NQT;                // consecutive value boxes of a 256-channel round owned by one group
constexpr int NV = 2 * NQT;                  // value slots: 2 per channel group
constexpr int K_BYTES = HH * KCH * ROWB;          // 12288: key box
constexpr int Q_BYTES = 2 * ROWS * KCH * ROWB;    // 8192: query box, behind the key box of the same stage
constexpr int KQ_BYTES = K_BYTES + Q_BYTES;       // 20480
constexpr int V_BYTES = HH * VCH * ROWB;          // 12288
static_assert(K_BYTES % 1024 == 0 && KQ_BYTES % 1024 == 0 && V_BYTES % 1024 == 0, "the 128-byte swizzle repeats every 1024 bytes");
constexpr int W_FLOATS = ROWS * 25 * 2 * 8 * 4;   // probabilities of one tile
constexpr int SMEM_BYTES = NKQ * KQ_BYTES + NV * V_BYTES + W_FLOATS * 4 + 1024;
constexpr int TILE_RING = 8;                 // claimed tiles remembered (the producer step runs at most 4 tiles ahead)

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
    int y_begin, y_end;    // low-res output rows produced by this launch (a band of [0, H))
    int tiles_x, tiles_y;  // tiles_y covers the band only
    int sched_slot;
};

// producer state, shared by all warps (touched under the try-lock only)
struct Producer {
    int lock;
    int s_kq;          // next key/query stage of the stream (tile s_kq / nk, stage s_kq % nk)
    int q_v[NQT];      // next value box of each channel quarter's stream
    int n_claimed;     // tiles claimed so far
    int flags;         // 1 = key/query stream ended, 2 << q = value stream of group q ended, 64 = no tiles left
};

// byte offset of element `col` of a 128-byte row under the 128-byte swizzle: the 16-byte chunk index is XORed with
// bits 7..9 of the row's byte offset, which for channel-minor rows of 128 bytes is channel & 7
__device__ __forceinline__ int swz(int col, int channel) { return ((((col >> 2) ^ channel) & 7) << 4) | ((col & 3) << 2); }

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

// boxes per tile of channel group q: box u (16 channels) belongs to group (u % 16) / BPG
__device__ __forceinline__ int boxes_of_quarter(int nv, int q) { return (nv / 16) * BPG + min(BPG, max(0, nv % 16 - BPG * q)); }

__global__ void __launch_bounds__(NT, CTAS_PER_SM)
sapa_cl_fused_f32_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                         const __grid_constant__ CUtensorMap vmap, const Args a) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) unsigned long long bars[2 * (NKQ + NV)];   // full_kq, full_v, empty_kq, empty_v
    __shared__ int tile_ids[TILE_RING];     // tile_ids[T % TILE_RING] = the T-th tile of this CTA, -1 = none
    __shared__ Producer prod;
    const unsigned ring_addr = ((unsigned)__cvta_generic_to_shared(smem_dyn) + 1023u) & ~1023u;
    const unsigned vring_addr = ring_addr + NKQ * KQ_BYTES;
    const unsigned full_kq = (unsigned)__cvta_generic_to_shared(bars), full_v = full_kq + 8 * NKQ;
    const unsigned empty_kq = full_v + 8 * NV, empty_v = empty_kq + 8 * NKQ;
    const unsigned w_addr = vring_addr + NV * V_BYTES;
    float *wbuf = reinterpret_cast<float *>(smem_dyn + (w_addr - (unsigned)__cvta_generic_to_shared(smem_dyn)));

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sW = 2 * a.W;
    const size_t hi_plane = (size_t)(2 * a.H) * sW;
    const int nk = (a.d + KCH - 1) / KCH, nv = (a.C + VCH - 1) / VCH;
    const int ntiles = a.B * a.tiles_x * a.tiles_y;

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < NKQ + NV; ++i) mbar_init(full_kq + 8 * i, 1);
#pragma unroll
        for (int i = 0; i < NKQ; ++i) mbar_init(empty_kq + 8 * i, NW);
#pragma unroll
        for (int i = 0; i < NV; ++i) mbar_init(empty_v + 8 * i, ROWS);      // the warps of one quarter: one per tile row
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        prod.lock = 0; prod.s_kq = 0; prod.n_claimed = 0; prod.flags = 0;
#pragma unroll
        for (int q = 0; q < NQT; ++q) {
            prod.q_v[q] = 0;
            if (boxes_of_quarter(nv, q) == 0) prod.flags |= 2 << q;
        }
    }
    __syncthreads();

    // ------------------------------------------------------------------ producer step
    // Never blocks: it issues what can be issued now.  Slot use: stream index x of a ring with n slots goes to slot
    // x % n in phase (x / n) & 1; a slot may be refilled when its "empty" barrier has completed the phase of the
    // previous use (on a fresh barrier the wait for the phase before the first succeeds at once).
    auto produce = [&]() {
        if (atomicCAS(&prod.lock, 0, 1) != 0) return;
        __threadfence_block();
        volatile Producer *ps = &prod;
        auto tile_of = [&](int T) {          // claims tiles in order until the T-th is known
            while (ps->n_claimed <= T) {
                int c = -1;
                if (!(ps->flags & 64)) {
                    c = ps->n_claimed == 0 ? (int)blockIdx.x : (int)(atomicAdd(&g_next_tile[a.sched_slot], 1u) + gridDim.x);
                    if (c >= ntiles) { c = -1; ps->flags = ps->flags | 64; }
                }
                tile_ids[ps->n_claimed % TILE_RING] = c;
                ps->n_claimed = ps->n_claimed + 1;
            }
            return tile_ids[T % TILE_RING];
        };
#pragma unroll 1
        for (int pass = 0; pass < 16; ++pass) {
            bool progress = false;
            if (!(ps->flags & 1)) {
                const int sk = ps->s_kq, slot = sk % NKQ;
                if (mbar_test_wait(empty_kq + 8 * slot, ((sk / NKQ) & 1) ^ 1)) {
                    progress = true;
                    const int T = sk / nk, it = sk % nk;
                    int tile = tile_of(T);
                    if (tile < 0) {
                        mbar_arrive(full_kq + 8 * slot);     // completes the phase without data: the warps read -1 and stop
                        ps->flags = ps->flags | 1;
                    } else {
                        const int x0 = (tile % a.tiles_x) * COLS; tile /= a.tiles_x;
                        const int y0 = a.y_begin + (tile % a.tiles_y) * ROWS; tile /= a.tiles_y;
                        const unsigned dst = ring_addr + slot * KQ_BYTES, bar = full_kq + 8 * slot;
                        mbar_expect_tx(bar, KQ_BYTES);
                        tma_load_4d(dst, &kmap, bar, x0 - 8, it * KCH, a.ytop0 + y0 - 2, tile);
                        tma_load_4d(dst + K_BYTES, &qmap, bar, 2 * x0, it * KCH, 2 * y0, tile);
                        ps->s_kq = sk + 1;
                    }
                }
            }
#pragma unroll 1
            for (int q = 0; q < NQT; ++q) {
                if (ps->flags & (2 << q)) continue;
                const int nb = boxes_of_quarter(nv, q), depth = min(2, nb);
                const int qv = ps->q_v[q], slot = 2 * q + qv % depth;
                if (!mbar_test_wait(empty_v + 8 * slot, ((qv / depth) & 1) ^ 1)) continue;
                progress = true;
                const int T = qv / nb, j = qv % nb;
                int tile = tile_of(T);
                if (tile < 0) { ps->flags = ps->flags | (2 << q); continue; }
                const int x0 = (tile % a.tiles_x) * COLS; tile /= a.tiles_x;
                const int y0 = a.y_begin + (tile % a.tiles_y) * ROWS; tile /= a.tiles_y;
                const int u = (j / BPG) * 16 + BPG * q + (j % BPG);
                const unsigned bar = full_v + 8 * slot;
                mbar_expect_tx(bar, V_BYTES);
                tma_load_4d(vring_addr + slot * V_BYTES, &vmap, bar, x0 - 8, u * VCH, a.ytop0 + y0 - 2, tile);
                ps->q_v[q] = qv + 1;
            }
            if (!progress) break;
        }
        __threadfence_block();
        atomicExch(&prod.lock, 0);
    };
    // wait for a "full" barrier; lane 0 keeps the loads flowing meanwhile.  false = gave up (flag raised)
    auto wait_full = [&](unsigned bar, unsigned parity) {
        if (mbar_test_wait(bar, parity)) return true;
#pragma unroll 1
        for (int spin = 0; spin < WAIT_LIMIT; ++spin) {
            if (lane == 0) produce();
            __syncwarp();
            if (mbar_try_wait(bar, parity)) return true;
        }
        atomicExch(&g_wait_timeout, 1);
        return false;
    };

    // The two phases of a tile use different per-lane constants.  They are recomputed from the lane / warp index in
    // every tile (the empty asm hides that these never change): kept live across the other phase they would push the
    // aggregation loop, which holds 200 weights in registers, into spilling.
    constexpr float LOG2E = 1.4426950408889634f;

    if (tid == 0) produce();
    int s_kq = 0, q_v = 0;
    PROF_DECL
    for (int T = 0;; ++T) {
        int n = 0, x0 = 0, y0 = 0;
        // ------------------------------------------------------------------ logits
        // warp = (tile row wrow, column quarter qt); lane (g, t) as in the m16n8k8 fragments: pixel column 8 qt + g of
        // the tile's 32, window cells j = 2t, 2t+1 of the quarter's 8-cell span (box columns 4 qt + 6 + j)
        int lane_s = lane, warp_s = warp;
        asm volatile("" : "+r"(lane_s), "+r"(warp_s));
        const int g = lane_s >> 2, t = lane_s & 3;
        const int l = g >> 1;                       // parent inside the quarter; its window = cells l .. l+4
        const bool ok0 = (2 * t >= l) && (2 * t <= l + 4), ok1 = (2 * t + 1 >= l) && (2 * t + 1 <= l + 4);
        float s[TASKS][5][4];
        bool stop = false;
        for (int it = 0; it < nk; ++it, ++s_kq) {
            const int slot = s_kq % NKQ;
            PROF(0)
            if (!wait_full(full_kq + 8 * slot, (s_kq / NKQ) & 1)) return;
            PROF(1)
            if (it == 0) {
                int tile = tile_ids[T % TILE_RING];      // published by the producer step before the barrier's phase completed
                if (tile < 0) { stop = true; break; }
                x0 = (tile % a.tiles_x) * COLS; tile /= a.tiles_x;
                y0 = a.y_begin + (tile % a.tiles_y) * ROWS; tile /= a.tiles_y;
                n = tile;
#pragma unroll
                for (int k = 0; k < TASKS; ++k)
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy)
#pragma unroll
                        for (int i = 0; i < 4; ++i) s[k][dy][i] = 0.f;
            }
            const unsigned stage = ring_addr + slot * KQ_BYTES;
#pragma unroll
            for (int k = 0; k < TASKS; ++k) {
                const int task = warp_s + k * NW, wrow = task >> 2, qt = task & 3;
                // k index t of a fragment reads channel 2t of the 8-channel step and k index t + 4 channel 2t + 1 (the
                // same permutation for query and key, so the sum over the 8 channels is unchanged): under the 128-byte
                // swizzle the even channels (and the odd ones) spread one 8-pixel span over all 32 banks: no conflicts
                const int q_off0 = (2 * t) * ROWB + swz(8 * qt + g, 2 * t), q_off1 = (2 * t + 1) * ROWB + swz(8 * qt + g, 2 * t + 1);
                const int k_off0 = (2 * t) * ROWB + swz(4 * qt + 6 + g, 2 * t), k_off1 = (2 * t + 1) * ROWB + swz(4 * qt + 6 + g, 2 * t + 1);
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
                    for (int dy = 0; dy < 5; ++dy) mma_tf32(s[k][dy], ah, b0[dy], b1[dy]);
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy) mma_tf32(s[k][dy], al, b0[dy], b1[dy]);
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy) mma_tf32(s[k][dy], ah, tf32_lo(b0[dy]), tf32_lo(b1[dy]));
                }
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(empty_kq + 8 * slot);
                if ((warp & 3) == 0) produce();
            }
            PROF(2)
        }
        if (stop) break;           // no tile left (warp-uniform)
#pragma unroll
        for (int k = 0; k < TASKS; ++k) {
            const int task = warp_s + k * NW, wrow = task >> 2, qt = task & 3;
            const int y = y0 + wrow;
            // where this lane's probabilities go: W[prow][slot][pc & 1][pc >> 1][2r + cx], parent column pc = 4 qt + l
            const int pc = 4 * qt + l;
            const int w_lane = ((pc & 1) * 8 + (pc >> 1)) * 4 + (g & 1);       // + (prow*25 + slot)*64 + 2r
            // softmax over the 25 window slots of each pixel (spread over the 4 lanes of a quad);
            // exp(x - m) = 2^(x log2(e) - m log2(e)): one FMA and one ex2 per element
    #pragma unroll
            for (int r = 0; r < 2; ++r) {
                float m = -INFINITY;
    #pragma unroll
                for (int dy = 0; dy < 5; ++dy) {
                    if (ok0) m = fmaxf(m, s[k][dy][2 * r]);
                    if (ok1) m = fmaxf(m, s[k][dy][2 * r + 1]);
                }
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
                m *= LOG2E;
                float z = 0.f;
    #pragma unroll
                for (int dy = 0; dy < 5; ++dy) {
                    s[k][dy][2 * r] = ok0 ? ex2(fmaf(s[k][dy][2 * r], LOG2E, -m)) : 0.f;
                    s[k][dy][2 * r + 1] = ok1 ? ex2(fmaf(s[k][dy][2 * r + 1], LOG2E, -m)) : 0.f;
                    z += s[k][dy][2 * r] + s[k][dy][2 * r + 1];
                }
                z += __shfl_xor_sync(0xffffffffu, z, 1);
                z += __shfl_xor_sync(0xffffffffu, z, 2);
                const float inv = 1.f / z;
    #pragma unroll
                for (int dy = 0; dy < 5; ++dy) { s[k][dy][2 * r] *= inv; s[k][dy][2 * r + 1] *= inv; }
            }
            if (a.attn != nullptr && y < a.y_end && x0 + pc < a.W) {
                float *an = a.attn + (size_t)n * 25 * hi_plane + (size_t)(2 * y) * sW + 2 * x0 + 8 * qt + g;
    #pragma unroll
                for (int dy = 0; dy < 5; ++dy)
    #pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        if (ok0) an[(size_t)(dy * 5 + 2 * t - l) * hi_plane + (size_t)r * sW] = s[k][dy][2 * r];
                        if (ok1) an[(size_t)(dy * 5 + 2 * t + 1 - l) * hi_plane + (size_t)r * sW] = s[k][dy][2 * r + 1];
                    }
            }
            {
                float *wp = wbuf + wrow * (25 * 64) + w_lane;
    #pragma unroll
                for (int dy = 0; dy < 5; ++dy)
    #pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        if (ok0) wp[(dy * 5 + 2 * t - l) * 64 + 2 * r] = s[k][dy][2 * r];
                        if (ok1) wp[(dy * 5 + 2 * t + 1 - l) * 64 + 2 * r] = s[k][dy][2 * r + 1];
                    }
            }
        }
        PROF(3)
        __syncthreads();         // the tile's probabilities are complete in shared memory
        PROF(4)

        // ------------------------------------------------------------------ aggregation
        // warp = (tile row py, channel quarter cqt); lane = (pair xq, channel slot cq -> channel {0, 4, 1, 5}[cq] of each
        // group of 8): the 16 lanes of a half-warp read channels c and c + 4, whose swizzle patterns interlock, so the
        // 64-bit window loads are conflict-free
        int lane_a = lane, warp_a = warp;
        asm volatile("" : "+r"(lane_a), "+r"(warp_a));
        const int py = warp_a & 1, cqt = warp_a >> 1;
        const int xq = lane_a & 7, cq = lane_a >> 3;
        const int ch8 = (cq >> 1) + 4 * (cq & 1);
        int voff[3];
#pragma unroll
        for (int p = 0; p < 3; ++p) voff[p] = ch8 * ROWB + swz(2 * xq + 6 + 2 * p, ch8);
        const int nb = boxes_of_quarter(nv, cqt), depth = min(2, nb);
        float wreg[25][2][4];
        {
            const unsigned w_lane_rd = w_addr + xq * 16;
#pragma unroll
            for (int k = 0; k < 25; ++k)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const float4 w = lds128(w_lane_rd + ((py * 25 + k) * 64 + j * 32) * 4);
                    wreg[k][j][0] = w.x; wreg[k][j][1] = w.y; wreg[k][j][2] = w.z; wreg[k][j][3] = w.w;
                }
        }
        __syncthreads();         // every warp holds its weights: the next tile's probabilities may overwrite the buffer
        PROF(5)
        const bool px_ok = x0 + 2 * xq < a.W && y0 + py < a.y_end;
        for (int j = 0; j < nb; ++j, ++q_v) {
            const int slot = 2 * cqt + q_v % depth;
            if (!wait_full(full_v + 8 * slot, (q_v / depth) & 1)) return;
            PROF(6)
            const int chb = ((j / BPG) * 16 + BPG * cqt + (j % BPG)) * VCH;
            const unsigned vb = vring_addr + slot * V_BYTES + py * (VCH * ROWB);
            float *op = a.out + ((size_t)n * a.C + chb + ch8) * hi_plane + (size_t)(2 * (y0 + py)) * sW + 2 * (x0 + 2 * xq);
            // pass i of a box: channels ch8 + {0, 2, 8, 10}[i]; + 2 flips bit 1 of the channel (clear in ch8), i.e. it
            // XORs the swizzled chunk index with 2
            float xc[6], xn[6];
#pragma unroll
            for (int p = 0; p < 3; ++p) lds64(vb + voff[p], xc[2 * p], xc[2 * p + 1]);
#pragma unroll 1
            for (int i = 0; i < 4; ++i) {
                const int coff = (i & 1) * 2 + (i >> 1) * 8;
                const unsigned vrow = vb + coff * ROWB;
                const int flip = (i & 1) << 5;
                float acc[2][4];
#pragma unroll
                for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[jj][e] = 0.f;
#pragma unroll
                for (int dy = 0; dy < 5; ++dy) {
                    // the next window row (of the next pass after the last row) is in flight during these 40 FMAs
                    if (dy < 4) {
#pragma unroll
                        for (int p = 0; p < 3; ++p)
                            lds64(vrow + (dy + 1) * (VCH * ROWB) + (voff[p] ^ flip), xn[2 * p], xn[2 * p + 1]);
                    } else if (i < 3) {
                        const int nxt = i + 1;
                        const unsigned nrow = vb + ((nxt & 1) * 2 + (nxt >> 1) * 8) * ROWB;
                        const int nflip = (nxt & 1) << 5;
#pragma unroll
                        for (int p = 0; p < 3; ++p) lds64(nrow + (voff[p] ^ nflip), xn[2 * p], xn[2 * p + 1]);
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
                if (px_ok && chb + ch8 + coff < a.C) {
                    float *o = op + (size_t)coff * hi_plane;
                    __stcs(reinterpret_cast<float4 *>(o), make_float4(acc[0][0], acc[0][1], acc[1][0], acc[1][1]));
                    __stcs(reinterpret_cast<float4 *>(o + sW), make_float4(acc[0][2], acc[0][3], acc[1][2], acc[1][3]));
                }
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(empty_v + 8 * slot);
                if (py == 0) produce();
            }
            PROF(7)
        }
    }
    PROF_FLUSH
    if (tid == 0 && atomicAdd(&g_ctas_done[a.sched_slot], 1u) == gridDim.x - 1) {   // last CTA out: reset the scheduler pair
        g_next_tile[a.sched_slot] = 0u;
        g_ctas_done[a.sched_slot] = 0u;
    }
}

static std::atomic<unsigned> g_next_sched_slot{0}, g_next_captured_slot{0};

}  // namespace cl

bool fused_cl_supported(int W, int dtype) { return dtype == SAPA_F32 && W % 4 == 0 && cl::encode_tiled_fn() != nullptr; }

// Fused float32 forward for K = 5, s = 2.  Returns SAPA_ERR_UNSUPPORTED when a tensor map cannot be built (the caller then
// uses another kernel).
int launch_fused_cl(const void *q, const void *k, const void *v, void *out, void *attn, int B, int d, int C, int H, int W,
                    int rows, int ytop0, int y_begin, int y_end, cudaStream_t st) {
    using namespace cl;
    const char *name = "sapa_cl_fused_f32_kernel";
    CUtensorMap qmap, kmap, vmap;
    const auto ty = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
    if (!make_nchw_map(&qmap, q, 2 * W, 2 * H, d, B, HC, KCH, 2 * ROWS, ty, 4, sw) ||
        !make_nchw_map(&kmap, k, W, rows, d, B, HC, KCH, HH, ty, 4, sw) ||
        !make_nchw_map(&vmap, v, W, rows, C, B, HC, VCH, HH, ty, 4, sw)) {
        set_error("%s: cuTensorMapEncodeTiled rejected the tensor layout (CUresult %d)", name, last_encode_result());
        return SAPA_ERR_UNSUPPORTED;
    }
    Args a{};
    a.out = static_cast<float *>(out); a.attn = static_cast<float *>(attn);
    a.B = B; a.d = d; a.C = C; a.H = H; a.W = W; a.rows = rows; a.ytop0 = ytop0;
    a.y_begin = y_begin; a.y_end = y_end;
    a.tiles_x = ceil_div(W, COLS);
    a.tiles_y = ceil_div(y_end - y_begin, ROWS);
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
    const long long resident = (long long)CTAS_PER_SM * sms;
    const unsigned grid = (unsigned)(nblocks < resident ? nblocks : resident);       // persistent grid
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
