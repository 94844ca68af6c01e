// sapa_tma.cu — float32 fused SAPA-B forward (K = 5, s = 2) with TMA staging.
//
// Same mathematics and MMA mapping as sapa_mma.cu (3 x tf32 m16n8k8, probabilities kept in registers), but the
// key / query / value tiles are brought into shared memory by the tensor memory accelerator instead of per-lane
// cp.async copies.  Measured reason: with 64-byte row segments the cp.async path delivers about one 16-byte
// lane-copy per clock per SM (4.6 TB/s over the GPU), which alone costs 43 us at config 2, more than the HBM
// time of the whole op.  One elected thread now issues one cp.async.bulk.tensor per tile:
//   * tensors are described as 4-D maps (x, channel, y, image); a box of 16 columns x NCH channels x 8 rows
//     lands in shared memory as [row][channel][16 columns], i.e. 64-byte rows, with the 64-byte swizzle mode;
//   * coordinates outside the tensor (image border, tile overhang, channel tails) are filled with zeros by the
//     hardware, which is exactly the reference's border rule;
//   * completion is signalled on an mbarrier per ring slot (expect_tx = box bytes); every wait is bounded and
//     raises a device-side error flag instead of spinning for ever.
// With channel-minor rows of 64 bytes and the 64-byte swizzle, the per-lane fragment loads of the aggregation
// (lane = 4 * channel + cell) touch 32 different banks.
//
// The logits are computed on the tensor cores as well (3 x tf32, M = 16 pixels, N = 8 window cells, K = 8
// channels): on the FP32 pipe that loop was bound by shared-memory wavefronts (12 per 10 packed FMAs).
#include "common.cuh"

#include <cuda.h>

#include <atomic>


namespace sapa {

namespace tma {

constexpr int ROWS = 4, COLS = 8;          // low-res tile of a CTA
constexpr int HH = ROWS + 4;               // halo rows
constexpr int HC = 16;                     // halo columns x0-4 .. x0+11 = one 64-byte row
constexpr int KCH = 16;                    // key / query channels per stage
constexpr int VCH = 32;                    // value channels per stage
constexpr int NSTAGE = 4;
constexpr int NT = 2 * ROWS * 32;          // 8 warps: (row, 4-pixel half)
constexpr int ROWB = HC * 4;               // 64 bytes
constexpr int K_BYTES = HH * KCH * ROWB;   // 8192: key box [8 rows][16 ch][16 cols]
constexpr int V_BYTES = HH * VCH * ROWB;   // 16384
constexpr int SLOT_BYTES = V_BYTES > 2 * K_BYTES ? V_BYTES : 2 * K_BYTES;
constexpr int O_BYTES = 2 * ROWS * VCH * ROWB;   // 16384: output box [8 hi rows][32 ch][16 hi cols], double-buffered        // = K_BYTES + the query box [8 hi rows][16 ch][16 hi cols] of 8192 bytes
constexpr unsigned TF32_MASK = 0xffffe000u;
constexpr int CTAS_PER_SM = 2;             // resident CTAs per SM the register budget is tuned for
constexpr int WAIT_LIMIT = 1 << 22;        // bounded mbarrier wait (each try suspends for a while in hardware)

__device__ int g_wait_timeout = 0;         // set when a bounded wait gave up (read by tma_wait_timeout_flag)
// Dynamic tile scheduler of the persistent grid.  Every launch uses one of SCHED_SLOTS counter pairs (chosen
// round-robin on the host); the last CTA of a launch to exit resets its pair, so a pair is clean again long
// before the round-robin comes back to it (that would need SCHED_SLOTS launches resident at the same time).
constexpr int SCHED_SLOTS = 256;
__device__ unsigned g_next_tile[SCHED_SLOTS];
__device__ unsigned g_ctas_done[SCHED_SLOTS];

struct Args {
    float *out, *attn;
    int B, d, C, H, W;
    int rows, ytop0;
    int tiles_x, tiles_y;
    int sched_slot;        // index into g_next_tile / g_ctas_done
};

__device__ __forceinline__ void mbar_init(unsigned bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// returns false when the limit was reached
__device__ __forceinline__ bool mbar_wait_bounded(unsigned bar, unsigned parity) {
    for (int i = 0; i < WAIT_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_4d(unsigned dst, const CUtensorMap *map, unsigned bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];\n"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

__device__ __forceinline__ void mma_tf32(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
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
// shared -> global tile store; out-of-range parts of the box (tile overhang, channel tail) are clipped
__device__ __forceinline__ void tma_store_4d(const CUtensorMap *map, unsigned src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];\n"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
// low term of the two-term tf32 split (the high term is the register itself: the tensor core reads its top 19 bits)
__device__ __forceinline__ unsigned tf32_lo(unsigned x) {
    return __float_as_uint(__uint_as_float(x) - __uint_as_float(x & TF32_MASK));
}
// byte offset of element `col` of a 64-byte row under the 64-byte swizzle: the 16-byte chunk index is XORed with
// bits 7..8 of the row's byte offset, which for channel-minor rows of 64 bytes is (channel >> 1) & 3
__device__ __forceinline__ int swz(int col, int channel) { return ((((col >> 2) ^ (channel >> 1)) & 3) << 4) | ((col & 3) << 2); }

__global__ void __launch_bounds__(NT, CTAS_PER_SM)
sapa_tma_fused_f32_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                          const __grid_constant__ CUtensorMap vmap, const __grid_constant__ CUtensorMap omap, const Args a) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) unsigned long long full_bar[NSTAGE];
    // the swizzle pattern is a function of the absolute shared-memory address: align the ring to 1024 bytes
    const unsigned ring_addr = ((unsigned)__cvta_generic_to_shared(smem_dyn) + 1023u) & ~1023u;
    const unsigned bar_addr = (unsigned)__cvta_generic_to_shared(full_bar);
    const unsigned obuf_addr = ring_addr + NSTAGE * SLOT_BYTES;      // two output staging buffers behind the ring

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wrow = warp >> 1, h = warp & 1;
    const int g = lane >> 2, t = lane & 3;
    const int sW = 2 * a.W;
    const size_t hi_plane = (size_t)(2 * a.H) * sW;
    const int nk = (a.d + KCH - 1) / KCH, nv = (a.C + VCH - 1) / VCH, total = nk + nv;
    // Persistent CTA: its first tile is blockIdx.x, further tiles come from a global counter.  The stages of
    // successive tiles form one continuous stream through the ring, so the first stages of the next tile are in
    // flight while the current tile finishes.  tile_ids[ti & 3] = tile of the ti-th tile of this CTA, -1 = none.
    const int ntiles = a.B * a.tiles_x * a.tiles_y;
    __shared__ int tile_ids[4];

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < NSTAGE; ++i) {
            mbar_init(bar_addr + 8 * i, 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    // stage gs of this CTA's stream goes to slot gs % NSTAGE; executed by thread 0 only
    bool exhausted = false;
    auto issue = [&](int gs) {
        if (exhausted) return;
        const int ti = gs / total, it = gs - ti * total;
        if (it == 0) {     // first stage of a tile: claim the tile
            int claimed = (int)blockIdx.x;
            if (ti > 0) claimed = (int)(atomicAdd(&g_next_tile[a.sched_slot], 1u) + gridDim.x);
            if (claimed >= ntiles) claimed = -1;
            tile_ids[ti & 3] = claimed;
            if (claimed < 0) { exhausted = true; return; }
        }
        int tile = tile_ids[ti & 3];
        const int tbx = tile % a.tiles_x; tile /= a.tiles_x;
        const int tby = tile % a.tiles_y; tile /= a.tiles_y;
        const int tx0 = tbx * COLS, ty0 = tby * ROWS;
        const unsigned slot = ring_addr + (gs % NSTAGE) * SLOT_BYTES, bar = bar_addr + 8 * (gs % NSTAGE);
        mbar_expect_tx(bar, it < nk ? 2 * K_BYTES : V_BYTES);
        if (it < nk) {
            tma_load_4d(slot, &kmap, bar, tx0 - 4, it * KCH, a.ytop0 + ty0 - 2, tile);
            tma_load_4d(slot + K_BYTES, &qmap, bar, 2 * tx0, it * KCH, 2 * ty0, tile);
        } else {
            tma_load_4d(slot, &vmap, bar, tx0 - 4, (it - nk) * VCH, a.ytop0 + ty0 - 2, tile);
        }
    };
    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < NSTAGE - 1; ++i) issue(i);
    }

    // Lane (g,t): high-res pixel 8h+g of the tile's 16 columns (both rows); after the logit MMAs it holds the
    // window cells j = 2t, 2t+1 of its half's 8-cell span (halo columns 2 + 4h + j); parent l = g/2, window [l, l+4]
    const int l = g >> 1;
    const bool ok0 = (2 * t >= l) && (2 * t <= l + 4), ok1 = (2 * t + 1 >= l) && (2 * t + 1 <= l + 4);

    // swizzled byte offsets inside a 64-byte row
    //   query A fragment: channel t (and t+4), pixel 8h+g        key B fragment: channel t (and t+4), cell g -> column 2+4h+g
    //   value A fragment: channel g (and g+8), cells t and t+4 -> columns 2+4h+t, 6+4h+t
    const int q_off0 = t * ROWB + swz(8 * h + g, t), q_off1 = (t + 4) * ROWB + swz(8 * h + g, t + 4);
    const int k_off0 = t * ROWB + swz(2 + 4 * h + g, t), k_off1 = (t + 4) * ROWB + swz(2 + 4 * h + g, t + 4);
    const int v_offa = g * ROWB + swz(2 + 4 * h + t, g), v_offb = g * ROWB + swz(6 + 4 * h + t, g);
    //   output D fragment: channel g (and g+8), pixels 8h+2t, 8h+2t+1 of high-res rows 2*wrow, 2*wrow+1
    const int o_off = (2 * wrow) * (VCH * ROWB) + g * ROWB + swz(8 * h + 2 * t, g);

    float s[2][5][2];                      // logits, then probabilities: [row][dy][cell 2t | 2t+1]
    unsigned phi[2][5][2];                 // B fragments of the aggregation: probabilities of cells (t, t+4); their
                                           // low tf32 terms are derived where they are used (2 ALU ops, 20 registers saved)

    int gs = 0;
    for (int ti = 0;; ++ti) {
    // written by thread 0 at least one barrier earlier (tile 0 is known to everybody)
    int tile = ti == 0 ? (int)blockIdx.x : tile_ids[ti & 3];
    if (tile < 0) break;
    const int bx = tile % a.tiles_x; tile /= a.tiles_x;
    const int by = tile % a.tiles_y; tile /= a.tiles_y;
    const int n = tile;
    const int x0 = bx * COLS, y0 = by * ROWS;
    const int y = y0 + wrow;
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int dy = 0; dy < 5; ++dy) s[r][dy][0] = s[r][dy][1] = 0.f;

    for (int it = 0; it < total; ++it, ++gs) {
        __syncthreads();     // everyone is done with the slot that is refilled next and has written its output fragment
        if (tid == 0) {
            if (it > nk) {   // the previous stage was a value stage: its output tile is complete in shared memory
                tma_store_4d(&omap, obuf_addr + ((it - nk - 1) & 1) * O_BYTES, 2 * x0, (it - nk - 1) * VCH, 2 * y0, n);
                asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
            }
            issue(gs + NSTAGE - 1);
        }
        if (!mbar_wait_bounded(bar_addr + 8 * (gs % NSTAGE), (gs / NSTAGE) & 1)) {
            atomicExch(&g_wait_timeout, 1);
            return;
        }
        const unsigned stage = ring_addr + (it % NSTAGE) * SLOT_BYTES;

        if (it < nk) {
            // ------------------------------------------------------------- logits: S[16 px][8 cells] += Qt[16 px][8 ch] K[8 ch][8 cells]
            const unsigned kb = stage + wrow * (KCH * ROWB);
            const unsigned qb = stage + K_BYTES + (2 * wrow) * (KCH * ROWB);
#pragma unroll
            for (int ks = 0; ks < KCH / 8; ++ks) {
                unsigned ah[4], al[4];
                ah[0] = lds32(qb + ks * 8 * ROWB + q_off0);                  // Q[ch t][row 0][px g]
                ah[1] = lds32(qb + KCH * ROWB + ks * 8 * ROWB + q_off0);     // Q[ch t][row 1][px g]
                ah[2] = lds32(qb + ks * 8 * ROWB + q_off1);                  // Q[ch t+4][row 0]
                ah[3] = lds32(qb + KCH * ROWB + ks * 8 * ROWB + q_off1);     // Q[ch t+4][row 1]
#pragma unroll
                for (int i = 0; i < 4; ++i) al[i] = tf32_lo(ah[i]);
#pragma unroll
                for (int dy = 0; dy < 5; ++dy) {
                    const unsigned b0 = lds32(kb + dy * (KCH * ROWB) + ks * 8 * ROWB + k_off0);
                    const unsigned b1 = lds32(kb + dy * (KCH * ROWB) + ks * 8 * ROWB + k_off1);
                    float dacc[4] = {s[0][dy][0], s[0][dy][1], s[1][dy][0], s[1][dy][1]};
                    mma_tf32(dacc, ah, b0, b1);
                    mma_tf32(dacc, al, b0, b1);
                    mma_tf32(dacc, ah, tf32_lo(b0), tf32_lo(b1));
                    s[0][dy][0] = dacc[0]; s[0][dy][1] = dacc[1]; s[1][dy][0] = dacc[2]; s[1][dy][1] = dacc[3];
                }
            }
            if (it == nk - 1) {
                // softmax over the 25 window slots of each pixel (spread over the 4 lanes of a quad)
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    float m = -INFINITY;
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy) {
                        if (ok0) m = fmaxf(m, s[r][dy][0]);
                        if (ok1) m = fmaxf(m, s[r][dy][1]);
                    }
                    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
                    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
                    float z = 0.f;
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy) {
                        s[r][dy][0] = ok0 ? expf(s[r][dy][0] - m) : 0.f;
                        s[r][dy][1] = ok1 ? expf(s[r][dy][1] - m) : 0.f;
                        z += s[r][dy][0] + s[r][dy][1];
                    }
                    z += __shfl_xor_sync(0xffffffffu, z, 1);
                    z += __shfl_xor_sync(0xffffffffu, z, 2);
                    const float inv = 1.f / z;
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy) { s[r][dy][0] *= inv; s[r][dy][1] *= inv; }
                }
                if (a.attn != nullptr && y < a.H && x0 + 4 * h + l < a.W) {
                    float *an = a.attn + (size_t)n * 25 * hi_plane + (size_t)(2 * y) * sW + 2 * (x0 + 4 * h) + g;
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy)
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            if (ok0) an[(size_t)(dy * 5 + 2 * t - l) * hi_plane + (size_t)r * sW] = s[r][dy][0];
                            if (ok1) an[(size_t)(dy * 5 + 2 * t + 1 - l) * hi_plane + (size_t)r * sW] = s[r][dy][1];
                        }
                }
                // cells (2t, 2t+1) -> cells (t, t+4), the k order of the value fragments; split into tf32 hi / lo
                const int src_a = (lane & ~3) | (t >> 1), src_b = src_a + 2;
                const bool odd = t & 1;
#pragma unroll
                for (int r = 0; r < 2; ++r)
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy) {
                        const float a0 = __shfl_sync(0xffffffffu, s[r][dy][0], src_a), a1 = __shfl_sync(0xffffffffu, s[r][dy][1], src_a);
                        const float b0 = __shfl_sync(0xffffffffu, s[r][dy][0], src_b), b1 = __shfl_sync(0xffffffffu, s[r][dy][1], src_b);
                        const unsigned ua = __float_as_uint(odd ? a1 : a0), ub = __float_as_uint(odd ? b1 : b0);
                        phi[r][dy][0] = ua; phi[r][dy][1] = ub;
                    }
            }
        } else {
            // ------------------------------------------------------------- aggregation: Out[16 ch][8 px] += V[16 ch][8 cells] P[8 cells][8 px]
            const unsigned vb = stage + wrow * (VCH * ROWB);
            float acc[VCH / 16][2][4];
#pragma unroll
            for (int b = 0; b < VCH / 16; ++b)
#pragma unroll
                for (int r = 0; r < 2; ++r)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[b][r][i] = 0.f;
            unsigned an[VCH / 16][4];                     // fragments of the next window row, loaded one row ahead
            auto load_row = [&](int dy) {
#pragma unroll
                for (int b = 0; b < VCH / 16; ++b) {
                    const unsigned p = vb + dy * (VCH * ROWB) + b * 16 * ROWB;
                    an[b][0] = lds32(p + v_offa);                 // V[ch g][cell t]
                    an[b][1] = lds32(p + 8 * ROWB + v_offa);      // V[ch g+8][cell t]
                    an[b][2] = lds32(p + v_offb);                 // V[ch g][cell t+4]
                    an[b][3] = lds32(p + 8 * ROWB + v_offb);      // V[ch g+8][cell t+4]
                }
            };
            load_row(0);
#pragma unroll
            for (int dy = 0; dy < 5; ++dy) {
                unsigned ah[VCH / 16][4], al[VCH / 16][4];
#pragma unroll
                for (int b = 0; b < VCH / 16; ++b)
#pragma unroll
                    for (int i = 0; i < 4; ++i) ah[b][i] = an[b][i];
                if (dy < 4) load_row(dy + 1);
#pragma unroll
                for (int b = 0; b < VCH / 16; ++b)
#pragma unroll
                    for (int i = 0; i < 4; ++i) al[b][i] = tf32_lo(ah[b][i]);
#pragma unroll
                for (int b = 0; b < VCH / 16; ++b)
#pragma unroll
                    for (int r = 0; r < 2; ++r) mma_tf32(acc[b][r], ah[b], phi[r][dy][0], phi[r][dy][1]);
#pragma unroll
                for (int b = 0; b < VCH / 16; ++b)
#pragma unroll
                    for (int r = 0; r < 2; ++r) mma_tf32(acc[b][r], al[b], phi[r][dy][0], phi[r][dy][1]);
#pragma unroll
                for (int b = 0; b < VCH / 16; ++b)
#pragma unroll
                    for (int r = 0; r < 2; ++r) mma_tf32(acc[b][r], ah[b], tf32_lo(phi[r][dy][0]), tf32_lo(phi[r][dy][1]));
            }
            // D fragment: d0,d1 = Out[ch g][px 2t, 2t+1], d2,d3 = Out[ch g+8][px 2t, 2t+1] -> staging buffer laid out
            // as the output box [hi row][channel][16 hi cols] (64-byte swizzle), stored by TMA after the next barrier
            {
                const unsigned ob = obuf_addr + ((it - nk) & 1) * O_BYTES + o_off;
#pragma unroll
                for (int b = 0; b < VCH / 16; ++b)
#pragma unroll
                    for (int half = 0; half < 2; ++half)
#pragma unroll
                        for (int r = 0; r < 2; ++r)
                            sts64(ob + r * (VCH * ROWB) + (16 * b + 8 * half) * ROWB, acc[b][r][2 * half], acc[b][r][2 * half + 1]);
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // make the writes visible to the TMA engine
                // the buffer written two value stages from now is this one: its store must have finished reading it
                if (tid == 0) asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
            }
        }
    }
    // the tile's last output block
    __syncthreads();
    if (tid == 0) {
        tma_store_4d(&omap, obuf_addr + ((nv - 1) & 1) * O_BYTES, 2 * x0, (nv - 1) * VCH, 2 * y0, n);
        asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
    }
    }
    if (tid == 0) {
        asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");   // all output tiles are written
        if (atomicAdd(&g_ctas_done[a.sched_slot], 1u) == gridDim.x - 1) {   // last CTA out: reset the scheduler slot
            g_next_tile[a.sched_slot] = 0u;
            g_ctas_done[a.sched_slot] = 0u;
        }
    }
}

// ---------------------------------------------------------------------------------- host side
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled is a driver entry point; it is looked up through the runtime so that the library links
// only against cudart.
static EncodeTiledFn encode_tiled_fn() {
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

// 4-D map over an NCHW float32 tensor seen as (x, channel, y, image); box = 16 columns x box_ch channels x 8 rows
static bool make_map(CUtensorMap *map, const void *base, int width, int height, int channels, int images, int box_ch) {
    EncodeTiledFn encode = encode_tiled_fn();
    if (encode == nullptr) return false;
    const cuuint64_t dims[4] = {(cuuint64_t)width, (cuuint64_t)channels, (cuuint64_t)height, (cuuint64_t)images};
    const cuuint64_t strides[3] = {(cuuint64_t)height * width * 4, (cuuint64_t)width * 4, (cuuint64_t)channels * height * width * 4};
    const cuuint32_t box[4] = {16u, (cuuint32_t)box_ch, 8u, 1u};
    const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tma

// float32, K = 5, s = 2 and every row of every tensor on a 16-byte boundary
bool fused_tma_supported(int W, int dtype) { return dtype == SAPA_F32 && W % 4 == 0 && tma::encode_tiled_fn() != nullptr; }

// Returns SAPA_ERR_UNSUPPORTED when a tensor map cannot be built (the caller then uses the cp.async kernel).
int launch_fused_tma(const void *q, const void *k, const void *v, void *out, void *attn, int B, int d, int C, int H, int W,
                     int rows, int ytop0, cudaStream_t st) {
    using namespace tma;
    CUtensorMap qmap, kmap, vmap, omap;
    if (!make_map(&qmap, q, 2 * W, 2 * H, d, B, KCH) || !make_map(&kmap, k, W, rows, d, B, KCH) ||
        !make_map(&vmap, v, W, rows, C, B, VCH) || !make_map(&omap, out, 2 * W, 2 * H, C, B, VCH)) {
        set_error("sapa_tma_fused: cuTensorMapEncodeTiled rejected the tensor layout");
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
    constexpr int smem = NSTAGE * SLOT_BYTES + 2 * O_BYTES + 1024;
    const cudaError_t e = cudaFuncSetAttribute(sapa_tma_fused_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
        set_error("sapa_tma_fused: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
        return SAPA_ERR_LAUNCH;
    }
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
        set_error("sapa_tma_fused: cannot query the SM count");
        return SAPA_ERR_LAUNCH;
    }
    const long long resident = (long long)CTAS_PER_SM * sms;
    // persistent grid with dynamic tile claiming (static striding left SMs with 6 to 8 tiles instead of ~6.9)
    const unsigned grid = (unsigned)(nblocks < resident ? nblocks : resident);
    static std::atomic<unsigned> next_slot{0};
    a.sched_slot = (int)(next_slot.fetch_add(1u) % SCHED_SLOTS);
    sapa_tma_fused_f32_kernel<<<grid, NT, smem, st>>>(qmap, kmap, vmap, omap, a);
    return check_launch("sapa_tma_fused_f32_kernel");
}

// 1 if a bounded mbarrier wait of the TMA kernel ever gave up on the current device (synchronises the device).
int tma_wait_timeout_flag() {
    int flag = 0;
    if (cudaMemcpyFromSymbol(&flag, tma::g_wait_timeout, sizeof(int)) != cudaSuccess) return -1;
    return flag;
}

}  // namespace sapa
