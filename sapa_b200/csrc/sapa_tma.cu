// sapa_tma.cu — SAPA-B for K = 5, s = 2 with TMA staging and the contractions on the tensor cores: one float32 kernel
// and one float16 / bfloat16 kernel, each in four modes (fused forward, stage 1 of the fused backward, logits only,
// aggregation only).
//
// Same mathematics as sapa_mma.cu (probabilities kept in registers between the logit MMAs and the aggregation
// MMAs), but the key / query / value tiles are brought into shared memory by the tensor memory accelerator instead
// of per-lane cp.async copies.  Measured reason: with 64-byte row segments the cp.async path delivers about one
// 16-byte lane-copy per clock per SM (4.6 TB/s over the GPU), which alone costs 43 us at B=8, C=256, d=64,
// 64x64 -> 128x128, more than the HBM time of the whole op.  One elected thread issues one cp.async.bulk.tensor per tile:
//   * tensors are described as 4-D maps (x, channel, y, image); a box of BW columns x NCH channels x 8 rows lands
//     in shared memory as [row][channel][BW columns] (float32: 16 columns = 64-byte rows with the 64-byte swizzle);
//   * coordinates outside the tensor (image border, tile overhang, channel tails) are filled with zeros by the
//     hardware, which is exactly the reference's border rule;
//   * completion is signalled on an mbarrier per ring slot (expect_tx = box bytes); every wait is bounded and
//     raises a device-side error flag instead of spinning for ever.
// With channel-minor rows of 64 bytes and the 64-byte swizzle, the per-lane fragment loads of the float32
// aggregation (lane = 4 * channel + cell) touch 32 different banks.
//
// float32 computes the logits on the tensor cores as well (3 x tf32, M = 16 pixels, N = 8 window cells, K = 8
// channels): on the FP32 pipe that loop was bound by shared-memory wavefronts (12 per 10 packed FMAs).
#include "tma_util.cuh"

#include <atomic>


namespace sapa {

namespace tma {

using namespace tmau;

constexpr int ROWS = 4, COLS = 8;          // low-res tile of a CTA
constexpr int HH = ROWS + 4;               // halo rows
constexpr int HC = 16;                     // halo columns x0-4 .. x0+11 = one 64-byte row
constexpr int F_KCH = 16;                  // key / query channels per stage (multiple of 8)
constexpr int F_VCH = 32;                  // value channels per stage (multiple of 16)
constexpr int NSTAGE = 4;                  // ring slots of 16 KB
constexpr int NT = 2 * ROWS * 32;          // 8 warps: (row, 4-pixel half)
constexpr int ROWB = HC * 4;               // 64 bytes
constexpr int K_BYTES = HH * F_KCH * ROWB;   // 8192: key box [8 rows][16 ch][16 cols]
constexpr int V_BYTES = HH * F_VCH * ROWB;   // 16384
constexpr int SLOT_BYTES = V_BYTES > 2 * K_BYTES ? V_BYTES : 2 * K_BYTES;   // a key stage = key box + query box of K_BYTES each
constexpr int O_BYTES = 2 * ROWS * F_VCH * ROWB;   // 16384: output box [8 hi rows][32 ch][16 hi cols], double-buffered
constexpr int CTAS_PER_SM = 2;             // resident CTAs per SM the register budget is tuned for

__device__ int g_wait_timeout = 0;         // set when a bounded wait gave up (read by tma_wait_timeout_flag)
// Dynamic tile scheduler of the persistent grid.  Every launch uses one of SCHED_SLOTS counter pairs (chosen
// round-robin on the host); the last CTA of a launch to exit resets its pair, so a pair is clean again long
// before the round-robin comes back to it (that would need SCHED_SLOTS launches resident at the same time).
__device__ unsigned g_next_tile[SCHED_SLOTS];
__device__ unsigned g_ctas_done[SCHED_SLOTS];

// kernel modes: the fused forward, stage 1 of the fused backward, and the two separate ops of the reference's API
constexpr int MODE_FWD = 0;    // out = atn(softmax(sim(query, key)), value); attn = optional softmax output
constexpr int MODE_BWD = 1;    // see the float32 kernel
constexpr int MODE_SIM = 2;    // logits only: attn (output) = sim(query, key); no value stages
constexpr int MODE_AGG = 3;    // aggregation only: out = atn(attn (input weights), value); no key stages

struct Args {
    void *out, *attn;      // attn: forward = optional output (softmax), backward = input (saved softmax)
    void *ws;              // backward only: logit gradients [B, 25, 2H, 2W], written for the key-gradient gather
    int B, d, C, H, W;
    int rows, ytop0;
    int y_begin, y_end;    // low-res output rows produced by this launch (a band of [0, H); the whole image except in row-slab calls)
    int tiles_x, tiles_y;  // tiles_y covers the band only
    int sched_slot;        // index into g_next_tile / g_ctas_done
    int slots_f32;         // 16-bit kernel, MODE_SIM: the logits are written as float32
};

// byte offset of element `col` of a 64-byte row under the 64-byte swizzle: the 16-byte chunk index is XORed with
// bits 7..8 of the row's byte offset, which for channel-minor rows of 64 bytes is (channel >> 1) & 3
__device__ __forceinline__ int swz(int col, int channel) { return ((((col >> 2) ^ (channel >> 1)) & 3) << 4) | ((col & 3) << 2); }

// BWD = false: out = atn(softmax(sim(query, key)), value).
// BWD = true : the first half of the backward pass with the same data flow.  The "query" map is grad_out and the
//              "key" map the value tensor (logits = dA = sim(grad_out, value) over C channels); the middle step is the
//              softmax backward dS = A * (dA - sum_k A_k dA_k) with the saved attention map, stored to `ws`; the
//              "value" map is the key tensor and the output is grad_query = agg(dS, key).
// MODE_SIM / MODE_AGG: the logit half / the aggregation half alone (sapa_qk_forward, sapa_av_forward and the halves of
//              the separate backward ops); the weights of MODE_AGG are read where MODE_BWD reads the attention map.
template <int MODE>
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
    const int nk = (a.d + F_KCH - 1) / F_KCH, nv = (a.C + F_VCH - 1) / F_VCH, total = nk + nv;
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

    // Stages are issued in stream order (stage gs goes to slot gs % NSTAGE) by thread 0 only.  The producer keeps its
    // position incrementally: per stage it costs a handful of instructions, which matters because the other seven
    // warps wait for warp 0 at the next barrier.
    bool exhausted = false;
    int p_it = 0, p_ti = 0, p_slot = 0, p_n = 0, p_x0 = 0, p_y0 = 0;
    auto issue = [&](int) {
        if (exhausted) return;
        if (p_it == 0) {     // first stage of a tile: claim the tile
            int claimed = (int)blockIdx.x;
            if (p_ti > 0) claimed = (int)(atomicAdd(&g_next_tile[a.sched_slot], 1u) + gridDim.x);
            if (claimed >= ntiles) claimed = -1;
            tile_ids[p_ti & 3] = claimed;
            if (claimed < 0) { exhausted = true; return; }
            p_x0 = (claimed % a.tiles_x) * COLS; claimed /= a.tiles_x;
            p_y0 = a.y_begin + (claimed % a.tiles_y) * ROWS; claimed /= a.tiles_y;
            p_n = claimed;
        }
        const unsigned slot = ring_addr + p_slot * SLOT_BYTES, bar = bar_addr + 8 * p_slot;
        if (p_it < nk) {
            mbar_expect_tx(bar, 2 * K_BYTES);
            tma_load_4d(slot, &kmap, bar, p_x0 - 4, p_it * F_KCH, a.ytop0 + p_y0 - 2, p_n);
            tma_load_4d(slot + K_BYTES, &qmap, bar, 2 * p_x0, p_it * F_KCH, 2 * p_y0, p_n);
        } else {
            mbar_expect_tx(bar, V_BYTES);
            tma_load_4d(slot, &vmap, bar, p_x0 - 4, (p_it - nk) * F_VCH, a.ytop0 + p_y0 - 2, p_n);
        }
        if (++p_it == total) { p_it = 0; ++p_ti; }
        p_slot = (p_slot + 1) % NSTAGE;
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
    //   query A fragment: channels ct, ct+2, pixel 8h+g          key B fragment: channels ct, ct+2, cell g -> column 2+4h+g
    //   value A fragment: channel g (and g+8), cells t and t+4 -> columns 2+4h+t, 6+4h+t
    // k index t of a logit fragment reads channel ct = {0, 1, 4, 5}[t] of the 8-channel step and k index t + 4 reads ct + 2
    // (the same permutation for query and key, so the sum over the 8 channels is unchanged): under the 64-byte swizzle
    // channels 0, 1, 4, 5 start in four different 16-byte bank groups, which makes these loads conflict-free (with the
    // identity order, channels t and t + 2 hit the same banks)
    const int ct = (t & 1) + 4 * (t >> 1);
    const int q_off0 = ct * ROWB + swz(8 * h + g, ct), q_off1 = (ct + 2) * ROWB + swz(8 * h + g, ct + 2);
    const int k_off0 = ct * ROWB + swz(2 + 4 * h + g, ct), k_off1 = (ct + 2) * ROWB + swz(2 + 4 * h + g, ct + 2);
    const int v_offa = g * ROWB + swz(2 + 4 * h + t, g), v_offb = g * ROWB + swz(6 + 4 * h + t, g);
    //   output D fragment: channel g (and g+8), pixels 8h+2t, 8h+2t+1 of high-res rows 2*wrow, 2*wrow+1
    const int o_off = (2 * wrow) * (F_VCH * ROWB) + g * ROWB + swz(8 * h + 2 * t, g);

    float s[5][4];                         // logits, then probabilities: [dy][2 * row + (cell 2t | 2t+1)], the MMA's D fragment
    unsigned phi[2][5][2];                 // B fragments of the aggregation: probabilities of cells (t, t+4); their
                                           // low tf32 terms are derived where they are used (2 ALU ops, 20 registers saved)

    // cells (2t, 2t+1) of the logit fragment -> cells (t, t+4), the k order of the value fragments
    auto realign = [&]() {
        const int src_a = (lane & ~3) | (t >> 1), src_b = src_a + 2;
        const bool odd = t & 1;
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int dy = 0; dy < 5; ++dy) {
                const float a0 = __shfl_sync(0xffffffffu, s[dy][2 * r], src_a), a1 = __shfl_sync(0xffffffffu, s[dy][2 * r + 1], src_a);
                const float b0 = __shfl_sync(0xffffffffu, s[dy][2 * r], src_b), b1 = __shfl_sync(0xffffffffu, s[dy][2 * r + 1], src_b);
                phi[r][dy][0] = __float_as_uint(odd ? a1 : a0);
                phi[r][dy][1] = __float_as_uint(odd ? b1 : b0);
            }
    };

    int gs = 0;
    for (int ti = 0;; ++ti) {
    // written by thread 0 at least one barrier earlier (tile 0 is known to everybody)
    int tile = ti == 0 ? (int)blockIdx.x : tile_ids[ti & 3];
    if (tile < 0) break;
    const int bx = tile % a.tiles_x; tile /= a.tiles_x;
    const int by = tile % a.tiles_y; tile /= a.tiles_y;
    const int n = tile;
    const int x0 = bx * COLS, y0 = a.y_begin + by * ROWS;
    const int y = y0 + wrow;
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int dy = 0; dy < 5; ++dy) s[dy][2 * r] = s[dy][2 * r + 1] = 0.f;

    if (MODE == MODE_AGG) {      // the weights come from memory instead of from the logit stages
        const bool pix_ok = y < a.y_end && x0 + 4 * h + l < a.W;
        const float *ap = static_cast<const float *>(a.attn) + (size_t)n * 25 * hi_plane + (size_t)(2 * y) * sW + 2 * (x0 + 4 * h) + g;
#pragma unroll
        for (int dy = 0; dy < 5; ++dy)
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                s[dy][2 * r] = (pix_ok && ok0) ? __ldg(ap + (size_t)(dy * 5 + 2 * t - l) * hi_plane + (size_t)r * sW) : 0.f;
                s[dy][2 * r + 1] = (pix_ok && ok1) ? __ldg(ap + (size_t)(dy * 5 + 2 * t + 1 - l) * hi_plane + (size_t)r * sW) : 0.f;
            }
        realign();
    }

    for (int it = 0; it < total; ++it, ++gs) {
        __syncthreads();     // everyone is done with the slot that is refilled next and has written its output fragment
        if (tid == 0) {
            if (it > nk) {   // the previous stage was a value stage: its output tile is complete in shared memory
                tma_store_4d(&omap, obuf_addr + ((it - nk - 1) & 1) * O_BYTES, 2 * x0, (it - nk - 1) * F_VCH, 2 * y0, n);
                asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
            }
            issue(gs + NSTAGE - 1);
        }
        if (!mbar_wait_bounded(bar_addr + 8 * (gs % NSTAGE), (gs / NSTAGE) & 1)) {
            atomicExch(&g_wait_timeout, 1);
            return;
        }
        const unsigned stage = ring_addr + (gs % NSTAGE) * SLOT_BYTES;

        if (it < nk) {
            // ------------------------------------------------------------- logits: S[16 px][8 cells] += Qt[16 px][8 ch] K[8 ch][8 cells]
            const unsigned kb = stage + wrow * (F_KCH * ROWB);
            const unsigned qb = stage + K_BYTES + (2 * wrow) * (F_KCH * ROWB);
#pragma unroll
            for (int ks = 0; ks < F_KCH / 8; ++ks) {
                unsigned ah[4], al[4];
                ah[0] = lds32(qb + ks * 8 * ROWB + q_off0);                  // Q[ch t][row 0][px g]
                ah[1] = lds32(qb + F_KCH * ROWB + ks * 8 * ROWB + q_off0);     // Q[ch t][row 1][px g]
                ah[2] = lds32(qb + ks * 8 * ROWB + q_off1);                  // Q[ch t+4][row 0]
                ah[3] = lds32(qb + F_KCH * ROWB + ks * 8 * ROWB + q_off1);     // Q[ch t+4][row 1]
#pragma unroll
                for (int i = 0; i < 4; ++i) al[i] = tf32_lo(ah[i]);
#pragma unroll
                for (int dy = 0; dy < 5; ++dy) {
                    const unsigned b0 = lds32(kb + dy * (F_KCH * ROWB) + ks * 8 * ROWB + k_off0);
                    const unsigned b1 = lds32(kb + dy * (F_KCH * ROWB) + ks * 8 * ROWB + k_off1);
                    mma_tf32(s[dy], ah, b0, b1);
                    mma_tf32(s[dy], al, b0, b1);
                    mma_tf32(s[dy], ah, tf32_lo(b0), tf32_lo(b1));
                }
            }
            if (it == nk - 1 && MODE == MODE_BWD) {
                // softmax backward over the 25 window slots of each pixel (spread over the 4 lanes of a quad)
                const bool pix_ok = y < a.y_end && x0 + 4 * h + l < a.W;
                const size_t poff = (size_t)n * 25 * hi_plane + (size_t)(2 * y) * sW + 2 * (x0 + 4 * h) + g;
                const float *ap = static_cast<const float *>(a.attn) + poff;
                float *wp = static_cast<float *>(a.ws) + poff;
                float av[5][4];
#pragma unroll
                for (int dy = 0; dy < 5; ++dy)
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        av[dy][2 * r] = (pix_ok && ok0) ? __ldg(ap + (size_t)(dy * 5 + 2 * t - l) * hi_plane + (size_t)r * sW) : 0.f;
                        av[dy][2 * r + 1] = (pix_ok && ok1) ? __ldg(ap + (size_t)(dy * 5 + 2 * t + 1 - l) * hi_plane + (size_t)r * sW) : 0.f;
                    }
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    float dot = 0.f;
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy) dot += av[dy][2 * r] * s[dy][2 * r] + av[dy][2 * r + 1] * s[dy][2 * r + 1];
                    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
                    dot += __shfl_xor_sync(0xffffffffu, dot, 2);
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy) {
                        s[dy][2 * r] = av[dy][2 * r] * (s[dy][2 * r] - dot);
                        s[dy][2 * r + 1] = av[dy][2 * r + 1] * (s[dy][2 * r + 1] - dot);
                    }
                }
                if (pix_ok) {
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy)
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            if (ok0) wp[(size_t)(dy * 5 + 2 * t - l) * hi_plane + (size_t)r * sW] = s[dy][2 * r];
                            if (ok1) wp[(size_t)(dy * 5 + 2 * t + 1 - l) * hi_plane + (size_t)r * sW] = s[dy][2 * r + 1];
                        }
                }
            }
            if (it == nk - 1 && MODE == MODE_FWD) {
                // softmax over the 25 window slots of each pixel (spread over the 4 lanes of a quad)
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
                    float z = 0.f;
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy) {
                        s[dy][2 * r] = ok0 ? expf(s[dy][2 * r] - m) : 0.f;
                        s[dy][2 * r + 1] = ok1 ? expf(s[dy][2 * r + 1] - m) : 0.f;
                        z += s[dy][2 * r] + s[dy][2 * r + 1];
                    }
                    z += __shfl_xor_sync(0xffffffffu, z, 1);
                    z += __shfl_xor_sync(0xffffffffu, z, 2);
                    const float inv = 1.f / z;
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy) { s[dy][2 * r] *= inv; s[dy][2 * r + 1] *= inv; }
                }
            }
            if (it == nk - 1 && (MODE == MODE_FWD || MODE == MODE_SIM)) {      // probabilities, or the raw logits of MODE_SIM
                if (a.attn != nullptr && y < a.y_end && x0 + 4 * h + l < a.W) {
                    float *an = static_cast<float *>(a.attn) + (size_t)n * 25 * hi_plane + (size_t)(2 * y) * sW + 2 * (x0 + 4 * h) + g;
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy)
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            if (ok0) an[(size_t)(dy * 5 + 2 * t - l) * hi_plane + (size_t)r * sW] = s[dy][2 * r];
                            if (ok1) an[(size_t)(dy * 5 + 2 * t + 1 - l) * hi_plane + (size_t)r * sW] = s[dy][2 * r + 1];
                        }
                }
            }
            if (it == nk - 1 && MODE != MODE_SIM) realign();
        } else {
            // ------------------------------------------------------------- aggregation: Out[16 ch][8 px] += V[16 ch][8 cells] P[8 cells][8 px]
            const unsigned vb = stage + wrow * (F_VCH * ROWB);
            float acc[F_VCH / 16][2][4];
#pragma unroll
            for (int b = 0; b < F_VCH / 16; ++b)
#pragma unroll
                for (int r = 0; r < 2; ++r)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[b][r][i] = 0.f;
            unsigned an[F_VCH / 16][4];                     // fragments of the next window row, loaded one row ahead
            auto load_row = [&](int dy) {
#pragma unroll
                for (int b = 0; b < F_VCH / 16; ++b) {
                    const unsigned p = vb + dy * (F_VCH * ROWB) + b * 16 * ROWB;
                    an[b][0] = lds32(p + v_offa);                 // V[ch g][cell t]
                    an[b][1] = lds32(p + 8 * ROWB + v_offa);      // V[ch g+8][cell t]
                    an[b][2] = lds32(p + v_offb);                 // V[ch g][cell t+4]
                    an[b][3] = lds32(p + 8 * ROWB + v_offb);      // V[ch g+8][cell t+4]
                }
            };
            load_row(0);
#pragma unroll
            for (int dy = 0; dy < 5; ++dy) {
                unsigned ah[F_VCH / 16][4], al[F_VCH / 16][4];
#pragma unroll
                for (int b = 0; b < F_VCH / 16; ++b)
#pragma unroll
                    for (int i = 0; i < 4; ++i) ah[b][i] = an[b][i];
                if (dy < 4) load_row(dy + 1);
#pragma unroll
                for (int b = 0; b < F_VCH / 16; ++b)
#pragma unroll
                    for (int i = 0; i < 4; ++i) al[b][i] = tf32_lo(ah[b][i]);
#pragma unroll
                for (int b = 0; b < F_VCH / 16; ++b)
#pragma unroll
                    for (int r = 0; r < 2; ++r) mma_tf32(acc[b][r], ah[b], phi[r][dy][0], phi[r][dy][1]);
#pragma unroll
                for (int b = 0; b < F_VCH / 16; ++b)
#pragma unroll
                    for (int r = 0; r < 2; ++r) mma_tf32(acc[b][r], al[b], phi[r][dy][0], phi[r][dy][1]);
#pragma unroll
                for (int b = 0; b < F_VCH / 16; ++b)
#pragma unroll
                    for (int r = 0; r < 2; ++r) mma_tf32(acc[b][r], ah[b], tf32_lo(phi[r][dy][0]), tf32_lo(phi[r][dy][1]));
            }
            // D fragment: d0,d1 = Out[ch g][px 2t, 2t+1], d2,d3 = Out[ch g+8][px 2t, 2t+1] -> staging buffer laid out
            // as the output box [hi row][channel][16 hi cols] (64-byte swizzle), stored by TMA after the next barrier
            {
                const unsigned ob = obuf_addr + ((it - nk) & 1) * O_BYTES + o_off;
#pragma unroll
                for (int b = 0; b < F_VCH / 16; ++b)
#pragma unroll
                    for (int half = 0; half < 2; ++half)
#pragma unroll
                        for (int r = 0; r < 2; ++r)
                            sts64(ob + r * (F_VCH * ROWB) + (16 * b + 8 * half) * ROWB, acc[b][r][2 * half], acc[b][r][2 * half + 1]);
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // make the writes visible to the TMA engine
                // the buffer written two value stages from now is this one: its store must have finished reading it
                if (tid == 0) asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
            }
        }
    }
    // the tile's last output block
    __syncthreads();
    if (tid == 0 && MODE != MODE_SIM) {
        tma_store_4d(&omap, obuf_addr + ((nv - 1) & 1) * O_BYTES, 2 * x0, (nv - 1) * F_VCH, 2 * y0, n);
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

// ---------------------------------------------------------------------------------- float16 / bfloat16
// Same tile (4 x 8 low-res pixels) and scheduler as the float32 kernel; what differs:
//   * key / value boxes are 24 columns wide and start at x0 - 8, the nearest 16-byte boundary below the halo
//     (window cell j of the tile sits in box column j + 6); rows are 48 bytes, unswizzled: eight consecutive
//     channels start in eight different 16-byte bank groups, so every ldmatrix is conflict-free;
//   * query boxes are [8 high-res rows][channels][16 pixels] with 32-byte rows and the 32-byte swizzle;
//   * a warp owns ONE high-res row (16 pixels = two groups of 8): warp = (low-res row, upper / lower high-res row);
//   * logits are computed TRANSPOSED, S^T[16 box columns][8 pixels] = K^T[16 columns][16 ch] Q[16 ch][8 pixels]
//     (m16n8k16; columns 0-15 for the left pixel group, 8-23 for the right one), so that the same 16 columns are
//     the k dimension of the aggregation Out[16 ch][8 px] += V[16 ch][16 columns] P^T[16 columns][8 px]; the
//     accumulator fragment of S^T becomes the B fragment of that product with one movmatrix (8x8 transpose) per
//     packed register;
//   * all fragments come from ldmatrix: K^T and Q with .trans, V without;
//   * no CTA-wide barrier in the steady state: ring slots are handed back on "empty" mbarriers (one arrival per
//     warp) and refilled by one lane of a ninth, producer-only warp; outputs go from registers to global memory.
namespace h16 {
constexpr int COLS = 8;                         // low-res columns of a CTA tile
constexpr int NSTAGE = 4;                       // ring slots of 20 KB
constexpr int NW = 2 * ROWS;                    // 8 consumer warps
constexpr int NT = (NW + 1) * 32;               // + one producer warp
constexpr int CTAS_PER_SM = 2;                  // resident CTAs per SM the register budget is tuned for
constexpr int KCH = 32;                         // key / query channels per stage (k steps of 16 for m16n8k16)
constexpr int VCH = 32;                         // value channels per stage (multiple of 16)
constexpr int BC = 24;                          // key / value box columns
constexpr int KROW = BC * 2;                    // 48 bytes
constexpr int QROW = 32;                        // 16 high-res pixels
constexpr int K_BYTES = HH * KCH * KROW;        // 6144
constexpr int Q_BYTES = 2 * ROWS * KCH * QROW;  // 4096
constexpr int V_BYTES = HH * VCH * KROW;        // 12288
constexpr int SLOT_BYTES = V_BYTES > K_BYTES + Q_BYTES ? V_BYTES : K_BYTES + Q_BYTES;
constexpr int SMEM_BYTES = NSTAGE * SLOT_BYTES + 1024;
static_assert(K_BYTES % 256 == 0 && SLOT_BYTES % 256 == 0, "the swizzled query box needs 256-byte alignment");
}  // namespace h16

__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(unsigned (&r)[2], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2_trans(unsigned (&r)[2], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// 8x8 transpose of a matrix of 16-bit elements held one row-pair per lane
__device__ __forceinline__ unsigned movmatrix_trans(unsigned v) {
    unsigned r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(r) : "r"(v));
    return r;
}
template <typename T>
__device__ __forceinline__ void mma_h16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    if constexpr (std::is_same<T, __half>::value)
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float2 unpack_pair(__half, unsigned u) { return __half22float2(*reinterpret_cast<const __half2 *>(&u)); }
__device__ __forceinline__ float2 unpack_pair(__nv_bfloat16, unsigned u) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&u));
}
__device__ __forceinline__ float ex2_ftz(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

template <typename T, int MODE>     // modes: see the float32 kernel
__global__ void __launch_bounds__(h16::NT, h16::CTAS_PER_SM)
sapa_tma_fused_16_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                         const __grid_constant__ CUtensorMap vmap, const Args a) {
    using namespace h16;
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) unsigned long long bars[2 * h16::NSTAGE];      // full[NSTAGE], empty[NSTAGE]
    __shared__ int tile_ids[4];       // tile_ids[ti & 3] = tile of the ti-th tile of this CTA, -1 = no more tiles
    const unsigned ring_addr = ((unsigned)__cvta_generic_to_shared(smem_dyn) + 1023u) & ~1023u;
    const unsigned full_addr = (unsigned)__cvta_generic_to_shared(bars), empty_addr = full_addr + 8 * h16::NSTAGE;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wrow = warp >> 1, r = warp & 1;
    const int g = lane >> 2, t = lane & 3;
    const int sW = 2 * a.W;
    const size_t hi_plane = (size_t)(2 * a.H) * sW;
    const int nk = (a.d + KCH - 1) / KCH, nv = (a.C + VCH - 1) / VCH, total = nk + nv;
    const int ntiles = a.B * a.tiles_x * a.tiles_y;

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < h16::NSTAGE; ++i) {
            mbar_init(full_addr + 8 * i, 1);
            mbar_init(empty_addr + 8 * i, NW);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    // ---- producer state (lane 0 of the producer warp).  The stages of successive tiles form one continuous stream through
    // the ring; the first tile of a CTA is blockIdx.x, further tiles come from a global counter.
    int p_issued = 0, p_slot = 0, p_phase = 0, p_it = 0, p_ti = 0, p_n = 0, p_x0 = 0, p_y0 = 0;
    bool p_done = false;
    // Issues every stage whose slot is free; when the stage `need` (the one the warp is about to wait for) has not
    // been issued yet it waits for that slot.  A slot is free when all NW warps have released its previous use; on
    // a fresh barrier the wait for the parity of the "previous" phase succeeds at once.
    auto produce = [&](int need) {
        while (!p_done) {
            const unsigned ebar = empty_addr + 8 * p_slot;
            if (!mbar_test_wait(ebar, p_phase ^ 1)) {
                if (p_issued > need) return;
                if (!mbar_wait_bounded(ebar, p_phase ^ 1)) {
                    atomicExch(&g_wait_timeout, 1);
                    p_done = true;
                    return;
                }
            }
            const unsigned bar = full_addr + 8 * p_slot;
            if (p_it == 0) {
                int claimed = (int)blockIdx.x;
                if (p_ti > 0) claimed = (int)(atomicAdd(&g_next_tile[a.sched_slot], 1u) + gridDim.x);
                if (claimed >= ntiles) claimed = -1;
                tile_ids[p_ti & 3] = claimed;
                if (claimed < 0) {
                    mbar_arrive(bar);          // completes the phase without data: the warps read -1 and stop
                    if (atomicAdd(&g_ctas_done[a.sched_slot], 1u) == gridDim.x - 1) {   // last CTA out: reset the scheduler slot
                        g_next_tile[a.sched_slot] = 0u;
                        g_ctas_done[a.sched_slot] = 0u;
                    }
                    p_done = true;
                    return;
                }
                p_x0 = (claimed % a.tiles_x) * h16::COLS; claimed /= a.tiles_x;
                p_y0 = a.y_begin + (claimed % a.tiles_y) * ROWS; claimed /= a.tiles_y;
                p_n = claimed;
            }
            const unsigned dst = ring_addr + p_slot * h16::SLOT_BYTES;
            if (p_it < nk) {
                mbar_expect_tx(bar, h16::K_BYTES + Q_BYTES);
                tma_load_4d(dst, &kmap, bar, p_x0 - 8, p_it * KCH, a.ytop0 + p_y0 - 2, p_n);
                tma_load_4d(dst + h16::K_BYTES, &qmap, bar, 2 * p_x0, p_it * KCH, 2 * p_y0, p_n);
            } else {
                mbar_expect_tx(bar, h16::V_BYTES);
                tma_load_4d(dst, &vmap, bar, p_x0 - 8, (p_it - nk) * VCH, a.ytop0 + p_y0 - 2, p_n);
            }
            ++p_issued;
            if (++p_it == total) { p_it = 0; ++p_ti; }
            if (++p_slot == h16::NSTAGE) { p_slot = 0; p_phase ^= 1; }
        }
    };

    // The producer is a warp of its own (one lane works): inside a consumer warp it sat on that warp's critical path -
    // 40 % of the warp's time at config 2 - and the other warps waited for the stages it had not issued yet.
    if (warp == NW) {
        if (lane == 0) produce(0x7fffffff);
        return;
    }

    // ---- per-lane constants
    // ldmatrix row addresses.  "A-type" lane order: matrices (rows 0-7 | 8-15) x (chunk 0 | 1) as m0..m3 =
    // (lo,0) (hi,0) (lo,1) (hi,1); "T-type": (lo,0) (lo,1) (hi,0) (hi,1).
    const int row_a = (lane & 7) + 8 * ((lane >> 3) & 1), chunk_a = lane >> 4;
    const int row_t = (lane & 7) + 8 * (lane >> 4), chunk_t = (lane >> 3) & 1;
    // query (B of the logits): m0..m3 = (ch 0-7, px 0-7) (ch 8-15, px 0-7) (ch 0-7, px 8-15) (ch 8-15, px 8-15)
    const int q_off = h16::K_BYTES + (2 * wrow + r) * (KCH * QROW) + row_a * QROW + (((chunk_a ^ (row_a >> 2)) & 1) << 4);
    // key (A of the logits, transposed): m0..m3 = (ch 0-7, col 0-7) (ch 0-7, col 8-15) (ch 8-15, col 0-7) (ch 8-15, col 8-15),
    // then m4, m5 = (ch 0-7, col 16-23) (ch 8-15, col 16-23).  The right pixel group's fragment is assembled from
    // m1, m4, m3, m5 (the shared middle columns are loaded once: the kernel is short of shared-memory bandwidth, not of
    // issue slots).
    const int k_off = wrow * (KCH * KROW) + row_t * KROW + chunk_t * 16;
    const int k_off2 = wrow * (KCH * KROW) + row_a * KROW + 32;
    // value (A of the aggregation): m0..m3 = (ch 0-7, col 0-7) (ch 8-15, col 0-7) (ch 0-7, col 8-15) (ch 8-15, col 8-15),
    // then m4, m5 = (ch 0-7, col 16-23) (ch 8-15, col 16-23)
    const int v_off = wrow * (VCH * KROW) + row_a * KROW + chunk_a * 16;
    const int v_off2 = wrow * (VCH * KROW) + row_a * KROW + 32;
    // Lane (g,t) of pixel group p (pixels 8p .. 8p+7 of the row) holds, for the pixels 8p+2t and 8p+2t+1 (parent
    // column l = 4p + t, window = box columns l+6 .. l+10), the box columns 8p+g ("lo") and 8p+g+8 ("hi").
    bool ok_lo[2], ok_hi[2];
    int dx_lo[2];                 // window column of the lo cell (hi = lo + 8)
#pragma unroll
    for (int p = 0; p < 2; ++p) {
        dx_lo[p] = 4 * p + g - t - 6;
        ok_lo[p] = dx_lo[p] >= 0 && dx_lo[p] <= 4;
        ok_hi[p] = dx_lo[p] + 8 >= 0 && dx_lo[p] + 8 <= 4;
    }

    float s[2][5][4];             // logits, then probabilities: [group][dy][(lo,px0) (lo,px1) (hi,px0) (hi,px1)]
    unsigned pb[2][5][2];         // B fragments of the aggregation

    int slot = 0, phase = 0, it = 0, ti = 0, gs = 0;
    int n = 0, x0 = 0, y = 0;
    // kernel-wide strides in 32-bit words of the 16-bit output / attention tensors (two elements per word)
    const size_t plane_w = hi_plane >> 1;
    const int C = a.C, Wlo = a.W, Hlo = a.H;
    unsigned *o_ptr = nullptr;            // this lane's output word for the first channel of the current value stage
    bool row_ok = false, col_ok0 = false, col_ok1 = false;
    constexpr float LOG2E = 1.4426950408889634f;
    for (;; ++gs) {
        if (!mbar_wait_bounded(full_addr + 8 * slot, phase)) {
            atomicExch(&g_wait_timeout, 1);
            return;
        }
        if (it == 0) {
            int tile = tile_ids[ti & 3];      // published by the producer before the barrier's phase completed
            if (tile < 0) break;
            x0 = (tile % a.tiles_x) * h16::COLS; tile /= a.tiles_x;
            y = a.y_begin + (tile % a.tiles_y) * ROWS + wrow; tile /= a.tiles_y;
            n = tile;
            row_ok = y < a.y_end; col_ok0 = x0 + t < Wlo; col_ok1 = x0 + 4 + t < Wlo;
            o_ptr = reinterpret_cast<unsigned *>(static_cast<T *>(a.out) + ((size_t)n * C + g) * hi_plane +
                                                 (size_t)(2 * y + r) * sW + 2 * x0 + 2 * t);
#pragma unroll
            for (int p = 0; p < 2; ++p)
#pragma unroll
                for (int dy = 0; dy < 5; ++dy)
#pragma unroll
                    for (int i = 0; i < 4; ++i) s[p][dy][i] = 0.f;
        }
        if (MODE == MODE_AGG && it == 0) {      // the weights come from memory, already in the packed pair layout
            const unsigned *ap = static_cast<const unsigned *>(a.attn) +
                                 (((size_t)n * 25 * hi_plane + (size_t)(2 * y + r) * sW + 2 * x0 + 2 * t) >> 1);
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                const bool pix = row_ok && (p == 0 ? col_ok0 : col_ok1);
#pragma unroll
                for (int dy = 0; dy < 5; ++dy) {
                    unsigned ulo = 0u, uhi = 0u;
                    if (pix && ok_lo[p]) ulo = __ldg(ap + (size_t)(dy * 5 + dx_lo[p]) * plane_w + 4 * p);
                    if (pix && ok_hi[p]) uhi = __ldg(ap + (size_t)(dy * 5 + dx_lo[p] + 8) * plane_w + 4 * p);
                    pb[p][dy][0] = movmatrix_trans(ulo);
                    pb[p][dy][1] = movmatrix_trans(uhi);
                }
            }
        }
        const unsigned stage = ring_addr + slot * h16::SLOT_BYTES;

        if (it < nk) {
            // ------------------------------------------------------------- logits
#pragma unroll
            for (int ks = 0; ks < KCH / 16; ++ks) {
                unsigned qb[4];
                ldsm_x4_trans(qb, stage + q_off + ks * 16 * QROW);
                const unsigned ka_addr = stage + k_off + ks * 16 * KROW, kc_addr = stage + k_off2 + ks * 16 * KROW;
#pragma unroll
                for (int dy = 0; dy < 5; ++dy) {
                    unsigned ka[4], kc[2];
                    ldsm_x4_trans(ka, ka_addr + dy * (KCH * KROW));
                    ldsm_x2_trans(kc, kc_addr + dy * (KCH * KROW));
                    mma_h16<T>(s[0][dy], ka[0], ka[1], ka[2], ka[3], qb[0], qb[1]);
                    mma_h16<T>(s[1][dy], ka[1], kc[0], ka[3], kc[1], qb[2], qb[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_addr + 8 * slot);
            if (it == nk - 1 && MODE == MODE_BWD) {
                // softmax backward; the saved attention map is read and the logit gradients are written as 32-bit
                // pairs (the two pixels of a lane are neighbours in memory)
                const size_t poff = ((size_t)n * 25 * hi_plane + (size_t)(2 * y + r) * sW + 2 * x0 + 2 * t) >> 1;
                const unsigned *ap = static_cast<const unsigned *>(a.attn) + poff;
                unsigned *wp = static_cast<unsigned *>(a.ws) + poff;
#pragma unroll
                for (int p = 0; p < 2; ++p) {
                    const bool pix = row_ok && (p == 0 ? col_ok0 : col_ok1);
                    float av[5][4];
                    float d0 = 0.f, d1 = 0.f;
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy) {
                        unsigned ulo = 0u, uhi = 0u;
                        if (pix && ok_lo[p]) ulo = __ldg(ap + (size_t)(dy * 5 + dx_lo[p]) * plane_w + 4 * p);
                        if (pix && ok_hi[p]) uhi = __ldg(ap + (size_t)(dy * 5 + dx_lo[p] + 8) * plane_w + 4 * p);
                        const float2 flo = unpack_pair(T(), ulo), fhi = unpack_pair(T(), uhi);
                        av[dy][0] = flo.x; av[dy][1] = flo.y; av[dy][2] = fhi.x; av[dy][3] = fhi.y;
                        d0 += av[dy][0] * s[p][dy][0] + av[dy][2] * s[p][dy][2];
                        d1 += av[dy][1] * s[p][dy][1] + av[dy][3] * s[p][dy][3];
                    }
#pragma unroll
                    for (int sh = 4; sh < 32; sh <<= 1) {
                        d0 += __shfl_xor_sync(0xffffffffu, d0, sh);
                        d1 += __shfl_xor_sync(0xffffffffu, d1, sh);
                    }
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy) {
                        pb[p][dy][0] = pack_pair(T(), av[dy][0] * (s[p][dy][0] - d0), av[dy][1] * (s[p][dy][1] - d1));
                        pb[p][dy][1] = pack_pair(T(), av[dy][2] * (s[p][dy][2] - d0), av[dy][3] * (s[p][dy][3] - d1));
                        if (pix && ok_lo[p]) wp[(size_t)(dy * 5 + dx_lo[p]) * plane_w + 4 * p] = pb[p][dy][0];
                        if (pix && ok_hi[p]) wp[(size_t)(dy * 5 + dx_lo[p] + 8) * plane_w + 4 * p] = pb[p][dy][1];
                    }
                }
            }
            if (it == nk - 1 && MODE == MODE_FWD) {
                // softmax over the 25 window slots of each pixel: 5 rows here x the lanes with the same t.
                // exp(x - m) = 2^(x * log2(e) - m * log2(e)): one FMA and one ex2 per element.
#pragma unroll
                for (int p = 0; p < 2; ++p) {
                    float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy) {
                        if (ok_lo[p]) { m0 = fmaxf(m0, s[p][dy][0]); m1 = fmaxf(m1, s[p][dy][1]); }
                        if (ok_hi[p]) { m0 = fmaxf(m0, s[p][dy][2]); m1 = fmaxf(m1, s[p][dy][3]); }
                    }
#pragma unroll
                    for (int sh = 4; sh < 32; sh <<= 1) {
                        m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, sh));
                        m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, sh));
                    }
                    m0 *= LOG2E; m1 *= LOG2E;
                    float z0 = 0.f, z1 = 0.f;
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy) {
                        s[p][dy][0] = ok_lo[p] ? ex2_ftz(fmaf(s[p][dy][0], LOG2E, -m0)) : 0.f;
                        s[p][dy][1] = ok_lo[p] ? ex2_ftz(fmaf(s[p][dy][1], LOG2E, -m1)) : 0.f;
                        s[p][dy][2] = ok_hi[p] ? ex2_ftz(fmaf(s[p][dy][2], LOG2E, -m0)) : 0.f;
                        s[p][dy][3] = ok_hi[p] ? ex2_ftz(fmaf(s[p][dy][3], LOG2E, -m1)) : 0.f;
                        z0 += s[p][dy][0] + s[p][dy][2];
                        z1 += s[p][dy][1] + s[p][dy][3];
                    }
#pragma unroll
                    for (int sh = 4; sh < 32; sh <<= 1) {
                        z0 += __shfl_xor_sync(0xffffffffu, z0, sh);
                        z1 += __shfl_xor_sync(0xffffffffu, z1, sh);
                    }
                    const float i0 = __frcp_rn(z0), i1 = __frcp_rn(z1);
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy) {
                        pb[p][dy][0] = pack_pair(T(), s[p][dy][0] * i0, s[p][dy][1] * i1);
                        pb[p][dy][1] = pack_pair(T(), s[p][dy][2] * i0, s[p][dy][3] * i1);
                    }
                }
            }
            if (it == nk - 1 && MODE == MODE_SIM) {      // raw logits
#pragma unroll
                for (int p = 0; p < 2; ++p)
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy) {
                        pb[p][dy][0] = pack_pair(T(), s[p][dy][0], s[p][dy][1]);
                        pb[p][dy][1] = pack_pair(T(), s[p][dy][2], s[p][dy][3]);
                    }
            }
            if (it == nk - 1 && MODE == MODE_SIM && a.slots_f32 != 0) {
                if (row_ok) {         // raw logits as float32 pairs (the dense similarity of the 16-bit SAPA-D path)
                    float2 *af = reinterpret_cast<float2 *>(static_cast<float *>(a.attn) + (size_t)n * 25 * hi_plane +
                                                            (size_t)(2 * y + r) * sW + 2 * x0 + 2 * t);
#pragma unroll
                    for (int p = 0; p < 2; ++p)
                        if (p == 0 ? col_ok0 : col_ok1) {
#pragma unroll
                            for (int dy = 0; dy < 5; ++dy) {
                                if (ok_lo[p]) af[(size_t)(dy * 5 + dx_lo[p]) * plane_w + 4 * p] = make_float2(s[p][dy][0], s[p][dy][1]);
                                if (ok_hi[p]) af[(size_t)(dy * 5 + dx_lo[p] + 8) * plane_w + 4 * p] = make_float2(s[p][dy][2], s[p][dy][3]);
                            }
                        }
                }
            } else if (it == nk - 1 && (MODE == MODE_FWD || MODE == MODE_SIM)) {
                if (a.attn != nullptr && row_ok) {
                    // the two pixels of a pair are neighbours in memory: one 32-bit store per (window slot, pair)
                    unsigned *an = reinterpret_cast<unsigned *>(static_cast<T *>(a.attn) + (size_t)n * 25 * hi_plane +
                                                                (size_t)(2 * y + r) * sW + 2 * x0 + 2 * t);
#pragma unroll
                    for (int p = 0; p < 2; ++p)
                        if (p == 0 ? col_ok0 : col_ok1) {
#pragma unroll
                            for (int dy = 0; dy < 5; ++dy) {
                                if (ok_lo[p]) an[(size_t)(dy * 5 + dx_lo[p]) * plane_w + 4 * p] = pb[p][dy][0];
                                if (ok_hi[p]) an[(size_t)(dy * 5 + dx_lo[p] + 8) * plane_w + 4 * p] = pb[p][dy][1];
                            }
                        }
                }
            }
            if (it == nk - 1 && MODE != MODE_SIM) {
                // S^T accumulator fragments -> B fragments of the aggregation
#pragma unroll
                for (int p = 0; p < 2; ++p)
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy) {
                        pb[p][dy][0] = movmatrix_trans(pb[p][dy][0]);
                        pb[p][dy][1] = movmatrix_trans(pb[p][dy][1]);
                    }
            }
        } else {
            // ------------------------------------------------------------- aggregation
            float acc[VCH / 16][2][4];
#pragma unroll
            for (int b = 0; b < VCH / 16; ++b)
#pragma unroll
                for (int p = 0; p < 2; ++p)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[b][p][i] = 0.f;
            const unsigned va_addr = stage + v_off, vc_addr = stage + v_off2;
#pragma unroll
            for (int dy = 0; dy < 5; ++dy)
#pragma unroll
                for (int b = 0; b < VCH / 16; ++b) {
                    unsigned va[4], vc[2];
                    ldsm_x4(va, va_addr + dy * (VCH * KROW) + b * 16 * KROW);
                    ldsm_x2(vc, vc_addr + dy * (VCH * KROW) + b * 16 * KROW);
                    mma_h16<T>(acc[b][0], va[0], va[1], va[2], va[3], pb[0][dy][0], pb[0][dy][1]);
                    mma_h16<T>(acc[b][1], va[2], va[3], vc[0], vc[1], pb[1][dy][0], pb[1][dy][1]);
                }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_addr + 8 * slot);
            // D fragment of group p: d0,d1 = Out[ch g][px 8p+2t, +1], d2,d3 = Out[ch g+8][same].  Neighbouring lanes swap one
            // pair so that even lanes hold pixels 2t .. 2t+3 of the left group and odd lanes 2(t-1) .. 2(t-1)+3 of the right
            // group: a quad then writes one full 32-byte sector per store instruction (half sectors cost an L1 tag cycle each).
            const int c0 = (it - nk) * VCH;
            unsigned *o = o_ptr + ((t & 1) ? 3 : 0);
            o_ptr += (size_t)VCH * plane_w;
            if (row_ok) {          // warp-uniform; columns are always inside (W is a multiple of the tile width here)
                const bool odd = t & 1;
#pragma unroll
                for (int j = 0; j < VCH / 8; ++j) {       // channel g + 8j: block j/2, half j%2
                    const unsigned v0 = pack_pair(T(), acc[j >> 1][0][2 * (j & 1)], acc[j >> 1][0][2 * (j & 1) + 1]);
                    const unsigned v1 = pack_pair(T(), acc[j >> 1][1][2 * (j & 1)], acc[j >> 1][1][2 * (j & 1) + 1]);
                    const unsigned got = __shfl_xor_sync(0xffffffffu, odd ? v0 : v1, 1);
                    if (c0 + 8 * j + g < C) __stcs(reinterpret_cast<uint2 *>(o), odd ? make_uint2(got, v1) : make_uint2(v0, got));
                    o += 8 * plane_w;
                }
            }
        }
        if (++slot == h16::NSTAGE) { slot = 0; phase ^= 1; }
        if (++it == total) { it = 0; ++ti; }
    }
}

// ---------------------------------------------------------------------------------- host side
// one host-side counter for every kernel of this file: they all share g_next_tile / g_ctas_done, so two launches that
// may be in flight together (different streams, different kernels) must never get the same slot
static std::atomic<unsigned> g_next_sched_slot{0}, g_next_captured_slot{0};

// Opts in to the dynamic shared memory, sizes the persistent grid, picks a scheduler slot and launches.
template <typename Kernel, typename... Maps>
static int launch_persistent(Kernel kernel, const char *name, int threads, int smem, int ctas_per_sm, Args &a, cudaStream_t st,
                             const Maps &...maps) {
    const long long nblocks = (long long)a.B * a.tiles_x * a.tiles_y;
    if (nblocks > 0x7fffffffLL) {
        set_error("too many tiles");
        return SAPA_ERR_ARGUMENT;
    }
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
        set_error("%s: cudaFuncSetAttribute failed: %s", name, cudaGetErrorString(e));
        return SAPA_ERR_LAUNCH;
    }
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
        set_error("%s: cannot query the SM count", name);
        return SAPA_ERR_LAUNCH;
    }
    const long long resident = (long long)ctas_per_sm * sms;
    // persistent grid with dynamic tile claiming (static striding left SMs with 6 to 8 tiles instead of ~6.9)
    const unsigned grid = (unsigned)(nblocks < resident ? nblocks : resident);
    a.sched_slot = next_sched_slot(g_next_sched_slot, g_next_captured_slot, st);
    kernel<<<grid, threads, smem, st>>>(maps..., a);
    return check_launch(name);
}

}  // namespace tma

// K = 5, s = 2 and every row of every tensor on a 16-byte boundary
bool fused_tma_supported(int W, int dtype) {
    if (tma::encode_tiled_fn() == nullptr) return false;
    if (dtype == SAPA_F32) return W % 4 == 0;
    if (dtype == SAPA_F16 || dtype == SAPA_BF16) return W % 8 == 0;
    return false;
}

int launch_fused_tma_slots(int mode, const void *q, const void *k, const void *v, void *out, void *attn, void *ws, int B, int d,
                           int C, int H, int W, int rows, int ytop0, int y_begin, int y_end, int dtype, bool slots_f32,
                           cudaStream_t st);

// Returns SAPA_ERR_UNSUPPORTED when a tensor map cannot be built (the caller then uses another kernel).
// mode 0 (forward): out = atn(softmax(sim(q, k)), v), attn = optional output.
// mode 1 (backward stage 1): q = grad_out [B,d,2H,2W], k = value [B,d,H,W] (d = value channels), v = key [B,C,H,W]
//        (C = key channels), attn = saved attention map (input), ws = logit gradients (output), out = grad_query.
// mode 2 (sim): attn (output) = sim(q, k); v, out unused, C ignored.   mode 3 (agg): out = atn(attn (input), v); q, k unused, d ignored.
int launch_fused_tma(int mode, const void *q, const void *k, const void *v, void *out, void *attn, void *ws, int B, int d, int C,
                     int H, int W, int rows, int ytop0, int y_begin, int y_end, int dtype, cudaStream_t st) {
    return launch_fused_tma_slots(mode, q, k, v, out, attn, ws, B, d, C, H, W, rows, ytop0, y_begin, y_end, dtype, false, st);
}

// slots_f32 (16-bit tensors, mode 2 only): `attn` is a float32 tensor - the logits are written at full precision while
// query and key stay 16-bit.
int launch_fused_tma_slots(int mode, const void *q, const void *k, const void *v, void *out, void *attn, void *ws, int B, int d,
                           int C, int H, int W, int rows, int ytop0, int y_begin, int y_end, int dtype, bool slots_f32,
                           cudaStream_t st) {
    using namespace tma;
    if (slots_f32 && (dtype == SAPA_F32 || mode != MODE_SIM)) {
        set_error("sapa_tma_fused: float32 slots are for the 16-bit logit mode");
        return SAPA_ERR_UNSUPPORTED;
    }
    if (mode == MODE_SIM) C = 0;
    if (mode == MODE_AGG) d = 0;
    const bool use_qk = mode != MODE_AGG, use_v = mode != MODE_SIM;
    CUtensorMap qmap, kmap, vmap, omap;
    bool ok = true;
    if (dtype == SAPA_F32) {
        const auto ty = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
        const auto sw = CU_TENSOR_MAP_SWIZZLE_64B;
        if (use_qk) ok = ok && make_nchw_map(&qmap, q, 2 * W, 2 * H, d, B, HC, F_KCH, HH, ty, 4, sw) && make_nchw_map(&kmap, k, W, rows, d, B, HC, F_KCH, HH, ty, 4, sw);
        if (use_v) ok = ok && make_nchw_map(&vmap, v, W, rows, C, B, HC, F_VCH, HH, ty, 4, sw) && make_nchw_map(&omap, out, 2 * W, 2 * H, C, B, HC, F_VCH, HH, ty, 4, sw);
    } else {
        const auto ty = dtype == SAPA_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
        if (use_qk) ok = ok && make_nchw_map(&qmap, q, 2 * W, 2 * H, d, B, 16, h16::KCH, HH, ty, 2, CU_TENSOR_MAP_SWIZZLE_32B) &&
                         make_nchw_map(&kmap, k, W, rows, d, B, h16::BC, h16::KCH, HH, ty, 2, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (use_v) ok = ok && make_nchw_map(&vmap, v, W, rows, C, B, h16::BC, h16::VCH, HH, ty, 2, CU_TENSOR_MAP_SWIZZLE_NONE);
    }
    if (!ok) {
        set_error("sapa_tma_fused (mode %d): cuTensorMapEncodeTiled rejected the tensor layout (CUresult %d)", mode,
                  last_encode_result());
        return SAPA_ERR_UNSUPPORTED;
    }
    // maps a mode never touches still travel as kernel parameters: give them defined contents
    if (!use_qk) { qmap = vmap; kmap = vmap; }
    if (!use_v) { vmap = kmap; omap = kmap; }
    if (dtype != SAPA_F32) omap = vmap;
    Args a{};
    a.out = out; a.attn = attn; a.ws = ws;
    a.B = B; a.d = d; a.C = C; a.H = H; a.W = W; a.rows = rows; a.ytop0 = ytop0;
    a.slots_f32 = slots_f32 ? 1 : 0;
    static_assert(h16::COLS == COLS, "both kernels use the same tile");
    a.y_begin = y_begin; a.y_end = y_end;
    a.tiles_x = ceil_div(W, COLS);
    a.tiles_y = ceil_div(y_end - y_begin, ROWS);
    constexpr int smem32 = NSTAGE * SLOT_BYTES + 2 * O_BYTES + 1024;
    static const char *const names32[4] = {"sapa_tma_fused_f32_kernel<fwd>", "sapa_tma_fused_f32_kernel<bwd>",
                                           "sapa_tma_fused_f32_kernel<sim>", "sapa_tma_fused_f32_kernel<agg>"};
    static const char *const names16[4] = {"sapa_tma_fused_16_kernel<fwd>", "sapa_tma_fused_16_kernel<bwd>",
                                           "sapa_tma_fused_16_kernel<sim>", "sapa_tma_fused_16_kernel<agg>"};
    const char *n32 = names32[mode & 3], *n16 = names16[mode & 3];
#define SAPA_TMA_LAUNCH32(M) launch_persistent(sapa_tma_fused_f32_kernel<M>, n32, NT, smem32, CTAS_PER_SM, a, st, qmap, kmap, vmap, omap)
#define SAPA_TMA_LAUNCH16(T, M) \
    launch_persistent(sapa_tma_fused_16_kernel<T, M>, n16, h16::NT, h16::SMEM_BYTES, h16::CTAS_PER_SM, a, st, qmap, kmap, vmap)
    if (dtype == SAPA_F32) {
        switch (mode) {
            case MODE_FWD: return SAPA_TMA_LAUNCH32(MODE_FWD);
            case MODE_BWD: return SAPA_TMA_LAUNCH32(MODE_BWD);
            case MODE_SIM: return SAPA_TMA_LAUNCH32(MODE_SIM);
            default: return SAPA_TMA_LAUNCH32(MODE_AGG);
        }
    }
    if (dtype == SAPA_F16) {
        switch (mode) {
            case MODE_FWD: return SAPA_TMA_LAUNCH16(__half, MODE_FWD);
            case MODE_BWD: return SAPA_TMA_LAUNCH16(__half, MODE_BWD);
            case MODE_SIM: return SAPA_TMA_LAUNCH16(__half, MODE_SIM);
            default: return SAPA_TMA_LAUNCH16(__half, MODE_AGG);
        }
    }
    switch (mode) {
        case MODE_FWD: return SAPA_TMA_LAUNCH16(__nv_bfloat16, MODE_FWD);
        case MODE_BWD: return SAPA_TMA_LAUNCH16(__nv_bfloat16, MODE_BWD);
        case MODE_SIM: return SAPA_TMA_LAUNCH16(__nv_bfloat16, MODE_SIM);
        default: return SAPA_TMA_LAUNCH16(__nv_bfloat16, MODE_AGG);
    }
#undef SAPA_TMA_LAUNCH32
#undef SAPA_TMA_LAUNCH16
}

// One CTA waits, with a short limit, on a shared-memory barrier that nothing ever signals: the bounded wait gives up,
// the kernel raises g_wait_timeout exactly as the production kernels would and returns normally.
__global__ void sapa_wait_selftest_kernel(int tries) {
    __shared__ __align__(8) unsigned long long bar;
    const unsigned addr = (unsigned)__cvta_generic_to_shared(&bar);
    if (threadIdx.x == 0) {
        tmau::mbar_init(addr, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        bool done = false;
        for (int i = 0; i < tries && !done; ++i) done = tmau::mbar_try_wait(addr, 0);
        if (!done) atomicExch(&tma::g_wait_timeout, 1);
    }
}

int launch_wait_selftest(cudaStream_t st) {
    sapa_wait_selftest_kernel<<<1, 32, 0, st>>>(64);
    return check_launch("sapa_wait_selftest_kernel");
}

// 1 if a bounded mbarrier wait of the TMA kernels gave up on the current device since the last query (synchronises the
// device).  A CTA that gives up leaves without taking part in the last-CTA reset of its scheduler pair, so a raised
// flag also means that pair may be dirty: reading a raised flag clears it and zeroes every scheduler pair.
int tma_wait_timeout_flag() {
    int flag = 0;
    if (cudaMemcpyFromSymbol(&flag, tma::g_wait_timeout, sizeof(int)) != cudaSuccess) return -1;
    if (flag != 0) {
        static const unsigned zeros[tmau::SCHED_SLOTS] = {};
        const int zero = 0;
        if (cudaMemcpyToSymbol(tma::g_next_tile, zeros, sizeof(zeros)) != cudaSuccess ||
            cudaMemcpyToSymbol(tma::g_ctas_done, zeros, sizeof(zeros)) != cudaSuccess ||
            cudaMemcpyToSymbol(tma::g_wait_timeout, &zero, sizeof(int)) != cudaSuccess)
            return -1;
    }
    return flag;
}

}  // namespace sapa
