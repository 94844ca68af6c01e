// sapa_gath_mma.cu — the transposed aggregation ("gath") of SAPA-B on the tensor cores, K = 5, s = 2:
//
//     G[c][u] = sum over high-res pixels p and window slots k with win_k(p) = u of  X[c][p] * Wt[k][p]
//
// which is dV = gath(dOut, A) and dKey = gath(Q, dS) of the backward pass (the reference scatters these with
// atomics, av_cuda_kernel.cu:103-148 and qk_cuda_kernel.cu:101-137).  Gather form: a CTA owns 4 x 8 low-res output
// cells and reads every high-res pixel whose window reaches them, so the result is deterministic.
//
// As a matrix product, per output row y and 16 channels:   G[16 ch][8 cols] += X[16 ch][8 px] * W[8 px][8 cols]
// for each of the 10 high-res rows (parents y-2 .. y+2) and 3 groups of 8 pixels (parents x0-2 .. x0+9) that
// touch the 8 columns; W[p][u] = Wt[slot(p, u)][p] is banded (42 % non-zero).  One m16n8k8 per block: tf32 with the
// 3-term split for float32 (hi*hi + lo*hi + hi*lo), f16 / bf16 natively.
//   * W does not depend on the channel: each warp loads its 15 B fragments (5 parent rows x 3 pixel groups) from
//     the weight tensor ONCE per tile and keeps them in registers while the channels stream by;
//   * X comes through a TMA ring (box = 32 px x 16 (float32) or 32 (16-bit) channels x 16 high-res rows, starting at pixel 2*x0 - 8 so that
//     rows begin on a 32-byte boundary; zero fill outside the image); swizzled rows make the per-lane fragment
//     loads bank-conflict-free;
//   * warp = (output row, upper / lower high-res row of the parents): the two warps of a row add their partial
//     sums through shared memory (an mbarrier handshake per pair and stage), nothing is CTA-wide in the steady state;
//   * ring protocol: full / empty mbarriers, one lane of a ninth, producer-only warp refills a slot as soon as all 8 warps released it;
//     every wait is bounded and raises g_wait_timeout instead of spinning for ever.
#include "tma_util.cuh"

#include <atomic>

namespace sapa {

namespace gmma {

using namespace tmau;

constexpr int ROWS = 4, COLS = 8;          // low-res output tile of a CTA
constexpr int HR = 2 * (ROWS + 4);         // high-res rows per box
constexpr int BPX = 32;                    // high-res pixels per box row: 2*x0-8 .. 2*x0+23 (used: 4 .. 27)
constexpr int NSTAGE = 3;                  // ring slots of 32 KB
constexpr int NW = 2 * ROWS;               // 8 consumer warps
constexpr int NT = (NW + 1) * 32;          // + one producer warp
constexpr int CTAS_PER_SM = 2;

__device__ int g_wait_timeout = 0;
__device__ unsigned g_next_tile[SCHED_SLOTS];
__device__ unsigned g_ctas_done[SCHED_SLOTS];

struct Args {
    const void *wt;        // [B, 25, 2H, 2W] window weights (attention map or logit gradients)
    void *out;             // [B, C, top + H + bottom, W]
    int B, C, H, W;        // H = low-res rows covered by the high-res inputs
    int top, Hout;         // row-slab form: the output has `top` extra rows above and Hout = top + H + bottom rows in all
                           // (the cells of the neighbouring slabs that this slab's pixels reach); 0 and H otherwise
    int tiles_x, tiles_y;
    int sched_slot;
};

template <typename T>
__device__ __forceinline__ void mma_16_k8(float (&d)[4], unsigned a0, unsigned a1, unsigned b0) {
    if constexpr (std::is_same<T, __half>::value)
        asm("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};\n"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(b0));
    else
        asm("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};\n"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(b0));
}
template <typename T> struct Geo {
    static constexpr int ES = (int)sizeof(T);
    static constexpr int ROWB = BPX * ES;                    // 128 bytes (float32, 128-byte swizzle) or 64 (64-byte swizzle)
    static constexpr int NB = ES == 4 ? 1 : 2;               // m blocks of 16 channels per stage (per-stage overhead dominates the
    static constexpr int NCH = 16 * NB;                      //   16-bit kernel with its single MMA per block: it takes two)
    static constexpr int BOX_BYTES = HR * NCH * ROWB;        // 32768
    static constexpr int SMEM_BYTES = NSTAGE * BOX_BYTES + 1024;
};
// byte offset of pixel `px` in the row of channel `ch` (rows are channel-minor: the row index modulo 8 is ch & 7)
template <typename T> __device__ __forceinline__ int px_off(int px, int ch) {
    if constexpr (sizeof(T) == 4) return ((((px >> 2) ^ ch) & 7) << 4) | ((px & 3) << 2);                    // 128-byte swizzle
    else                          return ((((px >> 3) ^ (ch >> 1)) & 3) << 4) | ((px & 7) << 1);             // 64-byte swizzle
}

template <typename T>
__global__ void __launch_bounds__(NT, CTAS_PER_SM)
sapa_gath_mma_kernel(const __grid_constant__ CUtensorMap xmap, const Args a) {
    using G = Geo<T>;
    constexpr bool F32 = sizeof(T) == 4;
    constexpr int NB = G::NB, NCH = G::NCH;
    extern __shared__ unsigned char smem_dyn[];
    // exchange buffers: the even-row warp releases a ring slot only after it has read its partner's sums of that stage,
    // so the partner is never more than NSTAGE - 1 stages ahead of an unread buffer
    constexpr int NX = NSTAGE;
    __shared__ __align__(8) unsigned long long bars[2 * NSTAGE + ROWS * NX];   // full[NSTAGE], empty[NSTAGE], pair[ROWS][NX]
    __shared__ int tile_ids[8];      // ring of claimed tiles: the producer is at most NSTAGE (< 8) tiles ahead
    __shared__ __align__(16) float xch[NX][ROWS][NB][32][4];           // partial sums of the odd-row warps
    const unsigned ring_addr = ((unsigned)__cvta_generic_to_shared(smem_dyn) + 1023u) & ~1023u;
    const unsigned full_addr = (unsigned)__cvta_generic_to_shared(bars), empty_addr = full_addr + 8 * NSTAGE;
    const unsigned pair_addr = empty_addr + 8 * NSTAGE;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wy = warp >> 1, r = warp & 1;        // output row of the tile, high-res row of each parent
    const int g = lane >> 2, t = lane & 3;
    const int sH = 2 * a.H, sW = 2 * a.W;
    const size_t hi_plane = (size_t)sH * sW;
    const int nst = (a.C + NCH - 1) / NCH;         // stages per tile
    const int ntiles = a.B * a.tiles_x * a.tiles_y;

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < NSTAGE; ++i) {
            mbar_init(full_addr + 8 * i, 1);
            mbar_init(empty_addr + 8 * i, NW);
        }
#pragma unroll
        for (int i = 0; i < ROWS * NX; ++i) mbar_init(pair_addr + 8 * i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    // ---- producer state (lane 0 of the producer warp): the stages of successive tiles form one stream through the ring
    int p_issued = 0, p_slot = 0, p_phase = 0, p_it = 0, p_ti = 0, p_n = 0, p_x0 = 0, p_y0 = 0;
    bool p_done = false;
    auto produce = [&](int need) {
        while (!p_done) {
            const unsigned ebar = empty_addr + 8 * p_slot;
            if (!mbar_test_wait(ebar, p_phase ^ 1)) {      // slot still in use (a fresh barrier passes at once)
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
                tile_ids[p_ti & 7] = claimed;
                if (claimed < 0) {
                    mbar_arrive(bar);          // completes the phase without data: the warps read -1 and stop
                    if (atomicAdd(&g_ctas_done[a.sched_slot], 1u) == gridDim.x - 1) {
                        g_next_tile[a.sched_slot] = 0u;
                        g_ctas_done[a.sched_slot] = 0u;
                    }
                    p_done = true;
                    return;
                }
                p_x0 = (claimed % a.tiles_x) * COLS; claimed /= a.tiles_x;
                p_y0 = (claimed % a.tiles_y) * ROWS; claimed /= a.tiles_y;
                p_n = claimed;
            }
            mbar_expect_tx(bar, G::BOX_BYTES);
            tma_load_4d(ring_addr + p_slot * G::BOX_BYTES, &xmap, bar, 2 * p_x0 - 8, p_it * NCH, 2 * (p_y0 - a.top - 2), p_n);
            ++p_issued;
            if (++p_it == nst) { p_it = 0; ++p_ti; }
            if (++p_slot == NSTAGE) { p_slot = 0; p_phase ^= 1; }
        }
    };

    // The producer is a warp of its own (one lane works): inside a consumer warp it took a quarter of that warp's time
    // and the other warps waited a third of theirs for stages it had not issued yet.
    if (warp == NW) {
        if (lane == 0) produce(0x7fffffff);
        return;
    }

    // ---- per-lane fragment offsets.  Pixel group kg covers box pixels 4 + 8*kg .. 11 + 8*kg.
    //   float32 A fragment: a0 = X[ch g][px t], a1 = X[ch g+8][px t], a2 = X[ch g][px t+4], a3 = X[ch g+8][px t+4]
    //   16-bit  A fragment: a0 = X[ch g][px 2t, 2t+1], a1 = X[ch g+8][same]
    int a_off[3][2];
#pragma unroll
    for (int kg = 0; kg < 3; ++kg) {
        if constexpr (F32) {
            a_off[kg][0] = g * G::ROWB + px_off<T>(4 + 8 * kg + t, g);
            a_off[kg][1] = g * G::ROWB + px_off<T>(8 + 8 * kg + t, g);
        } else {
            a_off[kg][0] = g * G::ROWB + px_off<T>(4 + 8 * kg + 2 * t, g);
            a_off[kg][1] = 0;
        }
    }

    // B fragments of the tile: W[px][col g] for the 5 parent rows x 3 pixel groups of this warp
    //   float32: bw[j][kg][0] = W[px t], [1] = W[px t+4];  16-bit: bw[j][kg][0] = packed W[px 2t, 2t+1]
    unsigned bw[5][3][F32 ? 2 : 1];

    int slot = 0, phase = 0, it = 0, ti = 0, gs = 0;
    int n = 0, x0 = 0, y = 0;
    T *o_ptr = nullptr;
    bool store_ok = false;
    for (;; ++gs) {
        if (!mbar_wait_bounded(full_addr + 8 * slot, phase)) {
            atomicExch(&g_wait_timeout, 1);
            return;
        }
        if (it == 0) {
            int tile = tile_ids[ti & 7];      // published by the producer before the barrier's phase completed
            if (tile < 0) break;
            x0 = (tile % a.tiles_x) * COLS; tile /= a.tiles_x;
            const int y0 = (tile % a.tiles_y) * ROWS; tile /= a.tiles_y;
            n = tile;
            y = y0 + wy;                  // output row in the (padded) output frame; the input frame is `top` rows further up
            store_ok = y < a.Hout && x0 + 2 * t < a.W;
            o_ptr = static_cast<T *>(a.out) + ((size_t)n * a.C + g) * a.Hout * a.W + (size_t)y * a.W + x0 + 2 * t;
            // weights of the tile: parent row yp = y - 2 + j uses window row 4 - j; the parent of box pixel b is
            // x0 - 4 + b/2 and reaches column x0 + g through window column g + 6 - b/2
            const T *wimg = static_cast<const T *>(a.wt) + (size_t)n * 25 * hi_plane;
#pragma unroll
            for (int j = 0; j < 5; ++j) {
                const int yp = y - a.top - 2 + j, hy = 2 * yp + r;
                const bool row_in = yp >= 0 && yp < a.H && y < a.Hout && x0 + g < a.W;
#pragma unroll
                for (int kg = 0; kg < 3; ++kg) {
                    if constexpr (F32) {
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int b = 4 + 8 * kg + t + 4 * e, dx = g + 6 - (b >> 1), hx = 2 * x0 - 8 + b;
                            float w = 0.f;
                            if (row_in && dx >= 0 && dx <= 4 && hx >= 0 && hx < sW)
                                w = __ldg(reinterpret_cast<const float *>(wimg) + (size_t)((4 - j) * 5 + dx) * hi_plane + (size_t)hy * sW + hx);
                            bw[j][kg][e] = __float_as_uint(w);
                        }
                    } else {
                        const int b = 4 + 8 * kg + 2 * t, dx = g + 6 - (b >> 1), hx = 2 * x0 - 8 + b;
                        unsigned w = 0u;
                        if (row_in && dx >= 0 && dx <= 4 && hx >= 0 && hx < sW)
                            w = __ldg(reinterpret_cast<const unsigned *>(wimg + (size_t)((4 - j) * 5 + dx) * hi_plane + (size_t)hy * sW + hx));
                        bw[j][kg][0] = w;
                    }
                }
            }
        }
        const unsigned stage = ring_addr + slot * G::BOX_BYTES + (2 * wy + r) * (NCH * G::ROWB);

        // one accumulator per parent row and m block: five (ten) independent MMA chains
        float acc[NB][5][4];
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int j = 0; j < 5; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[b][j][i] = 0.f;
#pragma unroll
        for (int j = 0; j < 5; ++j) {
#pragma unroll
            for (int kg = 0; kg < 3; ++kg) {
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    const unsigned row = stage + 2 * j * (NCH * G::ROWB) + b * 16 * G::ROWB;
                    if constexpr (F32) {
                        unsigned ah[4], al[4];
                        ah[0] = lds32(row + a_off[kg][0]);
                        ah[1] = lds32(row + a_off[kg][0] + 8 * G::ROWB);
                        ah[2] = lds32(row + a_off[kg][1]);
                        ah[3] = lds32(row + a_off[kg][1] + 8 * G::ROWB);
#pragma unroll
                        for (int i = 0; i < 4; ++i) al[i] = tf32_lo(ah[i]);
                        mma_tf32(acc[b][j], ah, bw[j][kg][0], bw[j][kg][1]);
                        mma_tf32(acc[b][j], al, bw[j][kg][0], bw[j][kg][1]);
                        mma_tf32(acc[b][j], ah, tf32_lo(bw[j][kg][0]), tf32_lo(bw[j][kg][1]));
                    } else {
                        const unsigned a0 = lds32(row + a_off[kg][0]), a1 = lds32(row + a_off[kg][0] + 8 * G::ROWB);
                        mma_16_k8<T>(acc[b][j], a0, a1, bw[j][kg][0]);
                    }
                }
            }
        }
        __syncwarp();
        if (r == 1 && lane == 0) mbar_arrive(empty_addr + 8 * slot);
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[b][0][i] += (acc[b][1][i] + acc[b][2][i]) + (acc[b][3][i] + acc[b][4][i]);

        // The odd-row warp hands its sums to the even-row warp of the same output row through one of NX buffers,
        // each with its own mbarrier (one arrival per use, so use number u of a buffer completes its phase u).
        const int xi = gs % NX;
        const unsigned pbar = pair_addr + 8 * (wy * NX + xi);
        if (r == 1) {
#pragma unroll
            for (int b = 0; b < NB; ++b)
                *reinterpret_cast<float4 *>(&xch[xi][wy][b][lane][0]) = make_float4(acc[b][0][0], acc[b][0][1], acc[b][0][2], acc[b][0][3]);
            __syncwarp();
            if (lane == 0) mbar_arrive(pbar);
        } else {
            if (!mbar_wait_bounded(pbar, (gs / NX) & 1)) {
                atomicExch(&g_wait_timeout, 1);
                return;
            }
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                const float4 o4 = *reinterpret_cast<const float4 *>(&xch[xi][wy][b][lane][0]);
                acc[b][0][0] += o4.x; acc[b][0][1] += o4.y; acc[b][0][2] += o4.z; acc[b][0][3] += o4.w;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_addr + 8 * slot);
            // D fragment: d0,d1 = G[ch g][cols 2t, 2t+1], d2,d3 = G[ch g+8][same]
            const int c0 = it * NCH;
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                if (store_ok) {
                    T *o = o_ptr + (size_t)(c0 + 16 * b) * a.Hout * a.W;
#pragma unroll
                    for (int half = 0; half < 2; ++half)
                        if (c0 + 16 * b + 8 * half + g < a.C) {
                            T *oh = o + (size_t)(8 * half) * a.Hout * a.W;
                            if constexpr (F32) *reinterpret_cast<float2 *>(oh) = make_float2(acc[b][0][2 * half], acc[b][0][2 * half + 1]);
                            else *reinterpret_cast<unsigned *>(oh) = pack_pair(T(), acc[b][0][2 * half], acc[b][0][2 * half + 1]);
                        }
                }
            }
        }
        if (++slot == NSTAGE) { slot = 0; phase ^= 1; }
        if (++it == nst) { it = 0; ++ti; }
    }
}

// ---------------------------------------------------------------------------------- host side
// one host-side counter for all element types: they share g_next_tile / g_ctas_done
static std::atomic<unsigned> g_next_sched_slot{0}, g_next_captured_slot{0};

template <typename T>
static int launch(const void *hi, const void *wt, void *out, int B, int C, int H, int W, int top, int bottom, cudaStream_t st) {
    using G = Geo<T>;
    const char *name = "sapa_gath_mma_kernel";
    CUtensorMap xmap;
    const CUtensorMapDataType ty = sizeof(T) == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const CUtensorMapSwizzle sw = sizeof(T) == 4 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    if (encode_tiled_fn() == nullptr) return SAPA_ERR_UNSUPPORTED;
    if (!make_nchw_map(&xmap, hi, 2 * W, 2 * H, C, B, BPX, G::NCH, HR, ty, G::ES, sw)) {
        set_error("%s: cuTensorMapEncodeTiled rejected the tensor layout", name);
        return SAPA_ERR_UNSUPPORTED;
    }
    Args a{};
    a.wt = wt; a.out = out; a.B = B; a.C = C; a.H = H; a.W = W; a.top = top; a.Hout = top + H + bottom;
    a.tiles_x = ceil_div(W, COLS);
    a.tiles_y = ceil_div(a.Hout, ROWS);
    const long long nblocks = (long long)B * a.tiles_x * a.tiles_y;
    if (nblocks > 0x7fffffffLL) {
        set_error("too many tiles");
        return SAPA_ERR_ARGUMENT;
    }
    const cudaError_t e = cudaFuncSetAttribute(sapa_gath_mma_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM_BYTES);
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
    const unsigned grid = (unsigned)(nblocks < resident ? nblocks : resident);
    a.sched_slot = next_sched_slot(g_next_sched_slot, g_next_captured_slot, st);
    sapa_gath_mma_kernel<T><<<grid, NT, G::SMEM_BYTES, st>>>(xmap, a);
    return check_launch(name);
}

}  // namespace gmma

// K = 5, s = 2; every high-res row on a 16-byte boundary and low-res rows of even length (paired stores)
bool gath_mma_supported(int W, int dtype) {
    if (gmma::encode_tiled_fn() == nullptr) return false;
    if (dtype == SAPA_F32) return W % 2 == 0;
    if (dtype == SAPA_F16 || dtype == SAPA_BF16) return W % 4 == 0;
    return false;
}

// Returns SAPA_ERR_UNSUPPORTED when the tensor map cannot be built (the caller then uses the FP32-pipe kernel).
// `top` / `bottom`: extra output rows above / below the H rows under the inputs (row-slab backward), 0 otherwise.
int launch_gath_mma(const void *hi, const void *wt, void *out, int B, int C, int H, int W, int top, int bottom, int dtype,
                    cudaStream_t st) {
    if (dtype == SAPA_F32) return gmma::launch<float>(hi, wt, out, B, C, H, W, top, bottom, st);
    if (dtype == SAPA_F16) return gmma::launch<__half>(hi, wt, out, B, C, H, W, top, bottom, st);
    if (dtype == SAPA_BF16) return gmma::launch<__nv_bfloat16>(hi, wt, out, B, C, H, W, top, bottom, st);
    return SAPA_ERR_UNSUPPORTED;
}

// 1 if a bounded mbarrier wait of the gather kernel gave up on the current device since the last query (synchronises
// the device); reading a raised flag clears it and zeroes every scheduler pair (a CTA that gave up skipped the
// last-CTA reset of its pair).
int gath_wait_timeout_flag() {
    int flag = 0;
    if (cudaMemcpyFromSymbol(&flag, gmma::g_wait_timeout, sizeof(int)) != cudaSuccess) return -1;
    if (flag != 0) {
        static const unsigned zeros[tmau::SCHED_SLOTS] = {};
        const int zero = 0;
        if (cudaMemcpyToSymbol(gmma::g_next_tile, zeros, sizeof(zeros)) != cudaSuccess ||
            cudaMemcpyToSymbol(gmma::g_ctas_done, zeros, sizeof(zeros)) != cudaSuccess ||
            cudaMemcpyToSymbol(gmma::g_wait_timeout, &zero, sizeof(int)) != cudaSuccess)
            return -1;
    }
    return flag;
}

}  // namespace sapa
