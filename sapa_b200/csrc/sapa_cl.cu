// sapa_cl.cu — float32 fused forward of SAPA-B for K = 5, s = 2: logits on the tensor cores, aggregation on the FP32
// pipe with one lane per value channel.
//
// Why a second float32 kernel.  The aggregation is 80 % of the arithmetic.  Through 3 x tf32 warp-level MMAs it
// is bound by the MMA issue path (the kernel of sapa_tma.cu spends its whole time there); on the FP32 pipe with one
// thread per pixel it is bound by shared-memory wavefronts (one load per four FMAs).  Here the roles are swapped:
//   * a lane owns value CHANNELS (4 of them) and keeps their 5 x 6 low-res window patch in registers, sliding down
//     the tile one halo row per step (each value element is read from shared memory once per tile);
//   * the 25 x 4 softmax weights of a low-res parent (its 2 x 2 high-res pixels) do not depend on the channel, so a
//     128-bit shared-memory load of them is a broadcast to the eight lanes that share the parent and feeds 16 FMAs.
// That is one shared-memory wavefront per ~6 FMA instructions instead of one per 4 FMAs per lane.
//
// Tile = 4 x 8 low-res pixels (8 x 16 high-res).  Per tile:
//   1. logits: key / query stages of 16 channels stream through a ring of 4 slots (TMA boxes [8 rows][16 ch][16 cols],
//      64-byte swizzle); S[16 px][8 cells] += Q^T K per window row as 3 x tf32 m16n8k8, softmax across the quad;
//   2. the probabilities go to shared memory as W[parent row][slot][parent parity][column pair][2 x 2 pixel];
//   3. aggregation: warp w owns value channels 32w .. 32w+31, which arrive as ONE TMA box [8 rows][32 ch][16 cols] in
//      the warp's own slot; lane = (column pair xb, channel c8) handles channels c8 + 8i (i < 4) of low-res columns
//      2xb, 2xb+1 and writes 16-byte row segments straight from registers.
// Values outside the image are zero-filled by the TMA unit (the reference's border rule: logit 0, weight kept, value
// 0).  Every barrier wait is bounded and raises a device flag instead of spinning for ever.
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
constexpr int VCH = 32;                      // value channels per warp and box
constexpr int NKQ = 4;                       // ring slots for key / query stages
constexpr int NW = 8;                        // warps; warp w also owns value slot NKQ + w
constexpr int NT = NW * 32;
constexpr int K_BYTES = HH * KCH * ROWB;     // 8192: key box; the query box of the same stage follows it
constexpr int SLOT_BYTES = HH * VCH * ROWB;  // 16384 = key box + query box = one value box
static_assert(2 * K_BYTES == SLOT_BYTES, "a key/query stage and a value box share the slot size");
constexpr int W_FLOATS = ROWS * 25 * 2 * 4 * 4;   // probabilities of one tile
constexpr int SMEM_BYTES = (NKQ + NW) * SLOT_BYTES + W_FLOATS * 4 + 1024;

__device__ int g_wait_timeout = 0;
__device__ unsigned g_next_tile[SCHED_SLOTS];
__device__ unsigned g_ctas_done[SCHED_SLOTS];

struct Args {
    float *out, *attn;     // attn: optional softmax output [B, 25, 2H, 2W]
    int B, d, C, H, W;
    int rows, ytop0;       // key / value tensors hold `rows` rows; output row 0 reads from row ytop0 - 2 on
    int tiles_x, tiles_y;
    int sched_slot;
};

__device__ __forceinline__ int swz(int col, int channel) { return ((((col >> 2) ^ (channel >> 1)) & 3) << 4) | ((col & 3) << 2); }

__device__ __forceinline__ void lds64(unsigned addr, float &a, float &b) {
    asm("ld.shared.v2.f32 {%0, %1}, [%2];\n" : "=f"(a), "=f"(b) : "r"(addr));
}
__device__ __forceinline__ float4 lds128(unsigned addr) {
    float4 v;
    asm("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}

__global__ void __launch_bounds__(NT, 1)
sapa_cl_fused_f32_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                         const __grid_constant__ CUtensorMap vmap, const Args a) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) unsigned long long full_bar[NKQ + NW];
    __shared__ int tile_ids[4];       // tile_ids[ti & 3] = tile of the ti-th tile of this CTA, -1 = none
    const unsigned ring_addr = ((unsigned)__cvta_generic_to_shared(smem_dyn) + 1023u) & ~1023u;
    const unsigned bar_addr = (unsigned)__cvta_generic_to_shared(full_bar);
    const unsigned w_addr = ring_addr + (NKQ + NW) * SLOT_BYTES;
    float *wbuf = reinterpret_cast<float *>(smem_dyn + (ring_addr - (unsigned)__cvta_generic_to_shared(smem_dyn)) +
                                            (NKQ + NW) * SLOT_BYTES);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sW = 2 * a.W;
    const size_t hi_plane = (size_t)(2 * a.H) * sW;
    const int nk = (a.d + KCH - 1) / KCH, nv = (a.C + VCH - 1) / VCH, nrounds = (nv + NW - 1) / NW;
    const int ntiles = a.B * a.tiles_x * a.tiles_y;

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < NKQ + NW; ++i) mbar_init(bar_addr + 8 * i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    // ---- producer (thread 0).  Key / query stages of successive tiles form one stream through slots 0 .. NKQ-1; the
    // first tile of a CTA is blockIdx.x, further tiles come from a global counter.
    bool exhausted = false;
    int p_it = 0, p_ti = 0, p_slot = 0, p_n = 0, p_x0 = 0, p_y0 = 0;
    auto issue_kq = [&]() {
        if (exhausted) return;
        if (p_it == 0) {
            int claimed = (int)blockIdx.x;
            if (p_ti > 0) claimed = (int)(atomicAdd(&g_next_tile[a.sched_slot], 1u) + gridDim.x);
            if (claimed >= ntiles) claimed = -1;
            tile_ids[p_ti & 3] = claimed;
            if (claimed < 0) { exhausted = true; return; }
            p_x0 = (claimed % a.tiles_x) * COLS; claimed /= a.tiles_x;
            p_y0 = (claimed % a.tiles_y) * ROWS; claimed /= a.tiles_y;
            p_n = claimed;
        }
        const unsigned slot = ring_addr + p_slot * SLOT_BYTES, bar = bar_addr + 8 * p_slot;
        mbar_expect_tx(bar, 2 * K_BYTES);
        tma_load_4d(slot, &kmap, bar, p_x0 - 4, p_it * KCH, a.ytop0 + p_y0 - 2, p_n);
        tma_load_4d(slot + K_BYTES, &qmap, bar, 2 * p_x0, p_it * KCH, 2 * p_y0, p_n);
        if (++p_it == nk) { p_it = 0; ++p_ti; }
        p_slot = (p_slot + 1) % NKQ;
    };
    // value boxes of one round (units round*NW .. round*NW+NW-1) of the tile at (x0, y0, n); every value barrier
    // completes one phase per round, with or without data
    auto issue_v = [&](int round, int x0, int y0, int n) {
#pragma unroll 1
        for (int w = 0; w < NW; ++w) {
            const int unit = round * NW + w;
            const unsigned bar = bar_addr + 8 * (NKQ + w);
            if (unit < nv) {
                mbar_expect_tx(bar, SLOT_BYTES);
                tma_load_4d(ring_addr + (NKQ + w) * SLOT_BYTES, &vmap, bar, x0 - 4, unit * VCH, a.ytop0 + y0 - 2, n);
            } else {
                mbar_arrive(bar);
            }
        }
    };
    if (tid == 0) {
#pragma unroll 1
        for (int i = 0; i < NKQ - 1; ++i) issue_kq();
    }

    // ---- logit phase constants (warp = (low-res row, 4-column half); lane (g, t) as in the m16n8k8 fragments)
    const int wrow = warp >> 1, h = warp & 1;
    const int g = lane >> 2, t = lane & 3;
    const int l = g >> 1;
    const bool ok0 = (2 * t >= l) && (2 * t <= l + 4), ok1 = (2 * t + 1 >= l) && (2 * t + 1 <= l + 4);
    const int q_off0 = t * ROWB + swz(8 * h + g, t), q_off1 = (t + 4) * ROWB + swz(8 * h + g, t + 4);
    const int k_off0 = t * ROWB + swz(2 + 4 * h + g, t), k_off1 = (t + 4) * ROWB + swz(2 + 4 * h + g, t + 4);
    // where this lane's probabilities go: W[prow][slot][pc & 1][pc >> 1][2r + cx], parent column pc = 4h + l
    const int pc = 4 * h + l;
    const int w_lane = ((pc & 1) * 4 + (pc >> 1)) * 4 + (g & 1);       // + (prow*25 + slot)*32 + 2r

    // ---- aggregation phase constants (lane = (column pair xb, channel c8))
    const int c8 = lane & 7, xb = lane >> 3;
    int voff[3];
#pragma unroll
    for (int p = 0; p < 3; ++p) voff[p] = swz(2 * xb + 2 + 2 * p, c8);      // (c8 + 8i) >> 1 == c8 >> 1 (mod 4)
    const unsigned v_lane = ring_addr + (NKQ + warp) * SLOT_BYTES + c8 * ROWB;
    const unsigned w_lane_rd = w_addr + xb * 16;

    int gsk = 0, vround = 0;
    for (int ti = 0;; ++ti) {
        int tile = ti == 0 ? (int)blockIdx.x : tile_ids[ti & 3];
        if (tile < 0) break;
        const int bx = tile % a.tiles_x; tile /= a.tiles_x;
        const int by = tile % a.tiles_y; tile /= a.tiles_y;
        const int n = tile;
        const int x0 = bx * COLS, y0 = by * ROWS;
        const int y = y0 + wrow;

        // ------------------------------------------------------------------ logits
        float s[5][4];
#pragma unroll
        for (int dy = 0; dy < 5; ++dy)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[dy][i] = 0.f;
        for (int it = 0; it < nk; ++it, ++gsk) {
            __syncthreads();     // the slot refilled next is free; at it == 0 also: the previous tile's aggregation is done
            if (tid == 0) {
                if (it == 0) issue_v(0, x0, y0, n);
                issue_kq();
            }
            if (!mbar_wait_bounded(bar_addr + 8 * (gsk % NKQ), (gsk / NKQ) & 1)) {
                atomicExch(&g_wait_timeout, 1);
                return;
            }
            const unsigned stage = ring_addr + (gsk % NKQ) * SLOT_BYTES;
            const unsigned kb = stage + wrow * (KCH * ROWB);
            const unsigned qb = stage + K_BYTES + (2 * wrow) * (KCH * ROWB);
#pragma unroll
            for (int ks = 0; ks < KCH / 8; ++ks) {
                unsigned ah[4], al[4];
                ah[0] = lds32(qb + ks * 8 * ROWB + q_off0);
                ah[1] = lds32(qb + KCH * ROWB + ks * 8 * ROWB + q_off0);
                ah[2] = lds32(qb + ks * 8 * ROWB + q_off1);
                ah[3] = lds32(qb + KCH * ROWB + ks * 8 * ROWB + q_off1);
#pragma unroll
                for (int i = 0; i < 4; ++i) al[i] = tf32_lo(ah[i]);
#pragma unroll
                for (int dy = 0; dy < 5; ++dy) {
                    const unsigned b0 = lds32(kb + dy * (KCH * ROWB) + ks * 8 * ROWB + k_off0);
                    const unsigned b1 = lds32(kb + dy * (KCH * ROWB) + ks * 8 * ROWB + k_off1);
                    mma_tf32(s[dy], ah, b0, b1);
                    mma_tf32(s[dy], al, b0, b1);
                    mma_tf32(s[dy], ah, tf32_lo(b0), tf32_lo(b1));
                }
            }
        }
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
        __syncthreads();         // the tile's probabilities are complete in shared memory

        // ------------------------------------------------------------------ aggregation
        for (int round = 0; round < nrounds; ++round, ++vround) {
            if (round > 0) {
                __syncthreads();     // every warp is done with its value slot
                if (tid == 0) issue_v(round, x0, y0, n);
            }
            if (!mbar_wait_bounded(bar_addr + 8 * (NKQ + warp), vround & 1)) {
                atomicExch(&g_wait_timeout, 1);
                return;
            }
            const int ch0 = (round * NW + warp) * VCH + c8;     // this lane's channels: ch0 + 8i
            if (ch0 - c8 >= a.C) continue;                       // warp-uniform: no unit for this warp in this round
            float v[5][4][6];
            auto load_row = [&](int r, float (&dst)[4][6]) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int p = 0; p < 3; ++p)
                        lds64(v_lane + r * (VCH * ROWB) + i * 8 * ROWB + voff[p], dst[i][2 * p], dst[i][2 * p + 1]);
            };
#pragma unroll
            for (int r = 0; r < 4; ++r) load_row(r, v[r]);
            const bool col_ok = x0 + 2 * xb < a.W;
            float *op = a.out + ((size_t)n * a.C + ch0) * hi_plane + (size_t)(2 * y0) * sW + 2 * (x0 + 2 * xb);
#pragma unroll
            for (int st = 0; st < ROWS; ++st) {
                load_row(st + 4, v[(st + 4) % 5]);
                float acc[4][2][4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 2; ++j)
#pragma unroll
                        for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int dy = 0; dy < 5; ++dy)
#pragma unroll
                        for (int dx = 0; dx < 5; ++dx) {
                            const float4 w = lds128(w_lane_rd + (((st * 25 + dy * 5 + dx) * 2 + j) * 4) * 16);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float x = v[(st + dy) % 5][i][j + dx];
                                acc[i][j][0] = fmaf(w.x, x, acc[i][j][0]);
                                acc[i][j][1] = fmaf(w.y, x, acc[i][j][1]);
                                acc[i][j][2] = fmaf(w.z, x, acc[i][j][2]);
                                acc[i][j][3] = fmaf(w.w, x, acc[i][j][3]);
                            }
                        }
                if (col_ok && y0 + st < a.H) {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (ch0 + 8 * i < a.C) {
                            float *o = op + (size_t)(8 * i) * hi_plane + (size_t)(2 * st) * sW;
                            __stcs(reinterpret_cast<float4 *>(o), make_float4(acc[i][0][0], acc[i][0][1], acc[i][1][0], acc[i][1][1]));
                            __stcs(reinterpret_cast<float4 *>(o + sW), make_float4(acc[i][0][2], acc[i][0][3], acc[i][1][2], acc[i][1][3]));
                        }
                }
            }
        }
    }
    if (tid == 0) {
        if (atomicAdd(&g_ctas_done[a.sched_slot], 1u) == gridDim.x - 1) {   // last CTA out: reset the scheduler pair
            g_next_tile[a.sched_slot] = 0u;
            g_ctas_done[a.sched_slot] = 0u;
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
