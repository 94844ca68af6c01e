// sapa_nhwc.cu — fused SAPA-B forward for channels-last tensors:
//   query [B, sH, sW, d], key [B, H, W, d], value [B, H, W, C] -> out [B, sH, sW, C] (attention [B, sH, sW, K*K] optional).
// Same arithmetic as sapa_fused_forward (sim -> softmax over the K*K window slots -> atn, zero padding at the border;
// reference: qk_cuda_kernel.cu:29-68, av_cuda_kernel.cu:29-75, sapa_base.py:38-40), other memory layout: with the channels
// contiguous a window cell is one vector, so the kernel needs no tiles (shared memory only holds a warp's weights).
// One warp per 2 x 2 group of high-res pixels of one parent (per pixel when s is odd): they share the parent's window, so
// every key / value vector that is loaded serves four pixels.  Logits: eight lanes read the d channels of one window
// slot's key cell with 16-byte loads (one 128-byte line per slot and load instruction; four slots at a time) and add
// their partial dot products by shuffle; the query vectors are broadcast loads.  Softmax: lane k owns slot k, two warp
// reductions per pixel; the weights then go to a per-warp scratch row in shared memory.  Aggregation: the lanes switch
// to channels - lane l owns 16 bytes of channels at a time - and read the four weights of a slot as one broadcast
// 16-byte shared-memory load; every load of the value tensor is a 512-byte run of one cell.  Neighbouring pixel groups
// read the same cells, so the key / value traffic is served by L1 / L2.
#include "common.cuh"

namespace sapa {
namespace nhwc {

constexpr int WARPS = 8;

template <typename T> struct Vec { static constexpr int N = 16 / (int)sizeof(T); };

__device__ __forceinline__ void load_vec(const float *p, float (&v)[4]) {
    const float4 t = __ldg(reinterpret_cast<const float4 *>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load_vec(const __half *p, float (&v)[8]) {
    const uint4 t = __ldg(reinterpret_cast<const uint4 *>(p));
    const unsigned w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
        v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void load_vec(const __nv_bfloat16 *p, float (&v)[8]) {
    const uint4 t = __ldg(reinterpret_cast<const uint4 *>(p));
    const unsigned w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ void store_vec(float *p, const float (&v)[4]) {
    __stcs(reinterpret_cast<float4 *>(p), make_float4(v[0], v[1], v[2], v[3]));
}
__device__ __forceinline__ void store_vec(__half *p, const float (&v)[8]) {
    uint4 t;
    unsigned *w = &t.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const unsigned *>(&h);
    }
    __stcs(reinterpret_cast<uint4 *>(p), t);
}
__device__ __forceinline__ void store_vec(__nv_bfloat16 *p, const float (&v)[8]) {
    uint4 t;
    unsigned *w = &t.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const unsigned *>(&h);
    }
    __stcs(reinterpret_cast<uint4 *>(p), t);
}

// NPX = high-res pixels of one parent handled together (they share the parent's window): 4 when s is even, else 1.
// Per warp: lg[slot][pixel] = logits, then the aggregation weights (0 for a slot outside the image: its value is zero
// padding); cell_k / cell_v = element offset of the slot's cell in the key / value image, -1 / 0 outside the image.
// Addresses are one 64-bit base per tensor and group plus 32-bit offsets: an image of any one tensor must hold fewer
// than 2^31 elements (checked by the entry point).
template <typename T, int NPX, int KFIX>     // KFIX: kernel_size known at compile time (0: read K at run time)
__global__ void __launch_bounds__(WARPS * 32, 4)
sapa_nhwc_fwd_kernel(const T *__restrict__ query, const T *__restrict__ key, const T *__restrict__ value, T *__restrict__ out,
                     T *__restrict__ attn, int B, int d, int C, int H, int W, int K_runtime, int s) {
    const int K = KFIX > 0 ? KFIX : K_runtime;
    constexpr int VN = Vec<T>::N;
    constexpr int PW = NPX == 4 ? 2 : 1;             // pixel group = PW x PW
    __shared__ __align__(16) float lg_all[WARPS][32 * NPX];
    __shared__ int cell_all[WARPS][64];
    float *lg = lg_all[threadIdx.x >> 5];
    int *cell_k = cell_all[threadIdx.x >> 5], *cell_v = cell_k + 32;
    const int lane = threadIdx.x & 31, KK = K * K, r = (K - 1) / 2;
    const int sH = s * H, sW = s * W, gw = sW / PW, gh = sH / PW;
    const unsigned groups = (unsigned)B * gh * gw;
    const unsigned warp0 = blockIdx.x * WARPS + (threadIdx.x >> 5), nwarps = gridDim.x * WARPS;
    const int sub = lane & 7, quarter = lane >> 3;           // logits: eight lanes per window slot, four slots at a time
    const bool slot = lane < KK;
    const int dy = lane / K - r, dx = lane % K - r;          // this lane's window slot
    int poff[NPX];                                           // pixel j of a group relative to its first pixel
#pragma unroll
    for (int j = 0; j < NPX; ++j) poff[j] = (j / PW) * sW + j % PW;
    int qoff[NPX];                                           // the same in elements of the query tensor
#pragma unroll
    for (int j = 0; j < NPX; ++j) qoff[j] = poff[j] * d;
    for (unsigned gi = warp0; gi < groups; gi += nwarps) {
        const int gx = (int)(gi % (unsigned)gw), gy = (int)((gi / (unsigned)gw) % (unsigned)gh), b = (int)(gi / ((unsigned)gw * gh));
        const int qh0 = gy * PW, qw0 = gx * PW, ph = qh0 / s, pw = qw0 / s;      // the group lies inside one parent
        const size_t pix0 = ((size_t)b * sH + qh0) * sW + qw0;
        const T *q0 = query + pix0 * d, *kimg = key + (size_t)b * H * W * d, *vimg = value + (size_t)b * H * W * C;
        __syncwarp();                      // the previous group's weights have been read by every lane
        bool inside = false;
        if (slot) {
            const int ky = ph + dy, kx = pw + dx;
            inside = ky >= 0 && ky < H && kx >= 0 && kx < W;
            cell_k[lane] = inside ? (ky * W + kx) * d : -1;
            cell_v[lane] = inside ? (ky * W + kx) * C : 0;
        }
        __syncwarp();
        // ---- logits: the key vector of a slot is read by eight lanes, 16 bytes each (one 128-byte line per slot and
        // load), the partial dot products are added over the eight lanes; a slot outside the image has logit exactly 0
        const T *qs = q0 + sub * VN;           // this lane's 16 bytes of the first query vector
#pragma unroll (KFIX > 0 && sizeof(T) == 2 ? (KFIX * KFIX + 3) / 4 : 1)      // float32 is short of registers here
        for (int k0 = 0; k0 < KK; k0 += 4) {
            const int k = k0 + quarter;
            const int cell = k < KK ? cell_k[k] : -1;
            float part[NPX];
#pragma unroll
            for (int j = 0; j < NPX; ++j) part[j] = 0.f;
            if (cell >= 0) {
                const T *kp = kimg + cell + sub * VN;
                for (int c = 0; c < d - sub * VN; c += 8 * VN) {
                    float kv[VN];
                    load_vec(kp + c, kv);
#pragma unroll
                    for (int j = 0; j < NPX; ++j) {
                        float qv[VN];
                        load_vec(qs + (qoff[j] + c), qv);
#pragma unroll
                        for (int i = 0; i < VN; ++i) part[j] += qv[i] * kv[i];
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < NPX; ++j) {
                part[j] += __shfl_xor_sync(0xffffffffu, part[j], 1);
                part[j] += __shfl_xor_sync(0xffffffffu, part[j], 2);
                part[j] += __shfl_xor_sync(0xffffffffu, part[j], 4);
            }
            if (sub == 0 && k < KK) {
#pragma unroll
                for (int j = 0; j < NPX; ++j) lg[k * NPX + j] = part[j];
            }
        }
        __syncwarp();
        // ---- softmax over the K*K slots: lane k owns slot k
        float a[NPX];
#pragma unroll
        for (int j = 0; j < NPX; ++j) {
            const float x = slot ? lg[lane * NPX + j] : -INFINITY;
            float m = x;
#pragma unroll
            for (int sh = 16; sh > 0; sh >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, sh));
            const float e = slot ? expf(x - m) : 0.f;
            float z = e;
#pragma unroll
            for (int sh = 16; sh > 0; sh >>= 1) z += __shfl_xor_sync(0xffffffffu, z, sh);
            a[j] = e / z;
            if (attn != nullptr && slot) attn[(pix0 + poff[j]) * KK + lane] = from_acc<T>(a[j]);
        }
        __syncwarp();                      // every lane has read its logits
        if (slot) {
#pragma unroll
            for (int j = 0; j < NPX; ++j) lg[lane * NPX + j] = inside ? a[j] : 0.f;
        }
        __syncwarp();
        // ---- aggregation: lane l owns VN channels at a time; the NPX weights of a slot are one broadcast read of the
        // scratch row, the slot's value vector one 16-byte load per lane (a 512-byte run of the cell per warp); a slot
        // outside the image reads cell 0 with weight 0, so the loop has no branch
        T *o0 = out + pix0 * C;
        for (int base = 0; base < C; base += 32 * VN) {
            const int c0 = base + lane * VN;
            if (c0 < C) {
                const T *vb = vimg + c0;
                float acc[NPX][VN];
#pragma unroll
                for (int j = 0; j < NPX; ++j)
#pragma unroll
                    for (int i = 0; i < VN; ++i) acc[j][i] = 0.f;
#pragma unroll (KFIX > 0 ? KFIX * KFIX : 5)
                for (int k = 0; k < KK; ++k) {
                    float vv[VN], ak[NPX];
                    load_vec(vb + cell_v[k], vv);
                    if (NPX == 4) {
                        const float4 w4 = *reinterpret_cast<const float4 *>(lg + k * NPX);
                        ak[0] = w4.x; ak[1 % NPX] = w4.y; ak[2 % NPX] = w4.z; ak[3 % NPX] = w4.w;
                    } else {
                        ak[0] = lg[k];
                    }
#pragma unroll
                    for (int j = 0; j < NPX; ++j)
#pragma unroll
                        for (int i = 0; i < VN; ++i) acc[j][i] += ak[j] * vv[i];
                }
#pragma unroll
                for (int j = 0; j < NPX; ++j) store_vec(o0 + (poff[j] * C + c0), acc[j]);
            }
        }
    }
}

}  // namespace nhwc
}  // namespace sapa

using namespace sapa;

extern "C" int sapa_fused_forward_nhwc(const void *query, const void *key, const void *value, void *out, void *attn, int B, int d,
                                       int C, int H, int W, int K, int s, int dtype, void *stream) {
    const char *fn = "sapa_fused_forward_nhwc";
    trace_reset();
    SAPA_REQUIRE(B > 0 && d > 0 && C > 0 && H > 0 && W > 0, SAPA_ERR_ARGUMENT, "%s: sizes must be positive", fn);
    SAPA_REQUIRE(K >= 1 && K % 2 == 1 && s >= 1, SAPA_ERR_ARGUMENT, "%s: kernel_size must be odd, scale_factor >= 1", fn);
    SAPA_REQUIRE(dtype == SAPA_F32 || dtype == SAPA_F16 || dtype == SAPA_BF16, SAPA_ERR_DTYPE,
                 "%s: float32, float16 or bfloat16 (dtype code %d)", fn, dtype);
    const int vn = 16 / (int)dtype_size(dtype);
    SAPA_REQUIRE(K * K <= 32 && d % vn == 0 && C % vn == 0, SAPA_ERR_UNSUPPORTED,
                 "%s: needs kernel_size <= 5 and channel counts that are multiples of %d (16-byte vectors)", fn, vn);
    SAPA_CHECK_PTR(fn, query); SAPA_CHECK_PTR(fn, key); SAPA_CHECK_PTR(fn, value); SAPA_CHECK_PTR(fn, out);
    SAPA_REQUIRE(all_aligned16(query, key, value, out), SAPA_ERR_ALIGNMENT, "%s: tensors must be 16-byte aligned", fn);
    SAPA_REQUIRE((long long)B * s * H * s * W < (1LL << 32) && (long long)H * W * (C > d ? C : d) < (1LL << 31) &&
                     (long long)(s * W + 1) * (C > d ? C : d) < (1LL << 31),
                 SAPA_ERR_ARGUMENT, "%s: image too large", fn);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool quad = s % 2 == 0;           // 2 x 2 pixel groups never straddle two parents when s is even
    const long long groups = (long long)B * s * H * s * W / (quad ? 4 : 1);
    const long long blocks = (groups + nhwc::WARPS - 1) / nhwc::WARPS;
    const unsigned grid = (unsigned)(blocks < 148LL * 64 ? blocks : 148LL * 64);
    return SAPA_DISPATCH_FAST(dtype, [&] {
        const scalar_t *q = static_cast<const scalar_t *>(query), *k = static_cast<const scalar_t *>(key);
        const scalar_t *v = static_cast<const scalar_t *>(value);
        scalar_t *o = static_cast<scalar_t *>(out), *at = static_cast<scalar_t *>(attn);
        if (quad && K == 5) nhwc::sapa_nhwc_fwd_kernel<scalar_t, 4, 5><<<grid, nhwc::WARPS * 32, 0, st>>>(q, k, v, o, at, B, d, C, H, W, K, s);
        else if (quad) nhwc::sapa_nhwc_fwd_kernel<scalar_t, 4, 0><<<grid, nhwc::WARPS * 32, 0, st>>>(q, k, v, o, at, B, d, C, H, W, K, s);
        else nhwc::sapa_nhwc_fwd_kernel<scalar_t, 1, 0><<<grid, nhwc::WARPS * 32, 0, st>>>(q, k, v, o, at, B, d, C, H, W, K, s);
        return check_launch("sapa_nhwc_fwd_kernel");
    });
}
