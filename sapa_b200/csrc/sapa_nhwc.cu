// sapa_nhwc.cu — fused SAPA-B forward for channels-last tensors:
//   query [B, sH, sW, d], key [B, H, W, d], value [B, H, W, C] -> out [B, sH, sW, C] (attention [B, sH, sW, K*K] optional).
// Same arithmetic as sapa_fused_forward (sim -> softmax over the K*K window slots -> atn, zero padding at the border;
// reference: qk_cuda_kernel.cu:29-68, av_cuda_kernel.cu:29-75, sapa_base.py:38-40), other memory layout: with the channels
// contiguous a window cell is one vector, so the kernel needs no tiles and no shared memory.
// One warp per 2 x 2 group of high-res pixels of one parent (per pixel when s is odd): they share the parent's window, so
// every key / value vector that is loaded serves four pixels.  Logits: lane k < K*K owns window slot k and walks the d channels of its key cell with
// 16-byte loads (the query vector is the same address in every lane: a broadcast load).  Softmax: two warp reductions.
// Aggregation: the lanes switch to channels - lane l owns 16 bytes of channels at a time - and take the K*K weights from
// the other lanes by shuffle; every load of the value tensor is a 512-byte run of one cell.  Neighbouring pixels read
// the same cells, so the key / value traffic is served by L1 / L2.
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
template <typename T, int NPX>
__global__ void __launch_bounds__(WARPS * 32)
sapa_nhwc_fwd_kernel(const T *__restrict__ query, const T *__restrict__ key, const T *__restrict__ value, T *__restrict__ out,
                     T *__restrict__ attn, int B, int d, int C, int H, int W, int K, int s) {
    constexpr int VN = Vec<T>::N;
    constexpr int PW = NPX == 4 ? 2 : 1;             // pixel group = PW x PW
    const int lane = threadIdx.x & 31, KK = K * K, r = (K - 1) / 2;
    const int sH = s * H, sW = s * W, gw = sW / PW, gh = sH / PW;
    const long long groups = (long long)B * gh * gw;
    const long long warp0 = (long long)blockIdx.x * WARPS + (threadIdx.x >> 5), nwarps = (long long)gridDim.x * WARPS;
    for (long long gi = warp0; gi < groups; gi += nwarps) {
        const int gx = (int)(gi % gw), gy = (int)((gi / gw) % gh), b = (int)(gi / ((long long)gw * gh));
        const int qh0 = gy * PW, qw0 = gx * PW, ph = qh0 / s, pw = qw0 / s;      // the group lies inside one parent
        // ---- logits: lane k owns window slot k, for the NPX pixels of the group
        const int ky = ph + lane / K - r, kx = pw + lane % K - r;
        const bool slot = lane < KK, inside = slot && ky >= 0 && ky < H && kx >= 0 && kx < W;
        const int cell = inside ? (ky * W + kx) : -1;
        size_t pix[NPX];
#pragma unroll
        for (int j = 0; j < NPX; ++j) pix[j] = ((size_t)b * sH + qh0 + j / PW) * sW + qw0 + j % PW;
        float logit[NPX];
#pragma unroll
        for (int j = 0; j < NPX; ++j) logit[j] = 0.f;   // a cell outside the image is zero padding: its logit is exactly 0
        if (inside) {
            const T *kp = key + ((size_t)b * H * W + cell) * d;
            for (int c = 0; c < d; c += VN) {
                float kv[VN];
                load_vec(kp + c, kv);
#pragma unroll
                for (int j = 0; j < NPX; ++j) {
                    float qv[VN];
                    load_vec(query + pix[j] * d + c, qv);        // the same address in every lane: a broadcast load
#pragma unroll
                    for (int i = 0; i < VN; ++i) logit[j] += qv[i] * kv[i];
                }
            }
        }
        // ---- softmax over the K*K slots
        float a[NPX];
#pragma unroll
        for (int j = 0; j < NPX; ++j) {
            float m = slot ? logit[j] : -INFINITY;
#pragma unroll
            for (int sh = 16; sh > 0; sh >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, sh));
            const float e = slot ? expf(logit[j] - m) : 0.f;
            float z = e;
#pragma unroll
            for (int sh = 16; sh > 0; sh >>= 1) z += __shfl_xor_sync(0xffffffffu, z, sh);
            a[j] = e / z;
            if (attn != nullptr && slot) attn[pix[j] * KK + lane] = from_acc<T>(a[j]);
        }
        // ---- aggregation: lane l owns VN channels at a time; the weights and the cells come from the slot lanes by shuffle
        // (the loop bounds are the same in every lane: the shuffles need the whole warp); one value vector serves NPX pixels
        const T *vimg = value + (size_t)b * H * W * C;
        for (int base = 0; base < C; base += 32 * VN) {
            const int c0 = base + lane * VN;
            const bool mine = c0 < C;
            float acc[NPX][VN];
#pragma unroll
            for (int j = 0; j < NPX; ++j)
#pragma unroll
                for (int i = 0; i < VN; ++i) acc[j][i] = 0.f;
#pragma unroll 5
            for (int k = 0; k < KK; ++k) {
                const int ck = __shfl_sync(0xffffffffu, cell, k);
                float ak[NPX];
#pragma unroll
                for (int j = 0; j < NPX; ++j) ak[j] = __shfl_sync(0xffffffffu, a[j], k);
                if (mine && ck >= 0) {
                    float vv[VN];
                    load_vec(vimg + (size_t)ck * C + c0, vv);
#pragma unroll
                    for (int j = 0; j < NPX; ++j)
#pragma unroll
                        for (int i = 0; i < VN; ++i) acc[j][i] += ak[j] * vv[i];
                }
            }
            if (mine) {
#pragma unroll
                for (int j = 0; j < NPX; ++j) store_vec(out + pix[j] * C + c0, acc[j]);
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
    SAPA_REQUIRE((long long)B * s * H * s * W < (1LL << 40), SAPA_ERR_ARGUMENT, "%s: image too large", fn);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool quad = s % 2 == 0;           // 2 x 2 pixel groups never straddle two parents when s is even
    const long long groups = (long long)B * s * H * s * W / (quad ? 4 : 1);
    const long long blocks = (groups + nhwc::WARPS - 1) / nhwc::WARPS;
    const unsigned grid = (unsigned)(blocks < 148LL * 64 ? blocks : 148LL * 64);
    return SAPA_DISPATCH_FAST(dtype, [&] {
        const scalar_t *q = static_cast<const scalar_t *>(query), *k = static_cast<const scalar_t *>(key);
        const scalar_t *v = static_cast<const scalar_t *>(value);
        scalar_t *o = static_cast<scalar_t *>(out), *at = static_cast<scalar_t *>(attn);
        if (quad) nhwc::sapa_nhwc_fwd_kernel<scalar_t, 4><<<grid, nhwc::WARPS * 32, 0, st>>>(q, k, v, o, at, B, d, C, H, W, K, s);
        else nhwc::sapa_nhwc_fwd_kernel<scalar_t, 1><<<grid, nhwc::WARPS * 32, 0, st>>>(q, k, v, o, at, B, d, C, H, W, K, s);
        return check_launch("sapa_nhwc_fwd_kernel");
    });
}
