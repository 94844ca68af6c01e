// sapa_b.cu — SAPA-B kernels: similarity (sim), softmax, aggregation (atn), forward and backward.
//
// Three primitives cover all eight tensor contractions of the forward and backward passes, because the
// backward of each op is another op with the roles of the tensors exchanged:
//
//   sim (hi X[.,Cc,sH,sW], lo L[.,Cc,H,W])  -> S[.,K*K,sH,sW]     S_k(p)  = sum_c X_c(p) * L_c(win_k(p))
//   agg (W [.,K*K,sH,sW],  lo L[.,Cc,H,W])  -> O[.,Cc,sH,sW]      O_c(p)  = sum_k W_k(p) * L_c(win_k(p))
//   gath(hi X[.,Cc,sH,sW], W [.,K*K,sH,sW]) -> G[.,Cc,H,W]        G_c(u)  = sum_{p,k: win_k(p)=u} X_c(p) * W_k(p)
//
//   qk forward = sim(Q, Key)          qk backward: dQ = agg(dS, Key), dKey = gath(Q, dS)
//   av forward = agg(A, V)            av backward: dA = sim(dOut, V), dV   = gath(dOut, A)
//
// win_k(p) is the low-res neighbour (ph/s - r + k/K, pw/s - r + k%K), r = (K-1)/2; neighbours outside the
// image read as zero.  All backward kernels are gathers: no atomics, bit-reproducible.
//
// Two families:
//   * tiled kernels for (K, s) in {(5,2), (3,2)}, f32/f16/bf16: one thread per LOW-res pixel, i.e. per
//     s x s group of high-res pixels that share one K x K window; the window weights of the whole group
//     (K*K*s*s values) live in registers, the low-res halo tile of L is staged in shared memory, and HBM is
//     touched once per element with vector loads/stores.  The fused kernel runs sim -> softmax -> agg
//     without the attention map ever leaving registers.
//   * generic kernels for every other odd K, s >= 1 and for f64: one thread per output element.
#include "common.cuh"

#include <cstring>
#include <mutex>

namespace sapa {

// ==================================================================================================
// Generic kernels
// ==================================================================================================

template <typename T>
__global__ void sim_generic_kernel(const T *__restrict__ hi, const T *__restrict__ lo, T *__restrict__ out,
                                   int B, int Cc, int H, int W, int K, int s) {
    using A = typename AccOf<T>::type;
    const int sH = s * H, sW = s * W, KK = K * K, r = (K - 1) / 2;
    const long long total = (long long)B * KK * sH * sW;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int pw = (int)(i % sW);
        const int ph = (int)((i / sW) % sH);
        const int k = (int)((i / ((long long)sW * sH)) % KK);
        const int n = (int)(i / ((long long)sW * sH * KK));
        const int y = ph / s - r + k / K, x = pw / s - r + k % K;
        A acc = 0;
        if (y >= 0 && y < H && x >= 0 && x < W) {
            const T *hp = hi + ((size_t)n * Cc * sH + ph) * sW + pw;
            const T *lp = lo + ((size_t)n * Cc * H + y) * W + x;
            for (int c = 0; c < Cc; ++c)
                acc += to_acc(hp[(size_t)c * sH * sW]) * to_acc(lp[(size_t)c * H * W]);
        }
        out[i] = from_acc<T>(acc);
    }
}

template <typename T>
__global__ void agg_generic_kernel(const T *__restrict__ wt, const T *__restrict__ lo, T *__restrict__ out,
                                   int B, int Cc, int H, int W, int K, int s) {
    using A = typename AccOf<T>::type;
    const int sH = s * H, sW = s * W, KK = K * K, r = (K - 1) / 2;
    const long long total = (long long)B * Cc * sH * sW;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int pw = (int)(i % sW);
        const int ph = (int)((i / sW) % sH);
        const int c = (int)((i / ((long long)sW * sH)) % Cc);
        const int n = (int)(i / ((long long)sW * sH * Cc));
        const T *wp = wt + ((size_t)n * KK * sH + ph) * sW + pw;
        const T *lp = lo + ((size_t)n * Cc + c) * H * W;
        const int y0 = ph / s - r, x0 = pw / s - r;
        A acc = 0;
        for (int dy = 0; dy < K; ++dy) {
            const int y = y0 + dy;
            if (y < 0 || y >= H) continue;
            for (int dx = 0; dx < K; ++dx) {
                const int x = x0 + dx;
                if (x < 0 || x >= W) continue;
                acc += to_acc(wp[(size_t)(dy * K + dx) * sH * sW]) * to_acc(lp[(size_t)y * W + x]);
            }
        }
        out[i] = from_acc<T>(acc);
    }
}

template <typename T>
__global__ void gath_generic_kernel(const T *__restrict__ hi, const T *__restrict__ wt, T *__restrict__ out,
                                    int B, int Cc, int H, int W, int K, int s) {
    using A = typename AccOf<T>::type;
    const int sH = s * H, sW = s * W, KK = K * K, r = (K - 1) / 2;
    const long long total = (long long)B * Cc * H * W;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int x = (int)(i % W);
        const int y = (int)((i / W) % H);
        const int c = (int)((i / ((long long)W * H)) % Cc);
        const int n = (int)(i / ((long long)W * H * Cc));
        const T *hp = hi + ((size_t)n * Cc + c) * sH * sW;
        const T *wp = wt + (size_t)n * KK * sH * sW;
        A acc = 0;
        for (int dy = 0; dy < K; ++dy) {
            const int py = y - dy + r;              // low-res parent whose tap dy lands on row y
            if (py < 0 || py >= H) continue;
            for (int dx = 0; dx < K; ++dx) {
                const int px = x - dx + r;
                if (px < 0 || px >= W) continue;
                const T *wk = wp + (size_t)(dy * K + dx) * sH * sW;
                for (int sy = 0; sy < s; ++sy)
                    for (int sx = 0; sx < s; ++sx) {
                        const size_t p = (size_t)(py * s + sy) * sW + (px * s + sx);
                        acc += to_acc(hp[p]) * to_acc(wk[p]);
                    }
            }
        }
        out[i] = from_acc<T>(acc);
    }
}

// Softmax over the K*K axis of [B,KK,N] (N = sH*sW) and its backward; one thread per (b, pixel).
template <typename T>
__global__ void softmax_generic_kernel(const T *__restrict__ x, T *__restrict__ y, int B, int KK, long long N) {
    using A = typename AccOf<T>::type;
    const long long total = (long long)B * N;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const size_t base = (size_t)(i / N) * KK * N + (size_t)(i % N);
        A m = to_acc(x[base]);
        for (int k = 1; k < KK; ++k) m = max(m, to_acc(x[base + (size_t)k * N]));
        A z = 0;
        for (int k = 0; k < KK; ++k) z += exp(to_acc(x[base + (size_t)k * N]) - m);
        const A inv = A(1) / z;
        for (int k = 0; k < KK; ++k) y[base + (size_t)k * N] = from_acc<T>(exp(to_acc(x[base + (size_t)k * N]) - m) * inv);
    }
}

template <typename T>
__global__ void softmax_bwd_generic_kernel(const T *__restrict__ y, const T *dy, T *dx /* may alias dy */,
                                           int B, int KK, long long N) {
    using A = typename AccOf<T>::type;
    const long long total = (long long)B * N;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const size_t base = (size_t)(i / N) * KK * N + (size_t)(i % N);
        A dot = 0;
        for (int k = 0; k < KK; ++k) dot += to_acc(y[base + (size_t)k * N]) * to_acc(dy[base + (size_t)k * N]);
        for (int k = 0; k < KK; ++k)
            dx[base + (size_t)k * N] =
                from_acc<T>(to_acc(y[base + (size_t)k * N]) * (to_acc(dy[base + (size_t)k * N]) - dot));
    }
}

// ==================================================================================================
// Tiled kernels: one thread per low-res pixel (= S x S group of high-res pixels)
// ==================================================================================================

enum TileMode {
    MODE_SIM = 0,    // hi X, lo L            -> logits S
    MODE_AGG = 1,    // weights Wt, lo L      -> hi output
    MODE_FUSED = 2,  // Q, Key, V             -> Out (+ optional attention map)
    MODE_BWD = 3     // dOut, V, A, Key       -> dS (to workspace) and dQ
};

template <int K_, int S_, int TH_, int TW_, int CH_>
struct TileShape {
    static constexpr int K = K_, S = S_, TH = TH_, TW = TW_, CH = CH_;
    static constexpr int R = (K - 1) / 2;
    static constexpr int NT = TH * TW;                // threads per CTA
    static constexpr int HH = TH + K - 1;             // halo tile rows
    static constexpr int HW = TW + K - 1;             // halo tile cols
    static constexpr int PLANE = HH * HW;             // elements per channel plane in smem
    static constexpr int PER = (PLANE + NT - 1) / NT; // halo elements fetched per thread per channel
    static constexpr int KK = K * K;
    static constexpr int SS = S * S;
};

// Per-thread record of which halo elements it fetches (identical for every channel chunk).
template <typename Shape>
struct HaloMap {
    int off[Shape::PER];   // gy * W + gx inside one channel plane, or -1 when outside the image / tile
    __device__ __forceinline__ void init(int tid, int ytop, int xleft, int rows, int W) {
#pragma unroll
        for (int j = 0; j < Shape::PER; ++j) {
            const int e = tid + j * Shape::NT;
            const int yy = e / Shape::HW, xx = e % Shape::HW;
            const int gy = ytop + yy, gx = xleft + xx;
            off[j] = (e < Shape::PLANE && gy >= 0 && gy < rows && gx >= 0 && gx < W) ? gy * W + gx : -1;
        }
    }
};

// Registers holding one chunk (CH channels) of halo data in flight between global and shared memory.
template <typename T, typename Shape>
struct HaloStage {
    float v[Shape::CH][Shape::PER];
    __device__ __forceinline__ void fetch(const T *__restrict__ img, size_t plane_stride, int c0, int Cc,
                                          const HaloMap<Shape> &m) {
#pragma unroll
        for (int c = 0; c < Shape::CH; ++c) {
            const bool cok = (c0 + c) < Cc;
            const T *p = img + (size_t)(c0 + c) * plane_stride;
#pragma unroll
            for (int j = 0; j < Shape::PER; ++j)
                v[c][j] = (cok && m.off[j] >= 0) ? to_acc(__ldg(p + m.off[j])) : 0.f;
        }
    }
    __device__ __forceinline__ void commit(float *__restrict__ sm, int tid) const {
#pragma unroll
        for (int c = 0; c < Shape::CH; ++c)
#pragma unroll
            for (int j = 0; j < Shape::PER; ++j) {
                const int e = tid + j * Shape::NT;
                if (e < Shape::PLANE) sm[c * Shape::PLANE + e] = v[c][j];
            }
    }
};

// Loads / stores the S x S high-res values of one low-res parent for one channel plane.
template <typename T, int S>
__device__ __forceinline__ void load_group(const T *__restrict__ plane, int sW, int y, int x, bool active,
                                           float (&g)[S * S]) {
    if (!active) {
#pragma unroll
        for (int i = 0; i < S * S; ++i) g[i] = 0.f;
        return;
    }
    if constexpr (S == 2) {
        const float2 a = load_pair<T>(plane + (size_t)(2 * y) * sW + 2 * x);
        const float2 b = load_pair<T>(plane + (size_t)(2 * y + 1) * sW + 2 * x);
        g[0] = a.x; g[1] = a.y; g[2] = b.x; g[3] = b.y;
    } else {
#pragma unroll
        for (int sy = 0; sy < S; ++sy)
#pragma unroll
            for (int sx = 0; sx < S; ++sx) g[sy * S + sx] = to_acc(plane[(size_t)(S * y + sy) * sW + S * x + sx]);
    }
}

template <typename T, int S>
__device__ __forceinline__ void store_group(T *__restrict__ plane, int sW, int y, int x, const float (&g)[S * S]) {
    if constexpr (S == 2) {
        store_pair<T>(plane + (size_t)(2 * y) * sW + 2 * x, g[0], g[1]);
        store_pair<T>(plane + (size_t)(2 * y + 1) * sW + 2 * x, g[2], g[3]);
    } else {
#pragma unroll
        for (int sy = 0; sy < S; ++sy)
#pragma unroll
            for (int sx = 0; sx < S; ++sx) plane[(size_t)(S * y + sy) * sW + S * x + sx] = from_acc<T>(g[sy * S + sx]);
    }
}

// acc[k][i] += hi_i * L(win_k) over the CH channels of one staged chunk.
template <typename T, typename Shape>
__device__ __forceinline__ void sim_chunk(float (&acc)[Shape::KK][Shape::SS], const float *__restrict__ sm,
                                          const T *__restrict__ hi_img, size_t hi_plane, int sW, int c0, int Cc,
                                          int y, int x, bool active, int ty, int tx) {
#pragma unroll
    for (int c = 0; c < Shape::CH; ++c) {
        float g[Shape::SS];
        load_group<T, Shape::S>(hi_img + (size_t)(c0 + c) * hi_plane, sW, y, x, active && (c0 + c) < Cc, g);
        const float *w = sm + c * Shape::PLANE + ty * Shape::HW + tx;
#pragma unroll
        for (int dy = 0; dy < Shape::K; ++dy)
#pragma unroll
            for (int dx = 0; dx < Shape::K; ++dx) {
                const float l = w[dy * Shape::HW + dx];
#pragma unroll
                for (int i = 0; i < Shape::SS; ++i) acc[dy * Shape::K + dx][i] = fmaf(g[i], l, acc[dy * Shape::K + dx][i]);
            }
    }
}

// out_c(group) = sum_k wt[k][i] * L_c(win_k) for the CH channels of one staged chunk; stores to global.
template <typename T, typename Shape>
__device__ __forceinline__ void agg_chunk(const float (&wt)[Shape::KK][Shape::SS], const float *__restrict__ sm,
                                          T *__restrict__ out_img, size_t hi_plane, int sW, int c0, int Cc,
                                          int y, int x, bool active, int ty, int tx) {
#pragma unroll
    for (int c = 0; c < Shape::CH; ++c) {
        float o[Shape::SS];
#pragma unroll
        for (int i = 0; i < Shape::SS; ++i) o[i] = 0.f;
        const float *w = sm + c * Shape::PLANE + ty * Shape::HW + tx;
#pragma unroll
        for (int dy = 0; dy < Shape::K; ++dy)
#pragma unroll
            for (int dx = 0; dx < Shape::K; ++dx) {
                const float l = w[dy * Shape::HW + dx];
#pragma unroll
                for (int i = 0; i < Shape::SS; ++i) o[i] = fmaf(wt[dy * Shape::K + dx][i], l, o[i]);
            }
        if (active && (c0 + c) < Cc) store_group<T, Shape::S>(out_img + (size_t)(c0 + c) * hi_plane, sW, y, x, o);
    }
}

// Softmax over the K*K window slots, independently for each of the S*S pixels of the group.
template <typename Shape>
__device__ __forceinline__ void softmax_regs(float (&a)[Shape::KK][Shape::SS]) {
#pragma unroll
    for (int i = 0; i < Shape::SS; ++i) {
        float m = a[0][i];
#pragma unroll
        for (int k = 1; k < Shape::KK; ++k) m = fmaxf(m, a[k][i]);
        float z = 0.f;
#pragma unroll
        for (int k = 0; k < Shape::KK; ++k) {
            a[k][i] = expf(a[k][i] - m);
            z += a[k][i];
        }
        const float inv = 1.f / z;
#pragma unroll
        for (int k = 0; k < Shape::KK; ++k) a[k][i] *= inv;
    }
}

template <typename T, typename Shape>
__device__ __forceinline__ void load_slots(const T *__restrict__ img /* [KK,sH,sW] of image n */, size_t hi_plane,
                                           int sW, int y, int x, bool active, float (&a)[Shape::KK][Shape::SS]) {
#pragma unroll
    for (int k = 0; k < Shape::KK; ++k) load_group<T, Shape::S>(img + (size_t)k * hi_plane, sW, y, x, active, a[k]);
}

template <typename T, typename Shape>
__device__ __forceinline__ void store_slots(T *__restrict__ img, size_t hi_plane, int sW, int y, int x,
                                            const float (&a)[Shape::KK][Shape::SS]) {
#pragma unroll
    for (int k = 0; k < Shape::KK; ++k) store_group<T, Shape::S>(img + (size_t)k * hi_plane, sW, y, x, a[k]);
}

struct TileArgs {
    // MODE_SIM:   hi = X, lo1 = L,                     out_slots = S
    // MODE_AGG:   slots_in = W, lo2 = L,               out_hi = O
    // MODE_FUSED: hi = Q, lo1 = Key, lo2 = V,          out_hi = Out, out_slots = attention (optional)
    // MODE_BWD:   hi = dOut, lo1 = V, slots_in = A, lo2 = Key, out_slots = dS, out_hi = dQ
    const void *hi;
    const void *lo1;
    const void *lo2;
    const void *slots_in;
    void *out_hi;
    void *out_slots;
    int B, C1, C2;      // channels contracted against lo1 / produced from lo2
    int H, W;           // low-res rows / cols for which outputs are produced
    int rows, ytop0;    // rows held by lo1/lo2 (H + halos) and the row of lo1/lo2 that is output row 0
    int tiles_x, tiles_y;
};

template <typename T, typename Shape, int MODE, int MINB>
__global__ void __launch_bounds__(Shape::NT, MINB) sapa_tile_kernel(const TileArgs a) {
    constexpr int K = Shape::K, S = Shape::S, KK = Shape::KK, SS = Shape::SS, CH = Shape::CH;
    __shared__ float sm[2][CH * Shape::PLANE];

    const int tid = threadIdx.x;
    const int tx = tid % Shape::TW, ty = tid / Shape::TW;
    int t = blockIdx.x;
    const int bx = t % a.tiles_x; t /= a.tiles_x;
    const int by = t % a.tiles_y; t /= a.tiles_y;
    const int n = t;
    const int y = by * Shape::TH + ty, x = bx * Shape::TW + tx;
    const bool active = (y < a.H) && (x < a.W);
    const int sW = S * a.W;
    const size_t hi_plane = (size_t)(S * a.H) * sW;
    const size_t lo_plane = (size_t)a.rows * a.W;

    HaloMap<Shape> map;
    map.init(tid, a.ytop0 + by * Shape::TH - Shape::R, bx * Shape::TW - Shape::R, a.rows, a.W);

    float acc[KK][SS];
#pragma unroll
    for (int k = 0; k < KK; ++k)
#pragma unroll
        for (int i = 0; i < SS; ++i) acc[k][i] = 0.f;

    HaloStage<T, Shape> stage;
    int buf = 0;

    // ---------------- phase 1: contraction against lo1 (sim) ----------------
    if constexpr (MODE != MODE_AGG) {
        const T *lo = static_cast<const T *>(a.lo1) + (size_t)n * a.C1 * lo_plane;
        const T *hi = static_cast<const T *>(a.hi) + (size_t)n * a.C1 * hi_plane;
        const int nchunks = (a.C1 + CH - 1) / CH;
        stage.fetch(lo, lo_plane, 0, a.C1, map);
        stage.commit(sm[0], tid);
        __syncthreads();
        for (int ch = 0; ch < nchunks; ++ch) {
            const bool more = (ch + 1) < nchunks;
            if (more) stage.fetch(lo, lo_plane, (ch + 1) * CH, a.C1, map);
            sim_chunk<T, Shape>(acc, sm[buf], hi, hi_plane, sW, ch * CH, a.C1, y, x, active, ty, tx);
            if (more) stage.commit(sm[buf ^ 1], tid);
            __syncthreads();
            buf ^= 1;
        }
    }

    if constexpr (MODE == MODE_SIM) {
        if (active)
            store_slots<T, Shape>(static_cast<T *>(a.out_slots) + (size_t)n * KK * hi_plane, hi_plane, sW, y, x, acc);
        return;
    }

    // ---------------- between the phases ----------------
    if constexpr (MODE == MODE_AGG) {
        load_slots<T, Shape>(static_cast<const T *>(a.slots_in) + (size_t)n * KK * hi_plane, hi_plane, sW, y, x,
                             active, acc);
    } else if constexpr (MODE == MODE_FUSED) {
        softmax_regs<Shape>(acc);
        if (a.out_slots != nullptr && active)
            store_slots<T, Shape>(static_cast<T *>(a.out_slots) + (size_t)n * KK * hi_plane, hi_plane, sW, y, x, acc);
    } else if constexpr (MODE == MODE_BWD) {
        // acc holds dA; dS_k = A_k * (dA_k - sum_j A_j dA_j), A streamed from the saved attention map
        const T *att = static_cast<const T *>(a.slots_in) + (size_t)n * KK * hi_plane;
        float dot[SS];
#pragma unroll
        for (int i = 0; i < SS; ++i) dot[i] = 0.f;
#pragma unroll
        for (int k = 0; k < KK; ++k) {
            float p[SS];
            load_group<T, S>(att + (size_t)k * hi_plane, sW, y, x, active, p);
#pragma unroll
            for (int i = 0; i < SS; ++i) dot[i] = fmaf(p[i], acc[k][i], dot[i]);
        }
#pragma unroll
        for (int k = 0; k < KK; ++k) {
            float p[SS];
            load_group<T, S>(att + (size_t)k * hi_plane, sW, y, x, active, p);
#pragma unroll
            for (int i = 0; i < SS; ++i) acc[k][i] = p[i] * (acc[k][i] - dot[i]);
        }
        if (active)
            store_slots<T, Shape>(static_cast<T *>(a.out_slots) + (size_t)n * KK * hi_plane, hi_plane, sW, y, x, acc);
    }

    // ---------------- phase 2: aggregation over lo2 (atn) ----------------
    {
        const T *lo = static_cast<const T *>(a.lo2) + (size_t)n * a.C2 * lo_plane;
        T *out = static_cast<T *>(a.out_hi) + (size_t)n * a.C2 * hi_plane;
        const int nchunks = (a.C2 + CH - 1) / CH;
        buf = 0;
        stage.fetch(lo, lo_plane, 0, a.C2, map);
        stage.commit(sm[0], tid);
        __syncthreads();
        for (int ch = 0; ch < nchunks; ++ch) {
            const bool more = (ch + 1) < nchunks;
            if (more) stage.fetch(lo, lo_plane, (ch + 1) * CH, a.C2, map);
            agg_chunk<T, Shape>(acc, sm[buf], out, hi_plane, sW, ch * CH, a.C2, y, x, active, ty, tx);
            if (more) stage.commit(sm[buf ^ 1], tid);
            __syncthreads();
            buf ^= 1;
        }
    }
}

// ---------------------------------------------------------------------------------- gath (tiled)
// One thread per low-res cell u = (y, x).  Its K*K*S*S weights W_k(p) for every (parent p, slot k) that lands
// on u stay in registers; the high-res tile of X (TH+K-1 x TW+K-1 parents) is staged per channel.
template <typename T, typename Shape>
__global__ void __launch_bounds__(Shape::NT) sapa_gath_kernel(const T *__restrict__ hi, const T *__restrict__ wt,
                                                              T *__restrict__ out, int B, int Cc, int H, int W,
                                                              int tiles_x, int tiles_y) {
    constexpr int K = Shape::K, S = Shape::S, KK = Shape::KK, SS = Shape::SS, R = Shape::R;
    constexpr int PH = Shape::HH, PW = Shape::HW;            // parents covered by the staged tile
    constexpr int ROWLEN = PW * S;                           // high-res columns per staged row
    constexpr int CHG = 2;                                   // channels staged per step
    constexpr int PLANE = PH * S * ROWLEN;
    __shared__ __align__(16) float sm[CHG][PLANE];

    const int tid = threadIdx.x;
    const int tx = tid % Shape::TW, ty = tid / Shape::TW;
    int t = blockIdx.x;
    const int bx = t % tiles_x; t /= tiles_x;
    const int by = t % tiles_y; t /= tiles_y;
    const int n = t;
    const int y = by * Shape::TH + ty, x = bx * Shape::TW + tx;
    const bool active = (y < H) && (x < W);
    const int sH = S * H, sW = S * W;
    const size_t hi_plane = (size_t)sH * sW;
    const int py0 = by * Shape::TH - R, px0 = bx * Shape::TW - R;   // first parent of the staged tile

    // weights: slot (dy,dx) of parent (y - dy + R, x - dx + R) reads cell (y, x)
    float w[KK][SS];
    {
        const T *wimg = wt + (size_t)n * KK * hi_plane;
#pragma unroll
        for (int dy = 0; dy < K; ++dy)
#pragma unroll
            for (int dx = 0; dx < K; ++dx) {
                const int py = y - dy + R, px = x - dx + R;
                const bool ok = active && py >= 0 && py < H && px >= 0 && px < W;
                load_group<T, S>(wimg + (size_t)(dy * K + dx) * hi_plane, sW, py, px, ok, w[dy * K + dx]);
            }
    }

    const T *himg = hi + (size_t)n * Cc * hi_plane;
    T *oimg = out + (size_t)n * Cc * H * W;
    for (int c0 = 0; c0 < Cc; c0 += CHG) {
        __syncthreads();
        // stage CHG channels of the high-res tile (zero outside the image)
        for (int e = tid; e < CHG * PLANE; e += Shape::NT) {
            const int c = e / PLANE, rem = e % PLANE;
            const int yy = rem / ROWLEN, xx = rem % ROWLEN;
            const int gy = py0 * S + yy, gx = px0 * S + xx;
            float v = 0.f;
            if ((c0 + c) < Cc && gy >= 0 && gy < sH && gx >= 0 && gx < sW)
                v = to_acc(__ldg(himg + (size_t)(c0 + c) * hi_plane + (size_t)gy * sW + gx));
            sm[c][rem] = v;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < CHG; ++c) {
            float acc = 0.f;
#pragma unroll
            for (int dy = 0; dy < K; ++dy)
#pragma unroll
                for (int dx = 0; dx < K; ++dx) {
                    // parent (ty - dy + 2R, tx - dx + 2R) in tile coordinates
                    const float *p = &sm[c][((ty - dy + 2 * R) * S) * ROWLEN + (tx - dx + 2 * R) * S];
#pragma unroll
                    for (int sy = 0; sy < S; ++sy)
#pragma unroll
                        for (int sx = 0; sx < S; ++sx)
                            acc = fmaf(w[dy * K + dx][sy * S + sx], p[sy * ROWLEN + sx], acc);
                }
            if (active && (c0 + c) < Cc) oimg[(size_t)(c0 + c) * H * W + (size_t)y * W + x] = from_acc<T>(acc);
        }
    }
}

// ==================================================================================================
// Host side
// ==================================================================================================

static inline int grid_1d(long long total, int threads) {
    long long blocks = (total + threads - 1) / threads;
    const long long cap = 148LL * 32;   // grid-stride loops: a few waves of a 148-SM part is enough
    return (int)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

// tensor-core fused forward (sapa_mma.cu)
bool fused_mma_supported(int W, int dtype);
bool fused_tma_supported(int W, int dtype);
int launch_fused_tma(int mode, const void *q, const void *k, const void *v, void *out, void *attn, void *ws, int B, int d, int C,
                     int H, int W, int rows, int ytop0, int y_begin, int y_end, int dtype, cudaStream_t st);
int launch_fused_mma(const void *q, const void *k, const void *v, void *out, void *attn, int B, int d, int C, int H, int W,
                     int rows, int ytop0, int dtype, cudaStream_t st);
int launch_fused_tma_slots(int mode, const void *q, const void *k, const void *v, void *out, void *attn, void *ws, int B, int d,
                           int C, int H, int W, int rows, int ytop0, int y_begin, int y_end, int dtype, bool slots_f32,
                           cudaStream_t st);

int tma_wait_timeout_flag();
int proj_wait_timeout_flag();
int launch_wait_selftest(cudaStream_t st);
int gath_wait_timeout_flag();
// tensor-core transposed aggregation (sapa_gath_mma.cu)
bool gath_mma_supported(int W, int dtype);
int launch_gath_mma(const void *hi, const void *wt, void *out, int B, int C, int H, int W, int top, int bottom, int dtype,
                    cudaStream_t st);

static bool tiled_supported(int K, int s, int dtype) {
    return dtype != SAPA_F64 && s == 2 && (K == 5 || K == 3);
}

template <typename T, int K, int S, int MODE>
static int launch_tile(TileArgs a, cudaStream_t st) {
    // 4 x 32 low-res pixels per CTA (128 threads, one warp per tile row), 4 channels per pipeline stage
    using Shape = TileShape<K, S, 4, 32, 4>;
    a.tiles_x = ceil_div(a.W, Shape::TW);
    a.tiles_y = ceil_div(a.H, Shape::TH);
    const long long blocks = (long long)a.B * a.tiles_x * a.tiles_y;
    if (blocks > 0x7fffffffLL) {
        set_error("too many tiles");
        return SAPA_ERR_ARGUMENT;
    }
    sapa_tile_kernel<T, Shape, MODE, 3><<<(unsigned)blocks, Shape::NT, 0, st>>>(a);
    constexpr const char *names[4] = {"sapa_tile_kernel<sim>", "sapa_tile_kernel<agg>", "sapa_tile_kernel<fused>",
                                      "sapa_tile_kernel<bwd>"};
    return check_launch(names[MODE]);
}

template <typename T, int MODE>
static int launch_tile_ks(const TileArgs &a, int K, cudaStream_t st) {
    if (K == 5) return launch_tile<T, 5, 2, MODE>(a, st);
    return launch_tile<T, 3, 2, MODE>(a, st);
}

template <typename T>
static int launch_gath(const T *hi, const T *wt, T *out, int B, int Cc, int H, int W, int K, cudaStream_t st) {
    auto go = [&](auto shape) -> int {
        using Shape = decltype(shape);
        const int tiles_x = ceil_div(W, Shape::TW), tiles_y = ceil_div(H, Shape::TH);
        const long long blocks = (long long)B * tiles_x * tiles_y;
        sapa_gath_kernel<T, Shape><<<(unsigned)blocks, Shape::NT, 0, st>>>(hi, wt, out, B, Cc, H, W, tiles_x, tiles_y);
        return check_launch("sapa_gath_kernel");
    };
    if (K == 5) return go(TileShape<5, 2, 4, 32, 1>{});
    return go(TileShape<3, 2, 4, 32, 1>{});
}

static int check_common(const char *fn, int B, int C, int H, int W, int K, int s, int dtype) {
    SAPA_REQUIRE(B > 0 && C > 0 && H > 0 && W > 0, SAPA_ERR_ARGUMENT, "%s: sizes must be positive (B=%d C=%d H=%d W=%d)",
                 fn, B, C, H, W);
    SAPA_REQUIRE(K >= 1 && (K - 1) % 2 == 0, SAPA_ERR_ARGUMENT, "%s: kernel_size must be odd and >= 1, got %d", fn, K);
    SAPA_REQUIRE(s >= 1, SAPA_ERR_ARGUMENT, "%s: scale_factor must be >= 1, got %d", fn, s);
    SAPA_REQUIRE(dtype_size(dtype) != 0, SAPA_ERR_DTYPE, "%s: unknown dtype code %d", fn, dtype);
    SAPA_REQUIRE((long long)s * H * s * W < (1LL << 31) && (long long)K * K * s * H * s * W < (1LL << 40), SAPA_ERR_ARGUMENT,
                 "%s: image too large", fn);
    return SAPA_OK;
}


// sim / agg / gath dispatchers (tiled when possible, else generic); sim and agg also serve the dense path of SAPA-D
// Slab form: `lo` holds `rows` = top + H + bottom low-res rows per plane, of which the H rows from `top` on are the
// ones the high-res rows of `hi` / `out` belong to (rows = H, top = 0: a whole image).
int run_sim_slab(const void *hi, const void *lo, void *out, int B, int Cc, int H, int W, int rows, int top, int K, int s,
                 int dtype, cudaStream_t st) {
    const bool al = all_aligned16(hi, lo, out);     // misaligned views take the scalar generic kernels
    if (al && K == 5 && s == 2 && fused_tma_supported(W, dtype)) {     // logit half of the TMA kernel
        const int e = launch_fused_tma(2, hi, lo, nullptr, nullptr, out, nullptr, B, Cc, 0, H, W, rows, top, 0, H, dtype, st);
        if (e != SAPA_ERR_UNSUPPORTED) return e;
    }
    if (al && tiled_supported(K, s, dtype)) {
        TileArgs a{};
        a.hi = hi; a.lo1 = lo; a.out_slots = out;
        a.B = B; a.C1 = Cc; a.C2 = 0; a.H = H; a.W = W; a.rows = rows; a.ytop0 = top;
        return SAPA_DISPATCH_FAST(dtype, [&] { return launch_tile_ks<scalar_t, MODE_SIM>(a, K, st); });
    }
    if (rows != H || top != 0) {
        set_error("run_sim_slab: a padded slab needs 16-byte aligned tensors and a tiled (K, s)");
        return SAPA_ERR_UNSUPPORTED;
    }
    return SAPA_DISPATCH_ALL(dtype, [&] {
        const long long total = (long long)B * K * K * s * H * s * W;
        sim_generic_kernel<scalar_t><<<grid_1d(total, 256), 256, 0, st>>>(
            static_cast<const scalar_t *>(hi), static_cast<const scalar_t *>(lo), static_cast<scalar_t *>(out), B, Cc, H, W, K, s);
        return check_launch("sim_generic_kernel");
    });
}

// 16-bit tensors with a float32 slot tensor (K = 5, s = 2, TMA kernel only): sim writes float32 logits.  The dense-window
// path of SAPA-D keeps its 25-slot similarity at full precision this way.
int run_sim_mixed(const void *hi, const void *lo, float *out, int B, int Cc, int H, int W, int rows, int top, int dtype,
                  cudaStream_t st) {
    if (!(all_aligned16(hi, lo, out) && (dtype == SAPA_F16 || dtype == SAPA_BF16) && fused_tma_supported(W, dtype))) {
        set_error("run_sim_mixed: needs 16-bit tensors, 16-byte aligned, rows of 16 bytes");
        return SAPA_ERR_UNSUPPORTED;
    }
    return launch_fused_tma_slots(2, hi, lo, nullptr, nullptr, out, nullptr, B, Cc, 0, H, W, rows, top, 0, H, dtype, true, st);
}

int run_sim(const void *hi, const void *lo, void *out, int B, int Cc, int H, int W, int K, int s, int dtype, cudaStream_t st) {
    return run_sim_slab(hi, lo, out, B, Cc, H, W, H, 0, K, s, dtype, st);
}

int run_agg_slab(const void *wt, const void *lo, void *out, int B, int Cc, int H, int W, int rows, int top, int K, int s,
                 int dtype, cudaStream_t st) {
    const bool al = all_aligned16(wt, lo, out);
    if (al && K == 5 && s == 2 && fused_tma_supported(W, dtype)) {     // aggregation half of the TMA kernel
        const int e = launch_fused_tma(3, nullptr, nullptr, lo, out, const_cast<void *>(wt), nullptr, B, 0, Cc, H, W, rows, top, 0, H,
                                       dtype, st);
        if (e != SAPA_ERR_UNSUPPORTED) return e;
    }
    if (al && tiled_supported(K, s, dtype)) {
        TileArgs a{};
        a.slots_in = wt; a.lo2 = lo; a.out_hi = out;
        a.B = B; a.C1 = 0; a.C2 = Cc; a.H = H; a.W = W; a.rows = rows; a.ytop0 = top;
        return SAPA_DISPATCH_FAST(dtype, [&] { return launch_tile_ks<scalar_t, MODE_AGG>(a, K, st); });
    }
    if (rows != H || top != 0) {
        set_error("run_agg_slab: a padded slab needs 16-byte aligned tensors and a tiled (K, s)");
        return SAPA_ERR_UNSUPPORTED;
    }
    return SAPA_DISPATCH_ALL(dtype, [&] {
        const long long total = (long long)B * Cc * s * H * s * W;
        agg_generic_kernel<scalar_t><<<grid_1d(total, 256), 256, 0, st>>>(
            static_cast<const scalar_t *>(wt), static_cast<const scalar_t *>(lo), static_cast<scalar_t *>(out), B, Cc, H, W, K, s);
        return check_launch("agg_generic_kernel");
    });
}

int run_agg(const void *wt, const void *lo, void *out, int B, int Cc, int H, int W, int K, int s, int dtype, cudaStream_t st) {
    return run_agg_slab(wt, lo, out, B, Cc, H, W, H, 0, K, s, dtype, st);
}

int run_gath(const void *hi, const void *wt, void *out, int B, int Cc, int H, int W, int K, int s, int dtype,
             cudaStream_t st) {
    const bool al = all_aligned16(hi, wt, out);
    if (al && K == 5 && s == 2 && gath_mma_supported(W, dtype)) {
        const int e = launch_gath_mma(hi, wt, out, B, Cc, H, W, 0, 0, dtype, st);
        if (e != SAPA_ERR_UNSUPPORTED) return e;
    }
    if (al && tiled_supported(K, s, dtype)) {
        return SAPA_DISPATCH_FAST(dtype, [&] {
            return launch_gath<scalar_t>(static_cast<const scalar_t *>(hi), static_cast<const scalar_t *>(wt),
                                         static_cast<scalar_t *>(out), B, Cc, H, W, K, st);
        });
    }
    return SAPA_DISPATCH_ALL(dtype, [&] {
        const long long total = (long long)B * Cc * H * W;
        gath_generic_kernel<scalar_t><<<grid_1d(total, 256), 256, 0, st>>>(
            static_cast<const scalar_t *>(hi), static_cast<const scalar_t *>(wt), static_cast<scalar_t *>(out), B, Cc, H, W, K, s);
        return check_launch("gath_generic_kernel");
    });
}

}  // namespace sapa

using namespace sapa;

extern "C" {

int sapa_wait_timeout_flags(void) {
    const int a = tma_wait_timeout_flag(), b = gath_wait_timeout_flag(), c = proj_wait_timeout_flag();
    if (a < 0 || b < 0 || c < 0) return -1;
    return (a ? 1 : 0) | (b ? 2 : 0) | (c ? 4 : 0);
}

int sapa_selftest_wait_timeout(void *stream) {
    trace_reset();
    return launch_wait_selftest(static_cast<cudaStream_t>(stream));
}

int sapa_qk_forward(const void *query, const void *key, void *out, int B, int d, int H, int W, int K, int s, int dtype,
                    void *stream) {
    const char *fn = "sapa_qk_forward";
    trace_reset();
    if (int e = check_common(fn, B, d, H, W, K, s, dtype)) return e;
    SAPA_CHECK_PTR(fn, query); SAPA_CHECK_PTR(fn, key); SAPA_CHECK_PTR(fn, out);
    return run_sim(query, key, out, B, d, H, W, K, s, dtype, static_cast<cudaStream_t>(stream));
}

int sapa_qk_backward(const void *grad_out, const void *query, const void *key, void *grad_query, void *grad_key, int B,
                     int d, int H, int W, int K, int s, int dtype, void *stream) {
    const char *fn = "sapa_qk_backward";
    trace_reset();
    if (int e = check_common(fn, B, d, H, W, K, s, dtype)) return e;
    SAPA_CHECK_PTR(fn, grad_out); SAPA_CHECK_PTR(fn, query); SAPA_CHECK_PTR(fn, key);
    SAPA_CHECK_PTR(fn, grad_query); SAPA_CHECK_PTR(fn, grad_key);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (int e = run_agg(grad_out, key, grad_query, B, d, H, W, K, s, dtype, st)) return e;   // dQ = agg(dS, Key)
    return run_gath(query, grad_out, grad_key, B, d, H, W, K, s, dtype, st);                 // dKey = gath(Q, dS)
}

int sapa_av_forward(const void *attn, const void *value, void *out, int B, int C, int H, int W, int K, int s, int dtype,
                    void *stream) {
    const char *fn = "sapa_av_forward";
    trace_reset();
    if (int e = check_common(fn, B, C, H, W, K, s, dtype)) return e;
    SAPA_CHECK_PTR(fn, attn); SAPA_CHECK_PTR(fn, value); SAPA_CHECK_PTR(fn, out);
    return run_agg(attn, value, out, B, C, H, W, K, s, dtype, static_cast<cudaStream_t>(stream));
}

int sapa_av_backward(const void *grad_out, const void *attn, const void *value, void *grad_attn, void *grad_value, int B,
                     int C, int H, int W, int K, int s, int dtype, void *stream) {
    const char *fn = "sapa_av_backward";
    trace_reset();
    if (int e = check_common(fn, B, C, H, W, K, s, dtype)) return e;
    SAPA_CHECK_PTR(fn, grad_out); SAPA_CHECK_PTR(fn, attn); SAPA_CHECK_PTR(fn, value);
    SAPA_CHECK_PTR(fn, grad_attn); SAPA_CHECK_PTR(fn, grad_value);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (int e = run_sim(grad_out, value, grad_attn, B, C, H, W, K, s, dtype, st)) return e;  // dA = sim(dOut, V)
    return run_gath(grad_out, attn, grad_value, B, C, H, W, K, s, dtype, st);                // dV = gath(dOut, A)
}

int sapa_fused_forward_slab_rows(const void *query, const void *key, const void *value, void *out, void *attn, int B, int d,
                                 int C, int H, int W, int halo_top, int halo_bottom, int row_begin, int row_end, int K, int s,
                                 int dtype, void *stream) {
    const char *fn = "sapa_fused_forward";
    trace_reset();
    if (int e = check_common(fn, B, d, H, W, K, s, dtype)) return e;
    SAPA_REQUIRE(C > 0, SAPA_ERR_ARGUMENT, "%s: C must be positive", fn);
    SAPA_REQUIRE(halo_top >= 0 && halo_bottom >= 0, SAPA_ERR_ARGUMENT, "%s: negative halo", fn);
    SAPA_REQUIRE(0 <= row_begin && row_begin <= row_end && row_end <= H, SAPA_ERR_ARGUMENT,
                 "%s: row band [%d, %d) is not inside [0, %d)", fn, row_begin, row_end, H);
    SAPA_CHECK_PTR(fn, query); SAPA_CHECK_PTR(fn, key); SAPA_CHECK_PTR(fn, value); SAPA_CHECK_PTR(fn, out);
    SAPA_REQUIRE(all_aligned16(query, key, value, out) && (attn == nullptr || aligned16(attn)), SAPA_ERR_ALIGNMENT,
                 "%s: the fused kernels need 16-byte aligned tensors (copy the misaligned view, or use the separate ops)", fn);
    SAPA_REQUIRE(tiled_supported(K, s, dtype), SAPA_ERR_UNSUPPORTED,
                 "%s: no fused kernel for K=%d s=%d dtype=%d (use the separate ops)", fn, K, s, dtype);
    if (row_begin == row_end) return SAPA_OK;
    TileArgs a{};
    a.hi = query; a.lo1 = key; a.lo2 = value; a.out_hi = out; a.out_slots = attn;
    a.B = B; a.C1 = d; a.C2 = C; a.H = H; a.W = W; a.rows = halo_top + H + halo_bottom; a.ytop0 = halo_top;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (K == 5 && fused_tma_supported(W, dtype)) {
        const int e = launch_fused_tma(0, query, key, value, out, attn, nullptr, B, d, C, H, W, a.rows, a.ytop0, row_begin, row_end,
                                       dtype, st);
        if (e != SAPA_ERR_UNSUPPORTED) return e;
    }
    // the remaining kernels (rows that are not 16-byte aligned, K = 3) always produce the whole slab
    SAPA_REQUIRE(row_begin == 0 && row_end == H, SAPA_ERR_UNSUPPORTED,
                 "%s: a partial row band needs K = 5 and rows of 16 bytes (call with the band [0, H) instead)", fn);
    if (K == 5 && fused_mma_supported(W, dtype))
        return launch_fused_mma(query, key, value, out, attn, B, d, C, H, W, a.rows, a.ytop0, dtype, st);
    return SAPA_DISPATCH_FAST(dtype, [&] { return launch_tile_ks<scalar_t, MODE_FUSED>(a, K, st); });
}

int sapa_fused_forward_slab(const void *query, const void *key, const void *value, void *out, void *attn, int B, int d,
                            int C, int H, int W, int halo_top, int halo_bottom, int K, int s, int dtype, void *stream) {
    return sapa_fused_forward_slab_rows(query, key, value, out, attn, B, d, C, H, W, halo_top, halo_bottom, 0, H, K, s, dtype,
                                        stream);
}

int sapa_fused_forward(const void *query, const void *key, const void *value, void *out, void *attn, int B, int d, int C,
                       int H, int W, int K, int s, int dtype, void *stream) {
    return sapa_fused_forward_slab(query, key, value, out, attn, B, d, C, H, W, 0, 0, K, s, dtype, stream);
}

size_t sapa_fused_backward_workspace(int B, int H, int W, int K, int s, int dtype) {
    if (B <= 0 || H <= 0 || W <= 0 || K <= 0 || s <= 0) return 0;
    return (size_t)B * K * K * s * H * s * W * dtype_size(dtype);
}

int sapa_fused_backward(const void *grad_out, const void *query, const void *key, const void *value, const void *attn,
                        void *grad_query, void *grad_key, void *grad_value, void *workspace, size_t workspace_bytes, int B,
                        int d, int C, int H, int W, int K, int s, int dtype, void *stream) {
    const char *fn = "sapa_fused_backward";
    trace_reset();
    if (int e = check_common(fn, B, d, H, W, K, s, dtype)) return e;
    SAPA_REQUIRE(C > 0, SAPA_ERR_ARGUMENT, "%s: C must be positive", fn);
    SAPA_CHECK_PTR(fn, grad_out); SAPA_CHECK_PTR(fn, query); SAPA_CHECK_PTR(fn, key); SAPA_CHECK_PTR(fn, value);
    SAPA_CHECK_PTR(fn, attn); SAPA_CHECK_PTR(fn, grad_query); SAPA_CHECK_PTR(fn, grad_key); SAPA_CHECK_PTR(fn, grad_value);
    const size_t need = sapa_fused_backward_workspace(B, H, W, K, s, dtype);
    SAPA_REQUIRE(workspace != nullptr && workspace_bytes >= need, SAPA_ERR_WORKSPACE,
                 "%s: workspace of %zu bytes required, got %zu", fn, need, workspace_bytes);
    SAPA_REQUIRE(aligned16(workspace), SAPA_ERR_ALIGNMENT, "%s: workspace is not 16-byte aligned", fn);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    void *dS = workspace;
    bool stage1_done = false;
    // misaligned views (a storage offset that is not a multiple of 16 bytes) take the chain of scalar generic kernels
    const bool al = all_aligned16(grad_out, query, key, value, attn, grad_query, grad_key, grad_value);
    if (al && K == 5 && s == 2 && fused_tma_supported(W, dtype)) {
        // tensor-core kernel (the fused forward's data flow with the softmax backward in the middle)
        const int e = launch_fused_tma(1, grad_out, value, key, grad_query, const_cast<void *>(attn), dS, B, C, d, H, W, H, 0,
                                       0, H, dtype, st);
        if (e != SAPA_OK && e != SAPA_ERR_UNSUPPORTED) return e;
        stage1_done = e == SAPA_OK;
    }
    if (stage1_done) {
    } else if (al && tiled_supported(K, s, dtype)) {
        // one kernel: dA = sim(dOut, V) -> softmax backward with the saved A -> dS (workspace), dQ = agg(dS, Key)
        TileArgs a{};
        a.hi = grad_out; a.lo1 = value; a.slots_in = attn; a.lo2 = key; a.out_slots = dS; a.out_hi = grad_query;
        a.B = B; a.C1 = C; a.C2 = d; a.H = H; a.W = W; a.rows = H; a.ytop0 = 0;
        if (int e = SAPA_DISPATCH_FAST(dtype, [&] { return launch_tile_ks<scalar_t, MODE_BWD>(a, K, st); })) return e;
    } else {
        // dA goes to the workspace, then dS overwrites it in place
        if (int e = run_sim(grad_out, value, dS, B, C, H, W, K, s, dtype, st)) return e;
        const long long N = (long long)s * H * s * W;
        if (int e = SAPA_DISPATCH_ALL(dtype, [&] {
                softmax_bwd_generic_kernel<scalar_t><<<grid_1d((long long)B * N, 256), 256, 0, st>>>(
                    static_cast<const scalar_t *>(attn), static_cast<const scalar_t *>(dS), static_cast<scalar_t *>(dS), B,
                    K * K, N);
                return check_launch("softmax_bwd_generic_kernel");
            }))
            return e;
        if (int e = run_agg(dS, key, grad_query, B, d, H, W, K, s, dtype, st)) return e;
    }
    if (int e = run_gath(query, dS, grad_key, B, d, H, W, K, s, dtype, st)) return e;       // dKey = gath(Q, dS)
    return run_gath(grad_out, attn, grad_value, B, C, H, W, K, s, dtype, st);               // dV = gath(dOut, A)
}

// Backward of sapa_fused_forward_slab for one row slab.  The slab's pixels reach `halo_top` / `halo_bottom` rows of key
// and value that belong to the neighbouring slabs, so the key / value gradients come out in the padded frame: rows
// [halo_top, halo_top + H) are this slab's own contribution to its own rows, the halo rows are its contribution to the
// neighbours' edge rows (the caller sends them there and adds what it receives to its own edge rows).
int sapa_fused_backward_slab(const void *grad_out, const void *query, const void *key, const void *value, const void *attn,
                             void *grad_query, void *grad_key, void *grad_value, void *workspace, size_t workspace_bytes,
                             int B, int d, int C, int H, int W, int halo_top, int halo_bottom, int K, int s, int dtype,
                             void *stream) {
    const char *fn = "sapa_fused_backward_slab";
    trace_reset();
    if (int e = check_common(fn, B, d, H, W, K, s, dtype)) return e;
    SAPA_REQUIRE(C > 0 && halo_top >= 0 && halo_bottom >= 0, SAPA_ERR_ARGUMENT, "%s: C must be positive, halos non-negative", fn);
    SAPA_CHECK_PTR(fn, grad_out); SAPA_CHECK_PTR(fn, query); SAPA_CHECK_PTR(fn, key); SAPA_CHECK_PTR(fn, value);
    SAPA_CHECK_PTR(fn, attn); SAPA_CHECK_PTR(fn, grad_query); SAPA_CHECK_PTR(fn, grad_key); SAPA_CHECK_PTR(fn, grad_value);
    const size_t need = sapa_fused_backward_workspace(B, H, W, K, s, dtype);
    SAPA_REQUIRE(workspace != nullptr && workspace_bytes >= need && aligned16(workspace), SAPA_ERR_WORKSPACE,
                 "%s: a 16-byte aligned workspace of %zu bytes is required, got %zu", fn, need, workspace_bytes);
    SAPA_REQUIRE(K == 5 && s == 2 && fused_tma_supported(W, dtype) && gath_mma_supported(W, dtype) &&
                 all_aligned16(grad_out, query, key, value, attn, grad_query, grad_key, grad_value), SAPA_ERR_UNSUPPORTED,
                 "%s: needs K = 5, s = 2, rows of 16 bytes and 16-byte aligned tensors", fn);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    void *dS = workspace;
    const int rows = halo_top + H + halo_bottom;
    // dA = sim(dOut, value slab) -> softmax backward -> dS; dQ = agg(dS, key slab)
    if (int e = launch_fused_tma(1, grad_out, value, key, grad_query, const_cast<void *>(attn), dS, B, C, d, H, W, rows, halo_top,
                                 0, H, dtype, st))
        return e;
    if (int e = launch_gath_mma(query, dS, grad_key, B, d, H, W, halo_top, halo_bottom, dtype, st)) return e;
    return launch_gath_mma(grad_out, attn, grad_value, B, C, H, W, halo_top, halo_bottom, dtype, st);
}

// ------------------------------------------------------------------ backward without any allocation
// Some callers cannot hand this library a workspace because they cannot allocate device memory at the point
// of the call: inference engines that size every buffer when the engine is built and run under that fixed memory
// plan, plugin hosts whose allocator is not reachable from the op, and real-time loops that forbid cudaMalloc
// after start-up because it synchronises the device.
// For them the logit-gradient scratch of the backward pass lives in a file-scope device array that every GPU
// loading this library holds until the process exits.
constexpr size_t kStaticScratchBytes = 16u << 20;     // 16 MiB: config-2-sized float32 problems (13.1 MB) fit
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// The array's name is only a host-side handle; kernels need its device address, looked up once per device
// while that device is current.
static int static_scratch_address(void **out) {
    constexpr int kMaxDevices = 64;
    static void *cache[kMaxDevices] = {};
    static std::mutex lock;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    SAPA_REQUIRE(e == cudaSuccess, SAPA_ERR_LAUNCH, "sapa_fused_backward_static: cudaGetDevice failed: %s", cudaGetErrorString(e));
    SAPA_REQUIRE(dev >= 0 && dev < kMaxDevices, SAPA_ERR_ARGUMENT, "sapa_fused_backward_static: device index %d out of range", dev);
    std::lock_guard<std::mutex> guard(lock);
    if (cache[dev] == nullptr) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        SAPA_REQUIRE(e == cudaSuccess && p != nullptr, SAPA_ERR_LAUNCH,
                     "sapa_fused_backward_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        cache[dev] = p;
    }
    *out = cache[dev];
    return SAPA_OK;
}

size_t sapa_fused_backward_static_capacity(void) { return kStaticScratchBytes; }

int sapa_fused_backward_static(const void *grad_out, const void *query, const void *key, const void *value, const void *attn,
                               void *grad_query, void *grad_key, void *grad_value, int B, int d, int C, int H, int W, int K,
                               int s, int dtype, void *stream) {
    const size_t need = sapa_fused_backward_workspace(B, H, W, K, s, dtype);
    SAPA_REQUIRE(need != 0, SAPA_ERR_ARGUMENT, "sapa_fused_backward_static: sizes must be positive and the dtype known");
    SAPA_REQUIRE(need <= kStaticScratchBytes, SAPA_ERR_WORKSPACE,
                 "sapa_fused_backward_static: the problem needs %zu bytes of scratch but the built-in buffer holds %zu; "
                 "use sapa_fused_backward with a caller-provided workspace",
                 need, kStaticScratchBytes);
    void *scratch = nullptr;
    if (int e = static_scratch_address(&scratch)) return e;
    // The scratch is written in full (gradient of the logits) before any kernel reads it, so nothing has to be
    // cleared between calls; it simply keeps the last call's values.
    return sapa_fused_backward(grad_out, query, key, value, attn, grad_query, grad_key, grad_value, scratch,
                               kStaticScratchBytes, B, d, C, H, W, K, s, dtype, stream);
}

}  // extern "C"
