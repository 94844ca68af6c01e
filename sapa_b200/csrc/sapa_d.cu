// sapa_d.cu — SAPA-D (deformable) kernels: similarity and aggregation at per-pixel learned sampling
// points, forward and backward, plus the fused forward.
//
// Every high-res pixel (qh, qw) samples, for each group g and point p, the low-res key / value plane at
//   (h, w) = (qh / s + off_h, qw / s + off_w)          off_w = offset[b, 2(gP+p)], off_h = offset[b, 2(gP+p)+1]
// bilinearly; a corner outside the plane reads 0 and a point outside (-1,H) x (-1,W) contributes nothing
// (forward and backward).  Because the sampling positions are data dependent the key/value gradients are a
// scatter: they use float atomics into a float32 (float64 for f64) accumulation buffer.  The gradients of
// the query, the attention and the offsets are owned by one thread each and written without atomics
// (query: P threads of a group add to one element, so it accumulates too).
#include "common.cuh"

namespace sapa {

constexpr int MAXP = 16;   // largest num_point handled by the fused kernel

// Bilinear footprint of one sampling point in an H x W plane.
template <typename A>
struct Bilinear {
    int i00, i01, i10, i11;   // plane offsets of the four corners, -1 when the corner is outside
    A w00, w01, w10, w11;     // corner weights
    A lh, lw;                 // fractional parts (for the offset derivatives)
    bool inside;              // the reference's outer guard: -1 < h < H and -1 < w < W

    __device__ __forceinline__ void setup(A h, A w, int H, int W) {
        inside = (h > A(-1)) && (h < A(H)) && (w > A(-1)) && (w < A(W));
        const A fh = floor(h), fw = floor(w);
        const int h0 = (int)fh, w0 = (int)fw, h1 = h0 + 1, w1 = w0 + 1;
        lh = h - fh;
        lw = w - fw;
        const A hh = A(1) - lh, hw = A(1) - lw;
        w00 = hh * hw; w01 = hh * lw; w10 = lh * hw; w11 = lh * lw;
        const bool t = h0 >= 0, b = h1 <= H - 1, l = w0 >= 0, r = w1 <= W - 1;
        i00 = (inside && t && l) ? h0 * W + w0 : -1;
        i01 = (inside && t && r) ? h0 * W + w1 : -1;
        i10 = (inside && b && l) ? h1 * W + w0 : -1;
        i11 = (inside && b && r) ? h1 * W + w1 : -1;
    }
    template <typename T>
    __device__ __forceinline__ void corners(const T *__restrict__ plane, A &v00, A &v01, A &v10, A &v11) const {
        v00 = i00 >= 0 ? to_acc(__ldg(plane + i00)) : A(0);
        v01 = i01 >= 0 ? to_acc(__ldg(plane + i01)) : A(0);
        v10 = i10 >= 0 ? to_acc(__ldg(plane + i10)) : A(0);
        v11 = i11 >= 0 ? to_acc(__ldg(plane + i11)) : A(0);
    }
    template <typename T>
    __device__ __forceinline__ A sample(const T *__restrict__ plane) const {
        A v00, v01, v10, v11;
        corners(plane, v00, v01, v10, v11);
        return w00 * v00 + w01 * v01 + w10 * v10 + w11 * v11;
    }
};

// ---------------------------------------------------------------------------------- forward, separate ops

// one thread per (b, k = g*P+p, qh, qw)
template <typename T>
__global__ void deform_qk_fwd_kernel(const T *__restrict__ query, const T *__restrict__ key, const T *__restrict__ offset,
                                     T *__restrict__ out, int B, int Cq, int H, int W, int P, int s, int G) {
    using A = typename AccOf<T>::type;
    const int sH = s * H, sW = s * W, AC = G * P, gc = Cq / G;
    const size_t hi = (size_t)sH * sW, lo = (size_t)H * W;
    const long long total = (long long)B * AC * hi;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const size_t pix = (size_t)(i % hi);
        const int qw = (int)(pix % sW), qh = (int)(pix / sW);
        const int k = (int)((i / hi) % AC);
        const int b = (int)(i / (hi * AC));
        const int g = k / P;
        const T *op = offset + ((size_t)b * AC + k) * 2 * hi + pix;
        Bilinear<A> bl;
        bl.setup(A(qh / s) + to_acc(op[hi]), A(qw / s) + to_acc(op[0]), H, W);
        A acc = 0;
        if (bl.inside) {
            const T *qp = query + ((size_t)b * Cq + (size_t)g * gc) * hi + pix;
            const T *kp = key + ((size_t)b * Cq + (size_t)g * gc) * lo;
            for (int c = 0; c < gc; ++c) acc += bl.sample(kp + (size_t)c * lo) * to_acc(qp[(size_t)c * hi]);
        }
        out[i] = from_acc<T>(acc);
    }
}

// one thread per (b, chunk of CPT channels of one group, qh, qw): sampling set-up shared by CPT channels
template <typename T, int CPT>
__global__ void deform_av_fwd_kernel(const T *__restrict__ attn, const T *__restrict__ value, const T *__restrict__ offset,
                                     T *__restrict__ out, int B, int C, int H, int W, int P, int s, int G) {
    using A = typename AccOf<T>::type;
    const int sH = s * H, sW = s * W, AC = G * P, gc = C / G;
    const int chunks = (gc + CPT - 1) / CPT;
    const size_t hi = (size_t)sH * sW, lo = (size_t)H * W;
    const long long total = (long long)B * G * chunks * hi;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const size_t pix = (size_t)(i % hi);
        const int qw = (int)(pix % sW), qh = (int)(pix / sW);
        long long t = i / hi;
        const int ck = (int)(t % chunks); t /= chunks;
        const int g = (int)(t % G);
        const int b = (int)(t / G);
        const int c0 = g * gc + ck * CPT;
        const int nc = min(CPT, gc - ck * CPT);
        A o[CPT];
#pragma unroll
        for (int j = 0; j < CPT; ++j) o[j] = 0;
        const T *vp = value + ((size_t)b * C + c0) * lo;
        for (int p = 0; p < P; ++p) {
            const size_t k = (size_t)b * AC + (size_t)g * P + p;
            Bilinear<A> bl;
            bl.setup(A(qh / s) + to_acc(offset[k * 2 * hi + hi + pix]), A(qw / s) + to_acc(offset[k * 2 * hi + pix]), H, W);
            if (!bl.inside) continue;
            const A a = to_acc(attn[k * hi + pix]);
#pragma unroll
            for (int j = 0; j < CPT; ++j)
                if (j < nc) o[j] += bl.sample(vp + (size_t)j * lo) * a;
        }
#pragma unroll
        for (int j = 0; j < CPT; ++j)
            if (j < nc) out[((size_t)b * C + c0 + j) * hi + pix] = from_acc<T>(o[j]);
    }
}

// ---------------------------------------------------------------------------------- forward, fused
// A block of 32 x FY threads handles 32 consecutive pixels of one (image, group).  Phase 1: thread (x, y) computes
// the logits of points y, y + FY, ... of pixel x and leaves them, with the sampling positions, in shared memory.
// Phase 2: every thread normalises the P logits of its pixel (softmax over the points) and aggregates the value
// channels y*CPT .. of the group, CPT at a time.  The attention reaches HBM only if `attn_out` is given.
constexpr int FY = 8;

template <typename T, int CPT>
__global__ void __launch_bounds__(32 * FY)
deform_fused_fwd_kernel(const T *__restrict__ query, const T *__restrict__ key, const T *__restrict__ value,
                        const T *__restrict__ offset, T *__restrict__ out, T *__restrict__ attn_out,
                        int B, int Cq, int C, int H, int W, int P, int s, int G, int pix_blocks) {
    __shared__ float s_a[MAXP][32], s_h[MAXP][32], s_w[MAXP][32];
    const int sH = s * H, sW = s * W, AC = G * P, gq = Cq / G, gc = C / G;
    const size_t hi = (size_t)sH * sW, lo = (size_t)H * W;
    const int tx = threadIdx.x, ty = threadIdx.y;
    long long blk = blockIdx.x;
    const int pb = (int)(blk % pix_blocks); blk /= pix_blocks;
    const int g = (int)(blk % G);
    const int b = (int)(blk / G);
    const size_t pix = (size_t)pb * 32 + tx;
    const bool live = pix < hi;
    const int qw = live ? (int)(pix % sW) : 0, qh = live ? (int)(pix / sW) : 0;

    // phase 1: logits
    if (live) {
        const T *qp = query + ((size_t)b * Cq + (size_t)g * gq) * hi + pix;
        const T *kp = key + ((size_t)b * Cq + (size_t)g * gq) * lo;
        const T *op = offset + ((size_t)b * AC + (size_t)g * P) * 2 * hi + pix;
        for (int p = ty; p < P; p += FY) {
            const float w = float(qw / s) + to_acc(op[(size_t)(2 * p) * hi]);
            const float h = float(qh / s) + to_acc(op[(size_t)(2 * p + 1) * hi]);
            Bilinear<float> bl;
            bl.setup(h, w, H, W);
            float acc = 0.f;
            if (bl.inside)
                for (int c = 0; c < gq; ++c) acc += bl.sample(kp + (size_t)c * lo) * to_acc(qp[(size_t)c * hi]);
            s_a[p][tx] = acc;
            s_h[p][tx] = h;
            s_w[p][tx] = w;
        }
    }
    __syncthreads();
    if (!live) return;

    // phase 2: softmax over the points (every thread of the pixel's column does the same few operations)
    float m = -INFINITY;
    for (int p = 0; p < P; ++p) m = fmaxf(m, s_a[p][tx]);
    float z = 0.f;
    for (int p = 0; p < P; ++p) z += expf(s_a[p][tx] - m);
    const float inv = 1.f / z;
    if (attn_out != nullptr)
        for (int p = ty; p < P; p += FY)
            attn_out[((size_t)b * AC + (size_t)g * P + p) * hi + pix] = from_acc<T>(expf(s_a[p][tx] - m) * inv);

    for (int c0 = ty * CPT; c0 < gc; c0 += FY * CPT) {
        const T *vp = value + ((size_t)b * C + (size_t)g * gc + c0) * lo;
        const int nc = min(CPT, gc - c0);
        float o[CPT];
#pragma unroll
        for (int j = 0; j < CPT; ++j) o[j] = 0.f;
        for (int p = 0; p < P; ++p) {
            Bilinear<float> bl;
            bl.setup(s_h[p][tx], s_w[p][tx], H, W);
            if (!bl.inside) continue;
            const float a = expf(s_a[p][tx] - m) * inv;
#pragma unroll
            for (int j = 0; j < CPT; ++j)
                if (j < nc) o[j] += bl.sample(vp + (size_t)j * lo) * a;
        }
#pragma unroll
        for (int j = 0; j < CPT; ++j)
            if (j < nc) out[((size_t)b * C + (size_t)g * gc + c0 + j) * hi + pix] = from_acc<T>(o[j]);
    }
}

// ---------------------------------------------------------------------------------- backward
// one thread per (b, k, qh, qw), looping over the channels of group g(k).
//   QK: top = dS[b,k,pix], weight_c = Q[b,c,pix]:   dQ_c += top*val_c (atomic), dKey_c[corner] += w*top*Q_c (atomic)
//   AV: top_c = dOut[b,c,pix], weight = A[b,k,pix]: dA = sum_c top_c*val_c,     dV_c[corner]   += w*top_c*A (atomic)
// and in both: dOff_w = sum_c (d val_c / d w) * top * weight, dOff_h likewise.
template <typename T, bool IS_QK>
__global__ void deform_bwd_kernel(const T *__restrict__ top, const T *__restrict__ hires /* Q | A */,
                                  const T *__restrict__ plane_src /* Key | V */, const T *__restrict__ offset,
                                  typename AccOf<T>::type *__restrict__ grad_hi_acc /* dQ (QK only) */,
                                  T *__restrict__ grad_attn /* dA (AV only) */,
                                  typename AccOf<T>::type *__restrict__ grad_plane /* dKey | dV */,
                                  T *__restrict__ grad_offset, int B, int Cc, int H, int W, int P, int s, int G) {
    using A = typename AccOf<T>::type;
    const int sH = s * H, sW = s * W, AC = G * P, gc = Cc / G;
    const size_t hi = (size_t)sH * sW, lo = (size_t)H * W;
    const long long total = (long long)B * AC * hi;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const size_t pix = (size_t)(i % hi);
        const int qw = (int)(pix % sW), qh = (int)(pix / sW);
        const int k = (int)((i / hi) % AC);
        const int b = (int)(i / (hi * AC));
        const int g = k / P;
        const size_t off_idx = ((size_t)b * AC + k) * 2 * hi + pix;
        Bilinear<A> bl;
        bl.setup(A(qh / s) + to_acc(offset[off_idx + hi]), A(qw / s) + to_acc(offset[off_idx]), H, W);
        A g_w = 0, g_h = 0, g_attn = 0;
        if (bl.inside) {
            const A hh = A(1) - bl.lh, hw = A(1) - bl.lw;
            const size_t ch0 = (size_t)b * Cc + (size_t)g * gc;
            const A top_k = IS_QK ? to_acc(top[i]) : A(0);
            const A wt_k = IS_QK ? A(0) : to_acc(hires[i]);
            for (int c = 0; c < gc; ++c) {
                const T *pl = plane_src + (ch0 + c) * lo;
                A v00, v01, v10, v11;
                bl.corners(pl, v00, v01, v10, v11);
                const A val = bl.w00 * v00 + bl.w01 * v01 + bl.w10 * v10 + bl.w11 * v11;
                A t, wt;
                if (IS_QK) {
                    t = top_k;
                    wt = to_acc(hires[(ch0 + c) * hi + pix]);
                    atomic_add(grad_hi_acc + (ch0 + c) * hi + pix, t * val);
                } else {
                    t = to_acc(top[(ch0 + c) * hi + pix]);
                    wt = wt_k;
                    g_attn += t * val;
                }
                const A tw = t * wt;
                A *gp = grad_plane + (ch0 + c) * lo;
                if (bl.i00 >= 0) atomic_add(gp + bl.i00, bl.w00 * tw);
                if (bl.i01 >= 0) atomic_add(gp + bl.i01, bl.w01 * tw);
                if (bl.i10 >= 0) atomic_add(gp + bl.i10, bl.w10 * tw);
                if (bl.i11 >= 0) atomic_add(gp + bl.i11, bl.w11 * tw);
                g_w += (-hh * v00 + hh * v01 - bl.lh * v10 + bl.lh * v11) * tw;
                g_h += (-hw * v00 - bl.lw * v01 + hw * v10 + bl.lw * v11) * tw;
            }
        }
        grad_offset[off_idx] = from_acc<T>(g_w);
        grad_offset[off_idx + hi] = from_acc<T>(g_h);
        if (!IS_QK) grad_attn[i] = from_acc<T>(g_attn);
    }
}

// ---------------------------------------------------------------------------------- forward, dense-window path
// With s = 2 and offsets inside [-2, 2) a sampling point's four corners lie in the 5 x 5 low-res window around the
// pixel's parent - the window of SAPA-B.  Then both contractions of SAPA-D are SAPA-B contractions:
//   logits:      sim_p = sum_c q_c * bilinear(key_c) = sum_corners w_corner * D[corner],  D[cell] = sum_c q_c key_c[cell]
//                (D = the dense 25-slot similarity of the group's 16 channels, one call of the SAPA-B logit kernel with
//                the B x G groups as images);
//   aggregation: out_c = sum_p a_p * bilinear(value_c) = sum_cells Wd[cell] * value_c[cell],  Wd[cell] = sum of a_p * w_corner
//                over the corners that land on the cell (one call of the SAPA-B aggregation kernel).
// deform_window_kernel sits between the two: one thread per (image, group, pixel) turns D and the offsets into the
// attention over the P points and the dense window weights Wd (the thread's two windows sit in its column of a shared
// array, where the four cells of a point can be addressed at run time).  A point with a corner outside the window
// (|offset| >= 2) is an "outlier": its logit is gathered directly here, it adds nothing to Wd, and its pixel is
// appended to a list from which deform_outlier_kernel adds the contribution to the output afterwards (rare for learned
// offsets, but always correct).  Points outside the image contribute exactly 0 to the logits and to the output, as in
// the reference.
constexpr int WIN_THREADS = 128;

// One entry per (image, group, pixel) that has at least one point outside its window: the points as a bit mask and
// the attention weights of all points of the pixel.
struct OutlierTap {
    unsigned int idx;    // (image * G + group) * sH * sW + high-res pixel
    unsigned int mask;   // bit p: point p left the window
    float a[MAXP];       // attention weight of every point (only the masked ones are read)
};

// Position of a sampling point relative to the window of its pixel: r0 / c0 = window row / column of the upper-left
// corner, lh / lw the fractional parts; `dense` = all four corners are window cells, `inside` = the reference's guard.
struct WindowTap {
    int r0, c0;
    float lh, lw;
    bool inside, dense;
    __device__ __forceinline__ void setup(float h, float w, int H, int W, int py, int px) {
        inside = (h > -1.f) && (h < float(H)) && (w > -1.f) && (w < float(W));
        const float fh = floorf(h), fw = floorf(w);
        lh = h - fh; lw = w - fw;
        r0 = (int)fh - (py - 2); c0 = (int)fw - (px - 2);
        dense = inside && r0 >= 0 && r0 <= 3 && c0 >= 0 && c0 <= 3;
    }
};

// NP = number of points known at compile time (0: read P at run time, up to MAXP).
// MODE: WIN_FUSED = logits -> softmax -> window weights (the fused op); WIN_LOGITS = raw logits only, written where the
// fused op writes the attention (deform_qk); WIN_WEIGHTS = window weights from a given attention map (deform_av).
constexpr int WIN_FUSED = 0, WIN_LOGITS = 1, WIN_WEIGHTS = 2;

// The two 25-slot windows of a thread (similarity in, window weights out) live in shared memory, column = thread, so
// every access is conflict-free: a point touches four cells of each window, and shared memory can be indexed with the
// cell computed at run time (a register array cannot: that form multiplies every point with all 25 cells and took
// 82 us where this takes 56 us at B=8, 4 groups, 128 x 128 pixels).  Two passes over the points: logits and their
// maximum, then exp and the window weights.  Six blocks per SM (80 registers; 4 and 8 measured slower).
template <typename T, int NP, int MODE>
__global__ void __launch_bounds__(WIN_THREADS, 6)
deform_window_kernel(const T *__restrict__ query, const T *__restrict__ key, const T *__restrict__ offset,
                          const float *__restrict__ dense, T *__restrict__ attn, T *__restrict__ window,
                          OutlierTap *__restrict__ taps, unsigned int *__restrict__ tap_count, int B, int Cq, int H, int W,
                          int P_runtime, int G, int rows, int ytop) {
    constexpr int PMAX = NP > 0 ? NP : MAXP;
    __shared__ float sd[MODE != WIN_WEIGHTS ? 25 : 1][WIN_THREADS];     // dense similarity of the thread's pixel
    __shared__ float sw[MODE != WIN_LOGITS ? 25 : 1][WIN_THREADS];      // window weights being collected
    const int P = NP > 0 ? NP : P_runtime;
    const int sH = 2 * H, sW = 2 * W, gq = Cq / G;
    const size_t hi = (size_t)sH * sW, lo = (size_t)rows * W;
    const int lane = threadIdx.x & 31, tid = threadIdx.x;
    const long long total = (long long)B * G * hi;
    for (long long i0 = (long long)blockIdx.x * WIN_THREADS; i0 < total; i0 += (long long)gridDim.x * WIN_THREADS) {
        const long long i = i0 + tid;
        const bool live = i < total;
        const size_t pix = live ? (size_t)(i % hi) : 0;
        const long long bg = live ? i / (long long)hi : 0;
        const int g = (int)(bg % G), b = (int)(bg / G);
        const int qw = (int)(pix % sW), qh = (int)(pix / sW), py = (qh >> 1) + ytop, px = qw >> 1;
        if (MODE != WIN_WEIGHTS) {
            const float *dp = dense + (size_t)bg * 25 * hi + pix;
#pragma unroll
            for (int k = 0; k < 25; ++k) sd[k][tid] = live ? __ldcs(dp + (size_t)k * hi) : 0.f;
        }
        if (MODE != WIN_LOGITS) {
#pragma unroll
            for (int k = 0; k < 25; ++k) sw[k][tid] = 0.f;
        }
        float oh[PMAX], ow[PMAX], logit[PMAX];
        const T *offp = offset + (size_t)bg * P * 2 * hi + pix;
#pragma unroll
        for (int p = 0; p < PMAX; ++p) {
            const bool on = live && p < P;
            ow[p] = on ? float(px) + to_acc(__ldg(offp + (size_t)(2 * p) * hi)) : 0.f;
            oh[p] = on ? float(py) + to_acc(__ldg(offp + (size_t)(2 * p + 1) * hi)) : 0.f;
        }
        unsigned int outliers = 0;
        float m = -INFINITY;
        // ---- pass 1: logits (or the given attention) and which points leave the window
#pragma unroll
        for (int p = 0; p < PMAX; ++p) {
            logit[p] = 0.f;
            if (live && p < P) {
                WindowTap t;
                t.setup(oh[p], ow[p], rows, W, py, px);
                if (!t.dense && t.inside) outliers |= 1u << p;
                float acc = 0.f;
                if (MODE == WIN_WEIGHTS) {
                    acc = to_acc(__ldg(attn + ((size_t)bg * P + p) * hi + pix));
                } else if (t.dense) {
                    const int c = t.r0 * 5 + t.c0;
                    const float top = (1.f - t.lw) * sd[c][tid] + t.lw * sd[c + 1][tid];
                    const float bot = (1.f - t.lw) * sd[c + 5][tid] + t.lw * sd[c + 6][tid];
                    acc = (1.f - t.lh) * top + t.lh * bot;
                } else if (t.inside) {        // outlier: gather the key directly
                    Bilinear<float> bl;
                    bl.setup(oh[p], ow[p], rows, W);
                    const T *qp = query + ((size_t)b * Cq + (size_t)g * gq) * hi + pix;
                    const T *kp = key + ((size_t)b * Cq + (size_t)g * gq) * lo;
                    for (int ch = 0; ch < gq; ++ch) acc += bl.sample(kp + (size_t)ch * lo) * to_acc(qp[(size_t)ch * hi]);
                }
                logit[p] = acc;
                m = fmaxf(m, acc);
                if (MODE == WIN_LOGITS) attn[((size_t)bg * P + p) * hi + pix] = from_acc<T>(acc);
            }
        }
        if (MODE == WIN_LOGITS) continue;                   // no lane-crossing operation below was entered by any lane yet
        // ---- pass 2: exp and the window weights (the bilinear set-up is recomputed: cheaper than keeping it)
        float z = 0.f;
#pragma unroll
        for (int p = 0; p < PMAX; ++p) {
            if (live && p < P) {
                const float e = MODE == WIN_WEIGHTS ? logit[p] : __expf(logit[p] - m);
                logit[p] = e;
                z += e;
                WindowTap t;
                t.setup(oh[p], ow[p], rows, W, py, px);
                if (t.dense) {
                    const int c = t.r0 * 5 + t.c0;
                    const float et = e * (1.f - t.lh), eb = e * t.lh;
                    sw[c][tid] += et * (1.f - t.lw);
                    sw[c + 1][tid] += et * t.lw;
                    sw[c + 5][tid] += eb * (1.f - t.lw);
                    sw[c + 6][tid] += eb * t.lw;
                }
            }
        }
        const float inv = MODE == WIN_WEIGHTS ? 1.f : 1.f / z;
        if (live) {
            T *wp = window + (size_t)bg * 25 * hi + pix;
#pragma unroll
            for (int k = 0; k < 25; ++k) wp[(size_t)k * hi] = from_acc<T>(sw[k][tid] * inv);
        }
        if (MODE == WIN_FUSED) {
#pragma unroll
            for (int p = 0; p < PMAX; ++p) {
                logit[p] *= inv;                             // the attention weight of the point
                if (live && p < P && attn != nullptr) attn[((size_t)bg * P + p) * hi + pix] = from_acc<T>(logit[p]);
            }
        }
        // append the pixels of this warp that have outlier points to the list: one counter update per warp
        const unsigned int any = __ballot_sync(0xffffffffu, outliers != 0);
        if (any != 0) {
            unsigned int base = 0;
            if (lane == 0) base = atomicAdd(tap_count, (unsigned int)__popc(any));
            base = __shfl_sync(0xffffffffu, base, 0);
            if (outliers != 0) {
                OutlierTap *t = taps + base + __popc(any & ((1u << lane) - 1u));
                t->idx = (unsigned int)i;
                t->mask = outliers;
#pragma unroll
                for (int p = 0; p < PMAX; ++p) t->a[p] = logit[p];
            }
        }
    }
}

// Adds a_p * bilinear(value_c) of the listed outlier points to the output.  Eight threads per listed pixel: each takes
// every eighth channel of the group, four channels at a time in registers, walks the pixel's outlier points for them
// and then updates the output elements once, read-modify-write without atomics (a listed pixel of a group belongs to
// exactly one thread group, and the aggregation kernel that wrote the output has finished): the forward pass is
// deterministic and a 16-bit output is rounded once more, not once per point.
template <typename T>
__global__ void deform_outlier_kernel(const OutlierTap *__restrict__ taps, const unsigned int *__restrict__ tap_count,
                                      const T *__restrict__ value, const T *__restrict__ offset, T *__restrict__ out,
                                      int C, int H, int W, int P, int G, int rows, int ytop) {
    constexpr int CH = 4;
    const int sW = 2 * W, gc = C / G;
    const size_t hi = (size_t)(2 * H) * sW, lo = (size_t)rows * W;
    const unsigned int n = *tap_count;
    const int sub = threadIdx.x & 7;
    for (unsigned int e = (blockIdx.x * blockDim.x + threadIdx.x) >> 3; e < n; e += (gridDim.x * blockDim.x) >> 3) {
        const OutlierTap *t = taps + e;
        const unsigned int idx = __ldg(&t->idx), mask = __ldg(&t->mask);
        const size_t bg = idx / hi, pix = idx % hi;
        const int px = (int)(pix % sW) >> 1, py = ((int)(pix / sW) >> 1) + ytop;
        const T *offp = offset + bg * P * 2 * hi + pix;
        const T *vp = value + bg * gc * lo;
        T *op = out + bg * gc * hi + pix;
        for (int c0 = sub; c0 < gc; c0 += 8 * CH) {
            float acc[CH];
#pragma unroll
            for (int j = 0; j < CH; ++j) acc[j] = 0.f;
            for (unsigned int m = mask; m != 0; m &= m - 1) {
                const int p = __ffs(m) - 1;
                const float w = float(px) + to_acc(__ldg(offp + (size_t)(2 * p) * hi));
                const float h = float(py) + to_acc(__ldg(offp + (size_t)(2 * p + 1) * hi));
                const float a = __ldg(&t->a[p]);
                Bilinear<float> bl;
                bl.setup(h, w, rows, W);
#pragma unroll
                for (int j = 0; j < CH; ++j) {
                    const int c = c0 + 8 * j;
                    if (c < gc) acc[j] += a * bl.sample(vp + (size_t)c * lo);
                }
            }
#pragma unroll
            for (int j = 0; j < CH; ++j) {
                const int c = c0 + 8 * j;
                if (c < gc) op[(size_t)c * hi] = from_acc<T>(to_acc(op[(size_t)c * hi]) + acc[j]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------- backward, dense-window path
// The forward identities read backwards (B_p = the 25-vector of bilinear weights of point p, vy (x) vx):
//   dWd[cell]   = sum_c dOut_c * value_c[cell]              = sim(dOut, value) per group           (SAPA-B logit kernel)
//   dA_p        = sum_cells B_p[cell] * dWd[cell];   dS_p = A_p * (dA_p - sum_q A_q dA_q)           (softmax over the points)
//   dD[cell]    = sum_p dS_p * B_p[cell],  Wd[cell] = sum_p A_p * B_p[cell]
//   dQ = agg(dD, key),  dKey = gath(Q, dD),  dV = gath(dOut, Wd)  per group                         (SAPA-B kernels, no atomics)
//   d offset_p  = A_p * (dB_p . dWd) + dS_p * (dB_p . D),   dB_p/dh = dvy (x) vx,  dB_p/dw = vy (x) dvx
// deform_window_bwd_kernel does the per-pixel part (one thread per (image, group, pixel); the windows in shared memory).
// Points that leave the window are listed with their A_p and dS_p; deform_outlier_bwd_kernel adds their gradients
// afterwards (atomics on dQ, dKey, dV; it owns their offset gradients).
struct OutlierGrad {
    unsigned int k;      // (image * G + group) * P + point
    unsigned int pix;    // high-res pixel
    float a;             // attention weight of the point
    float ds;            // gradient of its logit
};


// MODE: BWD_FUSED = the whole chain; BWD_AV = backward of deform_av alone (`attn` given, dA written to `ddense`'s place
// is not needed: it goes to `grad_attn`, no logit gradients); BWD_QK = backward of deform_qk alone (`attn` carries the
// logit gradients dS, no aggregation part).
constexpr int BWD_FUSED = 0, BWD_AV = 1, BWD_QK = 2;

template <typename T, int NP, int MODE>
__global__ void __launch_bounds__(WIN_THREADS, 4)
deform_window_bwd_kernel(const T *__restrict__ grad_out, const T *__restrict__ value, const T *__restrict__ offset,
                         const T *__restrict__ attn, const float *__restrict__ dense /* D [B*G, 25, hi] */,
                         const float *__restrict__ dwin /* dWd [B*G, 25, hi] */, T *__restrict__ ddense /* dD, out */,
                         T *__restrict__ window /* Wd, out */, T *__restrict__ grad_offset, T *__restrict__ grad_attn /* BWD_AV only */,
                         OutlierGrad *__restrict__ taps,
                         unsigned int *__restrict__ tap_count, int B, int C, int H, int W, int P_runtime, int G) {
    constexpr int PMAX = NP > 0 ? NP : MAXP;
    const int P = NP > 0 ? NP : P_runtime;
    const int sH = 2 * H, sW = 2 * W, gc = C / G;
    const size_t hi = (size_t)sH * sW, lo = (size_t)H * W;
    // The two 25-slot windows of a thread (D and dWd going in, dD and Wd coming out) live in shared memory, column =
    // thread (conflict-free): a point touches four cells of each, and shared memory can be indexed with the cell found
    // at run time, where registers force a product with all 25 cells.
    __shared__ float sd[25][WIN_THREADS], sw[25][WIN_THREADS];
    const int lane = threadIdx.x & 31, tid = threadIdx.x;
    const long long total = (long long)B * G * hi;
    for (long long i0 = (long long)blockIdx.x * WIN_THREADS; i0 < total; i0 += (long long)gridDim.x * WIN_THREADS) {
        const long long i = i0 + threadIdx.x;
        const bool live = i < total;
        const size_t pix = live ? (size_t)(i % hi) : 0;
        const long long bg = live ? i / (long long)hi : 0;
        const int qw = (int)(pix % sW), qh = (int)(pix / sW), py = qh >> 1, px = qw >> 1;
        float oh[PMAX], ow[PMAX], at[PMAX];
        const float *dp = dense + (size_t)bg * 25 * hi + pix, *wp = dwin + (size_t)bg * 25 * hi + pix;
#pragma unroll
        for (int k = 0; k < 25; ++k) {
            sd[k][tid] = (MODE != BWD_AV && live) ? __ldcs(dp + (size_t)k * hi) : 0.f;
            sw[k][tid] = (MODE != BWD_QK && live) ? __ldcs(wp + (size_t)k * hi) : 0.f;
        }
        const T *offp = offset + (size_t)bg * P * 2 * hi + pix, *ap = attn + (size_t)bg * P * hi + pix;
#pragma unroll
        for (int p = 0; p < PMAX; ++p) {
            const bool on = live && p < P;
            ow[p] = on ? float(px) + to_acc(__ldg(offp + (size_t)(2 * p) * hi)) : 0.f;
            oh[p] = on ? float(py) + to_acc(__ldg(offp + (size_t)(2 * p + 1) * hi)) : 0.f;
            at[p] = on ? to_acc(__ldg(ap + (size_t)p * hi)) : 0.f;
        }
        // ---- pass 1: dA_p and the four bilinear forms of the offset gradients
        float da[PMAX], gh1[PMAX], gw1[PMAX], gh2[PMAX], gw2[PMAX];
        float dot = 0.f;
        unsigned int outliers = 0;
#pragma unroll
        for (int p = 0; p < PMAX; ++p) {
            da[p] = 0.f; gh1[p] = 0.f; gw1[p] = 0.f; gh2[p] = 0.f; gw2[p] = 0.f;
            if (live && p < P) {
                WindowTap t;
                t.setup(oh[p], ow[p], H, W, py, px);
                if (t.dense) {
                    // bilinear forms over the four cells: value (1-lh, lh) x (1-lw, lw); d/dh (-1, 1) x (1-lw, lw); d/dw (1-lh, lh) x (-1, 1)
                    const int c = t.r0 * 5 + t.c0;
                    const float hw = 1.f - t.lw, hh = 1.f - t.lh;
                    if (MODE != BWD_QK) {
                        const float w00 = sw[c][tid], w01 = sw[c + 1][tid], w10 = sw[c + 5][tid], w11 = sw[c + 6][tid];
                        const float top = hw * w00 + t.lw * w01, bot = hw * w10 + t.lw * w11;
                        da[p] = hh * top + t.lh * bot;
                        gh1[p] = bot - top;
                        gw1[p] = (hh * w01 + t.lh * w11) - (hh * w00 + t.lh * w10);
                    }
                    if (MODE != BWD_AV) {
                        const float d00 = sd[c][tid], d01 = sd[c + 1][tid], d10 = sd[c + 5][tid], d11 = sd[c + 6][tid];
                        gh2[p] = (hw * d10 + t.lw * d11) - (hw * d00 + t.lw * d01);
                        gw2[p] = (hh * d01 + t.lh * d11) - (hh * d00 + t.lh * d10);
                    }
                } else if (t.inside) {        // outlier: dA by direct gather
                    outliers |= 1u << p;
                    if (MODE == BWD_QK) continue;
                    Bilinear<float> bl;
                    bl.setup(oh[p], ow[p], H, W);
                    const T *gp = grad_out + (size_t)bg * gc * hi + pix, *vp = value + (size_t)bg * gc * lo;
                    float acc = 0.f;
                    for (int c = 0; c < gc; ++c) acc += bl.sample(vp + (size_t)c * lo) * to_acc(gp[(size_t)c * hi]);
                    da[p] = acc;
                }
                dot += at[p] * da[p];
            }
        }
        // ---- pass 2: logit gradients, dD, Wd (the two shared windows become the accumulators), offset gradients
#pragma unroll
        for (int k = 0; k < 25; ++k) { sd[k][tid] = 0.f; sw[k][tid] = 0.f; }
        T *gop = grad_offset + (size_t)bg * P * 2 * hi + pix;
#pragma unroll
        for (int p = 0; p < PMAX; ++p) {
            if (live && p < P) {
                // BWD_QK: `attn` holds the logit gradients themselves; BWD_AV: no logit gradient, dA goes out as it is
                const float a = MODE == BWD_QK ? 0.f : at[p];
                const float ds = MODE == BWD_QK ? at[p] : MODE == BWD_AV ? 0.f : a * (da[p] - dot);
                if (MODE == BWD_AV) grad_attn[((size_t)bg * P + p) * hi + pix] = from_acc<T>(da[p]);
                da[p] = ds;
                WindowTap t;
                t.setup(oh[p], ow[p], H, W, py, px);
                if (t.dense) {
                    const int c = t.r0 * 5 + t.c0;
                    const float b00 = (1.f - t.lh) * (1.f - t.lw), b01 = (1.f - t.lh) * t.lw, b10 = t.lh * (1.f - t.lw), b11 = t.lh * t.lw;
                    if (MODE != BWD_AV) {
                        sd[c][tid] += ds * b00; sd[c + 1][tid] += ds * b01; sd[c + 5][tid] += ds * b10; sd[c + 6][tid] += ds * b11;
                    }
                    if (MODE != BWD_QK) {
                        sw[c][tid] += a * b00; sw[c + 1][tid] += a * b01; sw[c + 5][tid] += a * b10; sw[c + 6][tid] += a * b11;
                    }
                }
                if (!(outliers & (1u << p))) {      // the list kernel writes the offset gradients of the outliers
                    gop[(size_t)(2 * p) * hi] = from_acc<T>(a * gw1[p] + ds * gw2[p]);
                    gop[(size_t)(2 * p + 1) * hi] = from_acc<T>(a * gh1[p] + ds * gh2[p]);
                }
            }
        }
        if (live) {
            T *ddp = ddense + (size_t)bg * 25 * hi + pix, *wdp = window + (size_t)bg * 25 * hi + pix;
#pragma unroll
            for (int k = 0; k < 25; ++k) {
                if (MODE != BWD_AV) ddp[(size_t)k * hi] = from_acc<T>(sd[k][tid]);
                if (MODE != BWD_QK) wdp[(size_t)k * hi] = from_acc<T>(sw[k][tid]);
            }
        }
        const unsigned int any = __ballot_sync(0xffffffffu, outliers != 0);
        if (any != 0) {
            const int mine = __popc(outliers);
            int incl = mine;
#pragma unroll
            for (int sft = 1; sft < 32; sft <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, sft);
                if (lane >= sft) incl += up;
            }
            const int warp_total = __shfl_sync(0xffffffffu, incl, 31);
            unsigned int base = 0;
            if (lane == 0) base = atomicAdd(tap_count, (unsigned int)warp_total);
            base = __shfl_sync(0xffffffffu, base, 0);
            unsigned int pos = base + (unsigned int)(incl - mine);
#pragma unroll
            for (int p = 0; p < PMAX; ++p)
                if (outliers & (1u << p)) {
                    OutlierGrad t;
                    t.k = (unsigned int)(bg * P + p); t.pix = (unsigned int)pix; t.a = MODE == BWD_QK ? 0.f : at[p]; t.ds = da[p];
                    taps[pos++] = t;
                }
        }
    }
}

// Gradients of the listed outlier points: eight threads per point share its sampling set-up and take every eighth
// channel; dQ, dKey and dV are added to what the SAPA-B kernels wrote (atomics), the point's offset gradient is written.
// TA = type of the scatter targets grad_key / grad_value: T itself in float32; float for 16-bit tensors, where they are
// zeroed side buffers that deform_add_scatter_kernel folds into the 16-bit gradients afterwards (a 16-bit atomic per
// corner and channel was 2x slower than the whole float32 pass and rounds at every addition).
template <typename T, typename TA>
__global__ void deform_outlier_bwd_kernel(const OutlierGrad *__restrict__ taps, const unsigned int *__restrict__ tap_count,
                                          const T *__restrict__ grad_out, const T *__restrict__ query, const T *__restrict__ key,
                                          const T *__restrict__ value, const T *__restrict__ offset, T *__restrict__ grad_query,
                                          TA *__restrict__ grad_key, TA *__restrict__ grad_value, T *__restrict__ grad_offset,
                                          int Cq, int C, int H, int W, int P, int G) {
    const int sW = 2 * W, gq = Cq / G, gc = C / G;
    const size_t hi = (size_t)(2 * H) * sW, lo = (size_t)H * W;
    const unsigned int n = *tap_count;
    const int lane = threadIdx.x & 31, sub = lane & 7;
    const unsigned int group_mask = 0xffu << (lane & ~7);
    for (unsigned int e = (blockIdx.x * blockDim.x + threadIdx.x) >> 3; e < n; e += (gridDim.x * blockDim.x) >> 3) {
        const OutlierGrad t = taps[e];
        const size_t pix = t.pix;
        const int px = (int)(pix % sW) >> 1, py = (int)(pix / sW) >> 1;
        const float w = float(px) + to_acc(__ldg(offset + (size_t)t.k * 2 * hi + pix));
        const float h = float(py) + to_acc(__ldg(offset + (size_t)t.k * 2 * hi + hi + pix));
        Bilinear<float> bl;
        bl.setup(h, w, H, W);
        const float hh = 1.f - bl.lh, hw = 1.f - bl.lw;
        const size_t bg = t.k / (unsigned int)P;
        float g_w = 0.f, g_h = 0.f;
        for (int c = sub; c < gc && grad_value != nullptr; c += 8) {      // aggregation: dV scatter and its offset gradient
            float v00, v01, v10, v11;
            bl.corners(value + (bg * gc + c) * lo, v00, v01, v10, v11);
            const float tw = to_acc(grad_out[(bg * gc + c) * hi + pix]) * t.a;
            TA *gp = grad_value + (bg * gc + c) * lo;
            if (bl.i00 >= 0) atomicAdd(gp + bl.i00, from_acc<TA>(bl.w00 * tw));
            if (bl.i01 >= 0) atomicAdd(gp + bl.i01, from_acc<TA>(bl.w01 * tw));
            if (bl.i10 >= 0) atomicAdd(gp + bl.i10, from_acc<TA>(bl.w10 * tw));
            if (bl.i11 >= 0) atomicAdd(gp + bl.i11, from_acc<TA>(bl.w11 * tw));
            g_w += (-hh * v00 + hh * v01 - bl.lh * v10 + bl.lh * v11) * tw;
            g_h += (-hw * v00 - bl.lw * v01 + hw * v10 + bl.lw * v11) * tw;
        }
        for (int c = sub; c < gq && grad_query != nullptr; c += 8) {      // similarity: dQ, dKey scatter and its offset gradient
            float v00, v01, v10, v11;
            bl.corners(key + (bg * gq + c) * lo, v00, v01, v10, v11);
            atomicAdd(grad_query + (bg * gq + c) * hi + pix, from_acc<T>(t.ds * (bl.w00 * v00 + bl.w01 * v01 + bl.w10 * v10 + bl.w11 * v11)));
            const float tw = t.ds * to_acc(query[(bg * gq + c) * hi + pix]);
            TA *gp = grad_key + (bg * gq + c) * lo;
            if (bl.i00 >= 0) atomicAdd(gp + bl.i00, from_acc<TA>(bl.w00 * tw));
            if (bl.i01 >= 0) atomicAdd(gp + bl.i01, from_acc<TA>(bl.w01 * tw));
            if (bl.i10 >= 0) atomicAdd(gp + bl.i10, from_acc<TA>(bl.w10 * tw));
            if (bl.i11 >= 0) atomicAdd(gp + bl.i11, from_acc<TA>(bl.w11 * tw));
            g_w += (-hh * v00 + hh * v01 - bl.lh * v10 + bl.lh * v11) * tw;
            g_h += (-hw * v00 - bl.lw * v01 + hw * v10 + bl.lw * v11) * tw;
        }
#pragma unroll
        for (int sh = 1; sh < 8; sh <<= 1) {
            g_w += __shfl_xor_sync(group_mask, g_w, sh);
            g_h += __shfl_xor_sync(group_mask, g_h, sh);
        }
        if (sub == 0) {
            grad_offset[(size_t)t.k * 2 * hi + pix] = from_acc<T>(g_w);
            grad_offset[(size_t)t.k * 2 * hi + hi + pix] = from_acc<T>(g_h);
        }
    }
}

// dst[i] += side[i] for the 16-bit gradients whose outlier contributions were collected in float32; nothing to do (and
// nothing read) when the list was empty.
template <typename T>
__global__ void deform_add_scatter_kernel(const unsigned int *__restrict__ tap_count, T *__restrict__ dst_a,
                                          const float *__restrict__ side_a, size_t n_a, T *__restrict__ dst_b,
                                          const float *__restrict__ side_b, size_t n_b) {
    if (*tap_count == 0) return;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n_a + n_b; i += stride) {
        if (i < n_a) dst_a[i] = from_acc<T>(to_acc(dst_a[i]) + side_a[i]);
        else dst_b[i - n_a] = from_acc<T>(to_acc(dst_b[i - n_a]) + side_b[i - n_a]);
    }
}

// ---------------------------------------------------------------------------------- backward, fused
// Gradients of out = deform_av(softmax_p(deform_qk(q, k, off)), v, off) in ONE kernel.  One thread per (image, group,
// high-res pixel) walks the P points three times, with the per-point values parked in shared memory:
//   pass A (aggregation):  dA_p = sum_c dOut_c * val_c(p);  dV_c[corner] += w * dOut_c * A_p (atomic scatter);
//                          offset gradient of the aggregation;
//   pass B (softmax):      dS_p = A_p * (dA_p - sum_q A_q dA_q);
//   pass C (similarity):   dQ_c = sum_p dS_p * val_c(p) (this thread is the only writer: plain stores, deterministic);
//                          dKey_c[corner] += w * dS_p * Q_c (atomic scatter); offset gradient of the similarity.
// The two offset gradients are added here, so the offsets and the attention map are read once and no intermediate
// tensor ([B,G,P,sH,sW] attention gradient, logit gradient, second offset gradient) ever reaches HBM.
template <typename T, int NTHR>
__global__ void __launch_bounds__(NTHR)
deform_fused_bwd_kernel(const T *__restrict__ grad_out, const T *__restrict__ query, const T *__restrict__ key,
                        const T *__restrict__ value, const T *__restrict__ offset, const T *__restrict__ attn,
                        typename AccOf<T>::type *__restrict__ grad_query, typename AccOf<T>::type *__restrict__ grad_key,
                        typename AccOf<T>::type *__restrict__ grad_value, T *__restrict__ grad_offset,
                        int B, int Cq, int C, int H, int W, int P, int s, int G) {
    using A = typename AccOf<T>::type;
    __shared__ A s_h[MAXP][NTHR], s_w[MAXP][NTHR], s_d[MAXP][NTHR], s_gw[MAXP][NTHR], s_gh[MAXP][NTHR];
    const int sH = s * H, sW = s * W, AC = G * P, gq = Cq / G, gc = C / G;
    const size_t hi = (size_t)sH * sW, lo = (size_t)H * W;
    const int tx = threadIdx.x;
    const long long total = (long long)B * G * hi;
    for (long long i = blockIdx.x * (long long)NTHR + tx; i < total; i += (long long)gridDim.x * NTHR) {
        const size_t pix = (size_t)(i % hi);
        const int qw = (int)(pix % sW), qh = (int)(pix / sW);
        const int g = (int)((i / hi) % G);
        const int b = (int)(i / (hi * G));
        const size_t k0 = (size_t)b * AC + (size_t)g * P;              // first (group, point) plane of this thread
        const T *ap = attn + k0 * hi + pix;
        // ---- pass A
        A dot = 0;
        for (int p = 0; p < P; ++p) {
            const A w = A(qw / s) + to_acc(offset[(k0 + p) * 2 * hi + pix]);
            const A h = A(qh / s) + to_acc(offset[(k0 + p) * 2 * hi + hi + pix]);
            Bilinear<A> bl;
            bl.setup(h, w, H, W);
            A dA = 0, g_w = 0, g_h = 0;
            if (bl.inside) {
                const A hh = A(1) - bl.lh, hw = A(1) - bl.lw;
                const A a_p = to_acc(ap[(size_t)p * hi]);
                const size_t ch0 = (size_t)b * C + (size_t)g * gc;
                for (int c = 0; c < gc; ++c) {
                    A v00, v01, v10, v11;
                    bl.corners(value + (ch0 + c) * lo, v00, v01, v10, v11);
                    const A t = to_acc(grad_out[(ch0 + c) * hi + pix]);
                    dA += t * (bl.w00 * v00 + bl.w01 * v01 + bl.w10 * v10 + bl.w11 * v11);
                    const A tw = t * a_p;
                    A *gp = grad_value + (ch0 + c) * lo;
                    if (bl.i00 >= 0) atomic_add(gp + bl.i00, bl.w00 * tw);
                    if (bl.i01 >= 0) atomic_add(gp + bl.i01, bl.w01 * tw);
                    if (bl.i10 >= 0) atomic_add(gp + bl.i10, bl.w10 * tw);
                    if (bl.i11 >= 0) atomic_add(gp + bl.i11, bl.w11 * tw);
                    g_w += (-hh * v00 + hh * v01 - bl.lh * v10 + bl.lh * v11) * tw;
                    g_h += (-hw * v00 - bl.lw * v01 + hw * v10 + bl.lw * v11) * tw;
                }
                dot += a_p * dA;
            }
            s_h[p][tx] = h; s_w[p][tx] = w; s_d[p][tx] = dA; s_gw[p][tx] = g_w; s_gh[p][tx] = g_h;
        }
        // ---- pass B + C
        const size_t qch0 = (size_t)b * Cq + (size_t)g * gq;
        for (int p = 0; p < P; ++p) {
            const A dS = to_acc(ap[(size_t)p * hi]) * (s_d[p][tx] - dot);
            Bilinear<A> bl;
            bl.setup(s_h[p][tx], s_w[p][tx], H, W);
            A g_w = s_gw[p][tx], g_h = s_gh[p][tx];
            const bool first = p == 0;
            if (bl.inside) {
                const A hh = A(1) - bl.lh, hw = A(1) - bl.lw;
                for (int c = 0; c < gq; ++c) {
                    A v00, v01, v10, v11;
                    bl.corners(key + (qch0 + c) * lo, v00, v01, v10, v11);
                    const A val = bl.w00 * v00 + bl.w01 * v01 + bl.w10 * v10 + bl.w11 * v11;
                    A *qg = grad_query + (qch0 + c) * hi + pix;
                    *qg = first ? dS * val : *qg + dS * val;
                    const A tw = dS * to_acc(query[(qch0 + c) * hi + pix]);
                    A *gp = grad_key + (qch0 + c) * lo;
                    if (bl.i00 >= 0) atomic_add(gp + bl.i00, bl.w00 * tw);
                    if (bl.i01 >= 0) atomic_add(gp + bl.i01, bl.w01 * tw);
                    if (bl.i10 >= 0) atomic_add(gp + bl.i10, bl.w10 * tw);
                    if (bl.i11 >= 0) atomic_add(gp + bl.i11, bl.w11 * tw);
                    g_w += (-hh * v00 + hh * v01 - bl.lh * v10 + bl.lh * v11) * tw;
                    g_h += (-hw * v00 - bl.lw * v01 + hw * v10 + bl.lw * v11) * tw;
                }
            } else if (first) {
                for (int c = 0; c < gq; ++c) grad_query[(qch0 + c) * hi + pix] = A(0);
            }
            grad_offset[(k0 + p) * 2 * hi + pix] = from_acc<T>(g_w);
            grad_offset[(k0 + p) * 2 * hi + hi + pix] = from_acc<T>(g_h);
        }
    }
}

static inline int grid_1d(long long total, int threads) {
    long long blocks = (total + threads - 1) / threads;
    const long long cap = 148LL * 64;
    return (int)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

static int check_deform(const char *fn, int B, int Cq, int C, int H, int W, int P, int s, int G, int dtype) {
    SAPA_REQUIRE(B > 0 && Cq > 0 && C > 0 && H > 0 && W > 0, SAPA_ERR_ARGUMENT, "%s: sizes must be positive", fn);
    SAPA_REQUIRE(P >= 1, SAPA_ERR_ARGUMENT, "%s: num_point must be >= 1, got %d", fn, P);
    SAPA_REQUIRE(s >= 1, SAPA_ERR_ARGUMENT, "%s: scale_factor must be >= 1, got %d", fn, s);
    SAPA_REQUIRE(G >= 1 && Cq % G == 0 && C % G == 0, SAPA_ERR_ARGUMENT,
                 "%s: channels (%d, %d) must be divisible by groups (%d)", fn, Cq, C, G);
    SAPA_REQUIRE(dtype_size(dtype) != 0, SAPA_ERR_DTYPE, "%s: unknown dtype code %d", fn, dtype);
    SAPA_REQUIRE((long long)s * H * s * W < (1LL << 31), SAPA_ERR_ARGUMENT, "%s: image too large", fn);
    return SAPA_OK;
}


static int memset_async(void *p, size_t bytes, cudaStream_t st, const char *fn) {
    const cudaError_t e = cudaMemsetAsync(p, 0, bytes, st);
    SAPA_REQUIRE(e == cudaSuccess, SAPA_ERR_LAUNCH, "%s: cudaMemsetAsync failed: %s", fn, cudaGetErrorString(e));
    return SAPA_OK;
}

}  // namespace sapa

using namespace sapa;

extern "C" {

int sapa_deform_qk_forward(const void *query, const void *key, const void *offset, void *out, int B, int Cq, int H, int W,
                           int P, int s, int G, int dtype, void *stream) {
    const char *fn = "sapa_deform_qk_forward";
    trace_reset();
    if (int e = check_deform(fn, B, Cq, Cq, H, W, P, s, G, dtype)) return e;
    SAPA_CHECK_PTR(fn, query); SAPA_CHECK_PTR(fn, key); SAPA_CHECK_PTR(fn, offset); SAPA_CHECK_PTR(fn, out);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return SAPA_DISPATCH_ALL(dtype, [&] {
        const long long total = (long long)B * G * P * s * H * s * W;
        deform_qk_fwd_kernel<scalar_t><<<grid_1d(total, 256), 256, 0, st>>>(
            static_cast<const scalar_t *>(query), static_cast<const scalar_t *>(key), static_cast<const scalar_t *>(offset),
            static_cast<scalar_t *>(out), B, Cq, H, W, P, s, G);
        return check_launch("deform_qk_fwd_kernel");
    });
}

int sapa_deform_av_forward(const void *attn, const void *value, const void *offset, void *out, int B, int C, int H, int W,
                           int P, int s, int G, int dtype, void *stream) {
    const char *fn = "sapa_deform_av_forward";
    trace_reset();
    if (int e = check_deform(fn, B, C, C, H, W, P, s, G, dtype)) return e;
    SAPA_CHECK_PTR(fn, attn); SAPA_CHECK_PTR(fn, value); SAPA_CHECK_PTR(fn, offset); SAPA_CHECK_PTR(fn, out);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return SAPA_DISPATCH_ALL(dtype, [&] {
        constexpr int CPT = 8;
        const int chunks = (C / G + CPT - 1) / CPT;
        const long long total = (long long)B * G * chunks * s * H * s * W;
        deform_av_fwd_kernel<scalar_t, CPT><<<grid_1d(total, 256), 256, 0, st>>>(
            static_cast<const scalar_t *>(attn), static_cast<const scalar_t *>(value), static_cast<const scalar_t *>(offset),
            static_cast<scalar_t *>(out), B, C, H, W, P, s, G);
        return check_launch("deform_av_fwd_kernel");
    });
}

int sapa_deform_fused_forward(const void *query, const void *key, const void *value, const void *offset, void *out,
                              void *attn, int B, int Cq, int C, int H, int W, int P, int s, int G, int dtype, void *stream) {
    const char *fn = "sapa_deform_fused_forward";
    trace_reset();
    if (int e = check_deform(fn, B, Cq, C, H, W, P, s, G, dtype)) return e;
    SAPA_CHECK_PTR(fn, query); SAPA_CHECK_PTR(fn, key); SAPA_CHECK_PTR(fn, value); SAPA_CHECK_PTR(fn, offset);
    SAPA_CHECK_PTR(fn, out);
    SAPA_REQUIRE(P <= MAXP && dtype != SAPA_F64, SAPA_ERR_UNSUPPORTED,
                 "%s: no fused kernel for num_point=%d dtype=%d (use the separate ops)", fn, P, dtype);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return SAPA_DISPATCH_FAST(dtype, [&] {
        const int pix_blocks = ceil_div((long long)s * H * s * W, 32);
        const long long blocks = (long long)B * G * pix_blocks;
        if (blocks > 0x7fffffffLL) {
            set_error("too many blocks");
            return (int)SAPA_ERR_ARGUMENT;
        }
        deform_fused_fwd_kernel<scalar_t, 8><<<(unsigned)blocks, dim3(32, FY), 0, st>>>(
            static_cast<const scalar_t *>(query), static_cast<const scalar_t *>(key), static_cast<const scalar_t *>(value),
            static_cast<const scalar_t *>(offset), static_cast<scalar_t *>(out), static_cast<scalar_t *>(attn), B, Cq, C, H,
            W, P, s, G, pix_blocks);
        return check_launch("deform_fused_fwd_kernel");
    });
}

int sapa_deform_qk_backward(const void *grad_out, const void *query, const void *key, const void *offset, void *grad_query,
                            void *grad_key, void *grad_offset, int B, int Cq, int H, int W, int P, int s, int G, int dtype,
                            void *stream) {
    const char *fn = "sapa_deform_qk_backward";
    trace_reset();
    if (int e = check_deform(fn, B, Cq, Cq, H, W, P, s, G, dtype)) return e;
    SAPA_CHECK_PTR(fn, grad_out); SAPA_CHECK_PTR(fn, query); SAPA_CHECK_PTR(fn, key); SAPA_CHECK_PTR(fn, offset);
    SAPA_CHECK_PTR(fn, grad_query); SAPA_CHECK_PTR(fn, grad_key); SAPA_CHECK_PTR(fn, grad_offset);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t acc = dtype == SAPA_F64 ? 8 : 4;
    if (int e = memset_async(grad_query, (size_t)B * Cq * s * H * s * W * acc, st, fn)) return e;
    if (int e = memset_async(grad_key, (size_t)B * Cq * H * W * acc, st, fn)) return e;
    return SAPA_DISPATCH_ALL(dtype, [&] {
        using A = typename AccOf<scalar_t>::type;
        const long long total = (long long)B * G * P * s * H * s * W;
        deform_bwd_kernel<scalar_t, true><<<grid_1d(total, 256), 256, 0, st>>>(
            static_cast<const scalar_t *>(grad_out), static_cast<const scalar_t *>(query), static_cast<const scalar_t *>(key),
            static_cast<const scalar_t *>(offset), static_cast<A *>(grad_query), nullptr, static_cast<A *>(grad_key),
            static_cast<scalar_t *>(grad_offset), B, Cq, H, W, P, s, G);
        return check_launch("deform_bwd_kernel<qk>");
    });
}

int sapa_deform_av_backward(const void *grad_out, const void *attn, const void *value, const void *offset, void *grad_attn,
                            void *grad_value, void *grad_offset, int B, int C, int H, int W, int P, int s, int G, int dtype,
                            void *stream) {
    const char *fn = "sapa_deform_av_backward";
    trace_reset();
    if (int e = check_deform(fn, B, C, C, H, W, P, s, G, dtype)) return e;
    SAPA_CHECK_PTR(fn, grad_out); SAPA_CHECK_PTR(fn, attn); SAPA_CHECK_PTR(fn, value); SAPA_CHECK_PTR(fn, offset);
    SAPA_CHECK_PTR(fn, grad_attn); SAPA_CHECK_PTR(fn, grad_value); SAPA_CHECK_PTR(fn, grad_offset);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t acc = dtype == SAPA_F64 ? 8 : 4;
    if (int e = memset_async(grad_value, (size_t)B * C * H * W * acc, st, fn)) return e;
    return SAPA_DISPATCH_ALL(dtype, [&] {
        using A = typename AccOf<scalar_t>::type;
        const long long total = (long long)B * G * P * s * H * s * W;
        deform_bwd_kernel<scalar_t, false><<<grid_1d(total, 256), 256, 0, st>>>(
            static_cast<const scalar_t *>(grad_out), static_cast<const scalar_t *>(attn), static_cast<const scalar_t *>(value),
            static_cast<const scalar_t *>(offset), nullptr, static_cast<scalar_t *>(grad_attn), static_cast<A *>(grad_value),
            static_cast<scalar_t *>(grad_offset), B, C, H, W, P, s, G);
        return check_launch("deform_bwd_kernel<av>");
    });
}

int sapa_deform_fused_backward(const void *grad_out, const void *query, const void *key, const void *value,
                               const void *offset, const void *attn, void *grad_query, void *grad_key, void *grad_value,
                               void *grad_offset, int B, int Cq, int C, int H, int W, int P, int s, int G, int dtype,
                               void *stream) {
    const char *fn = "sapa_deform_fused_backward";
    trace_reset();
    if (int e = check_deform(fn, B, Cq, C, H, W, P, s, G, dtype)) return e;
    SAPA_CHECK_PTR(fn, grad_out); SAPA_CHECK_PTR(fn, query); SAPA_CHECK_PTR(fn, key); SAPA_CHECK_PTR(fn, value);
    SAPA_CHECK_PTR(fn, offset); SAPA_CHECK_PTR(fn, attn); SAPA_CHECK_PTR(fn, grad_offset);
    SAPA_REQUIRE(grad_query != nullptr && grad_key != nullptr && grad_value != nullptr, SAPA_ERR_ARGUMENT,
                 "%s: a gradient buffer is NULL", fn);
    SAPA_REQUIRE(P <= MAXP, SAPA_ERR_UNSUPPORTED, "%s: no fused kernel for num_point=%d (use the separate ops)", fn, P);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t acc = dtype == SAPA_F64 ? 8 : 4;
    if (int e = memset_async(grad_key, (size_t)B * Cq * H * W * acc, st, fn)) return e;
    if (int e = memset_async(grad_value, (size_t)B * C * H * W * acc, st, fn)) return e;
    return SAPA_DISPATCH_ALL(dtype, [&] {
        using A = typename AccOf<scalar_t>::type;
        constexpr int NTHR = sizeof(A) == 8 ? 64 : 128;      // five per-point arrays of MAXP x NTHR accumulators in shared memory
        const long long total = (long long)B * G * s * H * s * W;
        deform_fused_bwd_kernel<scalar_t, NTHR><<<grid_1d(total, NTHR), NTHR, 0, st>>>(
            static_cast<const scalar_t *>(grad_out), static_cast<const scalar_t *>(query), static_cast<const scalar_t *>(key),
            static_cast<const scalar_t *>(value), static_cast<const scalar_t *>(offset), static_cast<const scalar_t *>(attn),
            static_cast<A *>(grad_query), static_cast<A *>(grad_key), static_cast<A *>(grad_value),
            static_cast<scalar_t *>(grad_offset), B, Cq, C, H, W, P, s, G);
        return check_launch("deform_fused_bwd_kernel");
    });
}

}  // extern "C"

// dispatchers of the SAPA-B logit and aggregation kernels (sapa_b.cu)
namespace sapa {
int run_sim(const void *hi, const void *lo, void *out, int B, int Cc, int H, int W, int K, int s, int dtype, cudaStream_t st);
int run_agg(const void *wt, const void *lo, void *out, int B, int Cc, int H, int W, int K, int s, int dtype, cudaStream_t st);
int run_gath(const void *hi, const void *wt, void *out, int B, int Cc, int H, int W, int K, int s, int dtype, cudaStream_t st);
int run_sim_slab(const void *hi, const void *lo, void *out, int B, int Cc, int H, int W, int rows, int top, int K, int s, int dtype,
                 cudaStream_t st);
int run_agg_slab(const void *wt, const void *lo, void *out, int B, int Cc, int H, int W, int rows, int top, int K, int s, int dtype,
                 cudaStream_t st);
int run_sim_mixed(const void *hi, const void *lo, float *out, int B, int Cc, int H, int W, int rows, int top, int dtype, cudaStream_t st);
bool fused_tma_supported(int W, int dtype);
}

extern "C" {

size_t sapa_deform_fused_forward_workspace(int B, int H, int W, int P, int s, int G, int dtype) {
    if (B <= 0 || H <= 0 || W <= 0 || P <= 0 || G <= 0 || s != 2) return 0;
    // 16-bit tensors: the mixed modes of the TMA kernels (16-bit operands, float32 windows) need rows of 16 bytes
    if (dtype != SAPA_F32 && !((dtype == SAPA_F16 || dtype == SAPA_BF16) && W % 8 == 0 && fused_tma_supported(W, dtype))) return 0;
    const size_t hi = (size_t)s * H * s * W;
    if ((size_t)B * G * hi >= 0xffffffffull) return 0;       // the outlier list indexes (image, group, pixel) with 32 bits
    // dense similarity + window weights (float32 whatever the tensors' type), the outlier list (worst case: every
    // point) and its counter
    return (size_t)B * G * 50 * hi * sizeof(float) + (size_t)B * G * hi * sizeof(OutlierTap) + 16;
}

int sapa_deform_fused_forward_slab(const void *query, const void *key, const void *value, const void *offset, void *out,
                                   void *attn, void *workspace, size_t workspace_bytes, int B, int Cq, int C, int H, int W,
                                   int halo_top, int halo_bottom, int P, int s, int G, int dtype, void *stream) {
    const char *fn = "sapa_deform_fused_forward_slab";
    trace_reset();
    if (int e = check_deform(fn, B, Cq, C, H, W, P, s, G, dtype)) return e;
    SAPA_REQUIRE(halo_top >= 0 && halo_bottom >= 0 && ((long long)halo_top + H + halo_bottom) * W < (1LL << 31), SAPA_ERR_ARGUMENT,
                 "%s: bad halo (%d, %d)", fn, halo_top, halo_bottom);
    const int rows = halo_top + H + halo_bottom;
    SAPA_CHECK_PTR(fn, query); SAPA_CHECK_PTR(fn, key); SAPA_CHECK_PTR(fn, value); SAPA_CHECK_PTR(fn, offset);
    SAPA_CHECK_PTR(fn, out);
    const size_t need = sapa_deform_fused_forward_workspace(B, H, W, P, s, G, dtype);
    SAPA_REQUIRE(s == 2 && P <= MAXP && need != 0, SAPA_ERR_UNSUPPORTED,
                 "%s: the dense-window path needs s = 2, num_point <= %d and float32, or float16 / bfloat16 with rows of 16 bytes "
                 "(use sapa_deform_fused_forward)", fn, MAXP);
    SAPA_REQUIRE(workspace != nullptr && workspace_bytes >= need && aligned16(workspace), SAPA_ERR_WORKSPACE,
                 "%s: a 16-byte aligned workspace of %zu bytes is required, got %zu", fn, need, workspace_bytes);
    const size_t hi = (size_t)s * H * s * W;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // the window weights have the tensors' type (the aggregation kernel rounds them to it anyway), the similarity is
    // always float32; both regions are sized for float32
    float *dense = static_cast<float *>(workspace);
    void *window = dense + (size_t)B * G * 25 * hi;
    OutlierTap *taps = reinterpret_cast<OutlierTap *>(dense + (size_t)B * G * 50 * hi);
    unsigned int *tap_count = reinterpret_cast<unsigned int *>(taps + (size_t)B * G * hi);
    if (cudaMemsetAsync(tap_count, 0, sizeof(unsigned int), st) != cudaSuccess) {
        set_error("%s: clearing the outlier counter failed: %s", fn, cudaGetErrorString(cudaGetLastError()));
        return SAPA_ERR_LAUNCH;
    }
    // 1. dense 25-slot similarity of every group: the B x G groups are images of Cq / G channels.  16-bit tensors: the
    //    logits leave the tensor-core kernel as float32 (a 16-bit logit would cost the softmax two digits)
    if (dtype == SAPA_F32) {
        if (int e = run_sim_slab(query, key, dense, B * G, Cq / G, H, W, rows, halo_top, 5, 2, dtype, st)) return e;
    } else {
        if (int e = run_sim_mixed(query, key, dense, B * G, Cq / G, H, W, rows, halo_top, dtype, st)) return e;
    }
    // 2. attention over the points, dense window weights, list of the points that leave the window
    {
        const long long total = (long long)B * G * hi;
        const int grid = grid_1d(total, WIN_THREADS);
        const int e = SAPA_DISPATCH_FAST(dtype, [&] {
            const scalar_t *q = static_cast<const scalar_t *>(query), *k = static_cast<const scalar_t *>(key);
            const scalar_t *o = static_cast<const scalar_t *>(offset);
            scalar_t *at = static_cast<scalar_t *>(attn), *wn = static_cast<scalar_t *>(window);
            if (P == 9)          // the 3 x 3 points of the reference modules' default
                deform_window_kernel<scalar_t, 9, WIN_FUSED><<<grid, WIN_THREADS, 0, st>>>(q, k, o, dense, at, wn, taps, tap_count, B, Cq,
                                                                                  H, W, P, G, rows, halo_top);
            else
                deform_window_kernel<scalar_t, 0, WIN_FUSED><<<grid, WIN_THREADS, 0, st>>>(q, k, o, dense, at, wn, taps, tap_count, B, Cq,
                                                                                  H, W, P, G, rows, halo_top);
            return check_launch("deform_window_kernel");
        });
        if (e) return e;
    }
    // 3. aggregation of every group's channels over the window
    if (int e = run_agg_slab(window, value, out, B * G, C / G, H, W, rows, halo_top, 5, 2, dtype, st)) return e;
    // 4. the listed points (the count is only known on the device: a fixed grid strides over the list)
    return SAPA_DISPATCH_FAST(dtype, [&] {
        deform_outlier_kernel<scalar_t><<<148 * 8, 256, 0, st>>>(taps, tap_count, static_cast<const scalar_t *>(value),
                                                                 static_cast<const scalar_t *>(offset), static_cast<scalar_t *>(out),
                                                                 C, H, W, P, G, rows, halo_top);
        return check_launch("deform_outlier_kernel");
    });
}

int sapa_deform_fused_forward_dense(const void *query, const void *key, const void *value, const void *offset, void *out,
                                    void *attn, void *workspace, size_t workspace_bytes, int B, int Cq, int C, int H, int W,
                                    int P, int s, int G, int dtype, void *stream) {
    return sapa_deform_fused_forward_slab(query, key, value, offset, out, attn, workspace, workspace_bytes, B, Cq, C, H, W, 0, 0,
                                          P, s, G, dtype, stream);
}

// deform_qk and deform_av through the dense window (s = 2, float32): the halves of the fused forward, with the reference's
// op boundaries (raw logits out / attention in).  Workspace as for sapa_deform_fused_forward_dense.
int sapa_deform_qk_forward_dense(const void *query, const void *key, const void *offset, void *out, void *workspace,
                                 size_t workspace_bytes, int B, int Cq, int H, int W, int P, int s, int G, int dtype, void *stream) {
    const char *fn = "sapa_deform_qk_forward_dense";
    trace_reset();
    if (int e = check_deform(fn, B, Cq, Cq, H, W, P, s, G, dtype)) return e;
    SAPA_CHECK_PTR(fn, query); SAPA_CHECK_PTR(fn, key); SAPA_CHECK_PTR(fn, offset); SAPA_CHECK_PTR(fn, out);
    const size_t need = sapa_deform_fused_forward_workspace(B, H, W, P, s, G, dtype);
    SAPA_REQUIRE(s == 2 && P <= MAXP && need != 0, SAPA_ERR_UNSUPPORTED,
                 "%s: the dense-window path needs s = 2, num_point <= %d and float32, or float16 / bfloat16 with rows of 16 bytes "
                 "(use sapa_deform_qk_forward)", fn, MAXP);
    SAPA_REQUIRE(workspace != nullptr && workspace_bytes >= need && aligned16(workspace), SAPA_ERR_WORKSPACE,
                 "%s: a 16-byte aligned workspace of %zu bytes is required, got %zu", fn, need, workspace_bytes);
    const size_t hi = (size_t)s * H * s * W;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float *dense = static_cast<float *>(workspace);
    if (dtype == SAPA_F32) {
        if (int e = run_sim(query, key, dense, B * G, Cq / G, H, W, 5, 2, dtype, st)) return e;
    } else {
        if (int e = run_sim_mixed(query, key, dense, B * G, Cq / G, H, W, H, 0, dtype, st)) return e;
    }
    const long long total = (long long)B * G * hi;
    return SAPA_DISPATCH_FAST(dtype, [&] {
        if (P == 9)      // the 3 x 3 points of the reference modules' default: loops unrolled for nine points
            deform_window_kernel<scalar_t, 9, WIN_LOGITS><<<grid_1d(total, WIN_THREADS), WIN_THREADS, 0, st>>>(
                static_cast<const scalar_t *>(query), static_cast<const scalar_t *>(key), static_cast<const scalar_t *>(offset), dense,
                static_cast<scalar_t *>(out), nullptr, nullptr, nullptr, B, Cq, H, W, P, G, H, 0);
        else
            deform_window_kernel<scalar_t, 0, WIN_LOGITS><<<grid_1d(total, WIN_THREADS), WIN_THREADS, 0, st>>>(
                static_cast<const scalar_t *>(query), static_cast<const scalar_t *>(key), static_cast<const scalar_t *>(offset), dense,
                static_cast<scalar_t *>(out), nullptr, nullptr, nullptr, B, Cq, H, W, P, G, H, 0);
        return check_launch("deform_window_kernel<logits>");
    });
}

int sapa_deform_av_forward_dense(const void *attn, const void *value, const void *offset, void *out, void *workspace,
                                 size_t workspace_bytes, int B, int C, int H, int W, int P, int s, int G, int dtype, void *stream) {
    const char *fn = "sapa_deform_av_forward_dense";
    trace_reset();
    if (int e = check_deform(fn, B, C, C, H, W, P, s, G, dtype)) return e;
    SAPA_CHECK_PTR(fn, attn); SAPA_CHECK_PTR(fn, value); SAPA_CHECK_PTR(fn, offset); SAPA_CHECK_PTR(fn, out);
    const size_t need = sapa_deform_fused_forward_workspace(B, H, W, P, s, G, dtype);
    SAPA_REQUIRE(s == 2 && P <= MAXP && need != 0, SAPA_ERR_UNSUPPORTED,
                 "%s: the dense-window path needs s = 2, num_point <= %d and float32, or float16 / bfloat16 with rows of 16 bytes "
                 "(use sapa_deform_av_forward)", fn, MAXP);
    SAPA_REQUIRE(workspace != nullptr && workspace_bytes >= need && aligned16(workspace), SAPA_ERR_WORKSPACE,
                 "%s: a 16-byte aligned workspace of %zu bytes is required, got %zu", fn, need, workspace_bytes);
    const size_t hi = (size_t)s * H * s * W;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float *region = static_cast<float *>(workspace) + (size_t)B * G * 25 * hi;      // the window weights (tensor type) live here
    OutlierTap *taps = reinterpret_cast<OutlierTap *>(region + (size_t)B * G * 25 * hi);
    unsigned int *tap_count = reinterpret_cast<unsigned int *>(taps + (size_t)B * G * hi);
    if (cudaMemsetAsync(tap_count, 0, sizeof(unsigned int), st) != cudaSuccess) {
        set_error("%s: clearing the outlier counter failed: %s", fn, cudaGetErrorString(cudaGetLastError()));
        return SAPA_ERR_LAUNCH;
    }
    const long long total = (long long)B * G * hi;
    // the attention is only read in this mode
    if (int e = SAPA_DISPATCH_FAST(dtype, [&] {
            if (P == 9)      // the 3 x 3 points of the reference modules' default: loops unrolled for nine points
                deform_window_kernel<scalar_t, 9, WIN_WEIGHTS><<<grid_1d(total, WIN_THREADS), WIN_THREADS, 0, st>>>(
                    nullptr, nullptr, static_cast<const scalar_t *>(offset), nullptr, const_cast<scalar_t *>(static_cast<const scalar_t *>(attn)),
                    reinterpret_cast<scalar_t *>(region), taps, tap_count, B, C, H, W, P, G, H, 0);
            else
                deform_window_kernel<scalar_t, 0, WIN_WEIGHTS><<<grid_1d(total, WIN_THREADS), WIN_THREADS, 0, st>>>(
                    nullptr, nullptr, static_cast<const scalar_t *>(offset), nullptr, const_cast<scalar_t *>(static_cast<const scalar_t *>(attn)),
                    reinterpret_cast<scalar_t *>(region), taps, tap_count, B, C, H, W, P, G, H, 0);
            return check_launch("deform_window_kernel<weights>");
        }))
        return e;
    if (int e = run_agg(region, value, out, B * G, C / G, H, W, 5, 2, dtype, st)) return e;
    return SAPA_DISPATCH_FAST(dtype, [&] {
        deform_outlier_kernel<scalar_t><<<148 * 8, 256, 0, st>>>(taps, tap_count, static_cast<const scalar_t *>(value),
                                                                 static_cast<const scalar_t *>(offset), static_cast<scalar_t *>(out), C, H,
                                                                 W, P, G, H, 0);
        return check_launch("deform_outlier_kernel");
    });
}

size_t sapa_deform_fused_backward_workspace(int B, int H, int W, int P, int s, int G, int dtype) {
    if (B <= 0 || H <= 0 || W <= 0 || P <= 0 || G <= 0 || s != 2) return 0;
    // 16-bit tensors: 16-bit operands in the tensor-core kernels, float32 similarities between them (rows of 16 bytes)
    if (dtype != SAPA_F32 && !((dtype == SAPA_F16 || dtype == SAPA_BF16) && W % 8 == 0 && fused_tma_supported(W, dtype))) return 0;
    const size_t hi = (size_t)s * H * s * W;
    if ((size_t)B * G * P >= 0xffffffffull || hi >= 0xffffffffull) return 0;
    // D, dWd (float32), dD, Wd (the tensors' type; sized for float32), the outlier list (worst case: every point) and
    // its counter
    return (size_t)B * G * 100 * hi * sizeof(float) + (size_t)B * G * P * hi * sizeof(OutlierGrad) + 16;
}

// 16-bit tensors only: float32 side buffers for the scattered key / value gradients of the listed points
size_t sapa_deform_fused_backward_scatter_bytes(int B, int Cq, int C, int H, int W, int dtype) {
    if (dtype != SAPA_F16 && dtype != SAPA_BF16) return 0;
    return ((size_t)B * Cq * H * W + (size_t)B * C * H * W) * sizeof(float);
}

int sapa_deform_fused_backward_dense(const void *grad_out, const void *query, const void *key, const void *value,
                                     const void *offset, const void *attn, void *grad_query, void *grad_key, void *grad_value,
                                     void *grad_offset, void *workspace, size_t workspace_bytes, int B, int Cq, int C, int H,
                                     int W, int P, int s, int G, int dtype, void *stream) {
    const char *fn = "sapa_deform_fused_backward_dense";
    trace_reset();
    if (int e = check_deform(fn, B, Cq, C, H, W, P, s, G, dtype)) return e;
    SAPA_CHECK_PTR(fn, grad_out); SAPA_CHECK_PTR(fn, query); SAPA_CHECK_PTR(fn, key); SAPA_CHECK_PTR(fn, value);
    SAPA_CHECK_PTR(fn, offset); SAPA_CHECK_PTR(fn, attn); SAPA_CHECK_PTR(fn, grad_query); SAPA_CHECK_PTR(fn, grad_key);
    SAPA_CHECK_PTR(fn, grad_value); SAPA_CHECK_PTR(fn, grad_offset);
    const size_t base = sapa_deform_fused_backward_workspace(B, H, W, P, s, G, dtype);
    const size_t side_off = (base + 15) & ~(size_t)15;          // the side buffers of the 16-bit path start here
    const size_t need = side_off + sapa_deform_fused_backward_scatter_bytes(B, Cq, C, H, W, dtype);
    SAPA_REQUIRE(s == 2 && P <= MAXP && base != 0, SAPA_ERR_UNSUPPORTED,
                 "%s: the dense-window path needs s = 2, num_point <= %d and float32, or float16 / bfloat16 with rows of 16 bytes "
                 "(use sapa_deform_fused_backward)", fn, MAXP);
    SAPA_REQUIRE(workspace != nullptr && workspace_bytes >= need && aligned16(workspace), SAPA_ERR_WORKSPACE,
                 "%s: a 16-byte aligned workspace of %zu bytes is required, got %zu", fn, need, workspace_bytes);
    const size_t hi = (size_t)s * H * s * W, plane = (size_t)B * G * 25 * hi;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // D and dWd are float32 whatever the tensors' type; dD and Wd are weights of the SAPA-B kernels and have the tensors'
    // type (those kernels round their weights to it anyway); every region is sized for float32
    float *dense = static_cast<float *>(workspace), *dwin = dense + plane;
    void *ddense = dwin + plane, *window = dwin + 2 * plane;
    OutlierGrad *taps = reinterpret_cast<OutlierGrad *>(dense + 4 * plane);
    unsigned int *tap_count = reinterpret_cast<unsigned int *>(taps + (size_t)B * G * P * hi);
    if (cudaMemsetAsync(tap_count, 0, sizeof(unsigned int), st) != cudaSuccess) {
        set_error("%s: clearing the outlier counter failed: %s", fn, cudaGetErrorString(cudaGetLastError()));
        return SAPA_ERR_LAUNCH;
    }
    // 1. D = sim(Q, Key) and dWd = sim(dOut, Value), the B x G groups as images
    if (dtype == SAPA_F32) {
        if (int e = run_sim(query, key, dense, B * G, Cq / G, H, W, 5, 2, dtype, st)) return e;
        if (int e = run_sim(grad_out, value, dwin, B * G, C / G, H, W, 5, 2, dtype, st)) return e;
    } else {
        if (int e = run_sim_mixed(query, key, dense, B * G, Cq / G, H, W, H, 0, dtype, st)) return e;
        if (int e = run_sim_mixed(grad_out, value, dwin, B * G, C / G, H, W, H, 0, dtype, st)) return e;
    }
    // 2. per pixel: softmax backward over the points, dD, Wd, offset gradients, list of the points outside the window
    {
        const long long total = (long long)B * G * hi;
        const int grid = grid_1d(total, WIN_THREADS);
        const int e = SAPA_DISPATCH_FAST(dtype, [&] {
            const scalar_t *go = static_cast<const scalar_t *>(grad_out), *v = static_cast<const scalar_t *>(value);
            const scalar_t *o = static_cast<const scalar_t *>(offset), *a = static_cast<const scalar_t *>(attn);
            scalar_t *dd = static_cast<scalar_t *>(ddense), *wn = static_cast<scalar_t *>(window), *goff = static_cast<scalar_t *>(grad_offset);
            if (P == 9)
                deform_window_bwd_kernel<scalar_t, 9, BWD_FUSED><<<grid, WIN_THREADS, 0, st>>>(go, v, o, a, dense, dwin, dd, wn, goff, nullptr, taps,
                                                                                      tap_count, B, C, H, W, P, G);
            else
                deform_window_bwd_kernel<scalar_t, 0, BWD_FUSED><<<grid, WIN_THREADS, 0, st>>>(go, v, o, a, dense, dwin, dd, wn, goff, nullptr, taps,
                                                                                      tap_count, B, C, H, W, P, G);
            return check_launch("deform_window_bwd_kernel");
        });
        if (e) return e;
    }
    // 3. dQ = agg(dD, Key), dKey = gath(Q, dD), dV = gath(dOut, Wd): SAPA-B kernels per group, all outputs overwritten
    if (int e = run_agg(ddense, key, grad_query, B * G, Cq / G, H, W, 5, 2, dtype, st)) return e;
    if (int e = run_gath(query, ddense, grad_key, B * G, Cq / G, H, W, 5, 2, dtype, st)) return e;
    if (int e = run_gath(grad_out, window, grad_value, B * G, C / G, H, W, 5, 2, dtype, st)) return e;
    // 4. the listed points.  float32: atomics straight into the gradients.  16-bit: key / value contributions go to zeroed
    //    float32 side buffers behind the list and are folded into the 16-bit gradients by one more kernel.
    if (dtype == SAPA_F32) {
        deform_outlier_bwd_kernel<float, float><<<148 * 8, 256, 0, st>>>(
            taps, tap_count, static_cast<const float *>(grad_out), static_cast<const float *>(query), static_cast<const float *>(key),
            static_cast<const float *>(value), static_cast<const float *>(offset), static_cast<float *>(grad_query),
            static_cast<float *>(grad_key), static_cast<float *>(grad_value), static_cast<float *>(grad_offset), Cq, C, H, W, P, G);
        return check_launch("deform_outlier_bwd_kernel");
    }
    const size_t n_k = (size_t)B * Cq * H * W, n_v = (size_t)B * C * H * W;
    float *side_k = reinterpret_cast<float *>(static_cast<char *>(workspace) + side_off), *side_v = side_k + n_k;
    if (int e = memset_async(side_k, (n_k + n_v) * sizeof(float), st, fn)) return e;
    return SAPA_DISPATCH_FAST(dtype, [&] {
        deform_outlier_bwd_kernel<scalar_t, float><<<148 * 8, 256, 0, st>>>(
            taps, tap_count, static_cast<const scalar_t *>(grad_out), static_cast<const scalar_t *>(query),
            static_cast<const scalar_t *>(key), static_cast<const scalar_t *>(value), static_cast<const scalar_t *>(offset),
            static_cast<scalar_t *>(grad_query), side_k, side_v, static_cast<scalar_t *>(grad_offset), Cq, C, H, W, P, G);
        if (int e = check_launch("deform_outlier_bwd_kernel")) return e;
        deform_add_scatter_kernel<scalar_t><<<148 * 8, 256, 0, st>>>(tap_count, static_cast<scalar_t *>(grad_key), side_k, n_k,
                                                                    static_cast<scalar_t *>(grad_value), side_v, n_v);
        return check_launch("deform_add_scatter_kernel");
    });
}

// Backward of deform_av and of deform_qk alone through the dense window (s = 2, float32): the two halves of
// sapa_deform_fused_backward_dense without the softmax between them.  Workspace as for that entry point.
int sapa_deform_av_backward_dense(const void *grad_out, const void *attn, const void *value, const void *offset, void *grad_attn,
                                  void *grad_value, void *grad_offset, void *workspace, size_t workspace_bytes, int B, int C,
                                  int H, int W, int P, int s, int G, int dtype, void *stream) {
    const char *fn = "sapa_deform_av_backward_dense";
    trace_reset();
    if (int e = check_deform(fn, B, C, C, H, W, P, s, G, dtype)) return e;
    SAPA_CHECK_PTR(fn, grad_out); SAPA_CHECK_PTR(fn, attn); SAPA_CHECK_PTR(fn, value); SAPA_CHECK_PTR(fn, offset);
    SAPA_CHECK_PTR(fn, grad_attn); SAPA_CHECK_PTR(fn, grad_value); SAPA_CHECK_PTR(fn, grad_offset);
    const size_t base = sapa_deform_fused_backward_workspace(B, H, W, P, s, G, dtype);
    const size_t side_off = (base + 15) & ~(size_t)15;
    const size_t need = side_off + sapa_deform_fused_backward_scatter_bytes(B, 0, C, H, W, dtype);
    SAPA_REQUIRE(s == 2 && P <= MAXP && base != 0, SAPA_ERR_UNSUPPORTED,
                 "%s: the dense-window path needs s = 2, num_point <= %d and float32, or float16 / bfloat16 with rows of 16 bytes "
                 "(use sapa_deform_av_backward)", fn, MAXP);
    SAPA_REQUIRE(workspace != nullptr && workspace_bytes >= need && aligned16(workspace), SAPA_ERR_WORKSPACE,
                 "%s: a 16-byte aligned workspace of %zu bytes is required, got %zu", fn, need, workspace_bytes);
    const size_t hi = (size_t)s * H * s * W, plane = (size_t)B * G * 25 * hi;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float *dwin = static_cast<float *>(workspace) + plane;
    void *window = dwin + 2 * plane;                                   // Wd, in the tensors' type
    OutlierGrad *taps = reinterpret_cast<OutlierGrad *>(static_cast<float *>(workspace) + 4 * plane);
    unsigned int *tap_count = reinterpret_cast<unsigned int *>(taps + (size_t)B * G * P * hi);
    if (cudaMemsetAsync(tap_count, 0, sizeof(unsigned int), st) != cudaSuccess) {
        set_error("%s: clearing the outlier counter failed: %s", fn, cudaGetErrorString(cudaGetLastError()));
        return SAPA_ERR_LAUNCH;
    }
    if (dtype == SAPA_F32) {
        if (int e = run_sim(grad_out, value, dwin, B * G, C / G, H, W, 5, 2, dtype, st)) return e;        // dWd
    } else {
        if (int e = run_sim_mixed(grad_out, value, dwin, B * G, C / G, H, W, H, 0, dtype, st)) return e;
    }
    const long long total = (long long)B * G * hi;
    if (int e = SAPA_DISPATCH_FAST(dtype, [&] {
            if (P == 9)      // the 3 x 3 points of the reference modules' default: loops unrolled for nine points
                deform_window_bwd_kernel<scalar_t, 9, BWD_AV><<<grid_1d(total, WIN_THREADS), WIN_THREADS, 0, st>>>(
                    static_cast<const scalar_t *>(grad_out), static_cast<const scalar_t *>(value), static_cast<const scalar_t *>(offset),
                    static_cast<const scalar_t *>(attn), nullptr, dwin, nullptr, static_cast<scalar_t *>(window),
                    static_cast<scalar_t *>(grad_offset), static_cast<scalar_t *>(grad_attn), taps, tap_count, B, C, H, W, P, G);
            else
                deform_window_bwd_kernel<scalar_t, 0, BWD_AV><<<grid_1d(total, WIN_THREADS), WIN_THREADS, 0, st>>>(
                    static_cast<const scalar_t *>(grad_out), static_cast<const scalar_t *>(value), static_cast<const scalar_t *>(offset),
                    static_cast<const scalar_t *>(attn), nullptr, dwin, nullptr, static_cast<scalar_t *>(window),
                    static_cast<scalar_t *>(grad_offset), static_cast<scalar_t *>(grad_attn), taps, tap_count, B, C, H, W, P, G);
            return check_launch("deform_window_bwd_kernel<av>");
        }))
        return e;
    if (int e = run_gath(grad_out, window, grad_value, B * G, C / G, H, W, 5, 2, dtype, st)) return e;  // dV
    if (dtype == SAPA_F32) {
        deform_outlier_bwd_kernel<float, float><<<148 * 8, 256, 0, st>>>(
            taps, tap_count, static_cast<const float *>(grad_out), nullptr, nullptr, static_cast<const float *>(value),
            static_cast<const float *>(offset), nullptr, nullptr, static_cast<float *>(grad_value), static_cast<float *>(grad_offset),
            C, C, H, W, P, G);
        return check_launch("deform_outlier_bwd_kernel");
    }
    const size_t n_v = (size_t)B * C * H * W;
    float *side_v = reinterpret_cast<float *>(static_cast<char *>(workspace) + side_off);
    if (int e = memset_async(side_v, n_v * sizeof(float), st, fn)) return e;
    return SAPA_DISPATCH_FAST(dtype, [&] {
        deform_outlier_bwd_kernel<scalar_t, float><<<148 * 8, 256, 0, st>>>(
            taps, tap_count, static_cast<const scalar_t *>(grad_out), nullptr, nullptr, static_cast<const scalar_t *>(value),
            static_cast<const scalar_t *>(offset), nullptr, nullptr, side_v, static_cast<scalar_t *>(grad_offset), C, C, H, W, P, G);
        if (int e = check_launch("deform_outlier_bwd_kernel")) return e;
        deform_add_scatter_kernel<scalar_t><<<148 * 8, 256, 0, st>>>(tap_count, static_cast<scalar_t *>(grad_value), side_v, n_v,
                                                                    static_cast<scalar_t *>(nullptr), nullptr, 0);
        return check_launch("deform_add_scatter_kernel");
    });
}

int sapa_deform_qk_backward_dense(const void *grad_out, const void *query, const void *key, const void *offset, void *grad_query,
                                  void *grad_key, void *grad_offset, void *workspace, size_t workspace_bytes, int B, int Cq,
                                  int H, int W, int P, int s, int G, int dtype, void *stream) {
    const char *fn = "sapa_deform_qk_backward_dense";
    trace_reset();
    if (int e = check_deform(fn, B, Cq, Cq, H, W, P, s, G, dtype)) return e;
    SAPA_CHECK_PTR(fn, grad_out); SAPA_CHECK_PTR(fn, query); SAPA_CHECK_PTR(fn, key); SAPA_CHECK_PTR(fn, offset);
    SAPA_CHECK_PTR(fn, grad_query); SAPA_CHECK_PTR(fn, grad_key); SAPA_CHECK_PTR(fn, grad_offset);
    const size_t base = sapa_deform_fused_backward_workspace(B, H, W, P, s, G, dtype);
    const size_t side_off = (base + 15) & ~(size_t)15;
    const size_t need = side_off + sapa_deform_fused_backward_scatter_bytes(B, Cq, 0, H, W, dtype);
    SAPA_REQUIRE(s == 2 && P <= MAXP && base != 0, SAPA_ERR_UNSUPPORTED,
                 "%s: the dense-window path needs s = 2, num_point <= %d and float32, or float16 / bfloat16 with rows of 16 bytes "
                 "(use sapa_deform_qk_backward)", fn, MAXP);
    SAPA_REQUIRE(workspace != nullptr && workspace_bytes >= need && aligned16(workspace), SAPA_ERR_WORKSPACE,
                 "%s: a 16-byte aligned workspace of %zu bytes is required, got %zu", fn, need, workspace_bytes);
    const size_t hi = (size_t)s * H * s * W, plane = (size_t)B * G * 25 * hi;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float *dense = static_cast<float *>(workspace);
    void *ddense = dense + 2 * plane;                                  // dD, in the tensors' type
    OutlierGrad *taps = reinterpret_cast<OutlierGrad *>(dense + 4 * plane);
    unsigned int *tap_count = reinterpret_cast<unsigned int *>(taps + (size_t)B * G * P * hi);
    if (cudaMemsetAsync(tap_count, 0, sizeof(unsigned int), st) != cudaSuccess) {
        set_error("%s: clearing the outlier counter failed: %s", fn, cudaGetErrorString(cudaGetLastError()));
        return SAPA_ERR_LAUNCH;
    }
    if (dtype == SAPA_F32) {
        if (int e = run_sim(query, key, dense, B * G, Cq / G, H, W, 5, 2, dtype, st)) return e;         // D, for the offset gradients
    } else {
        if (int e = run_sim_mixed(query, key, dense, B * G, Cq / G, H, W, H, 0, dtype, st)) return e;
    }
    const long long total = (long long)B * G * hi;
    // the logit gradients enter where the fused chain reads the attention
    if (int e = SAPA_DISPATCH_FAST(dtype, [&] {
            if (P == 9)      // the 3 x 3 points of the reference modules' default: loops unrolled for nine points
                deform_window_bwd_kernel<scalar_t, 9, BWD_QK><<<grid_1d(total, WIN_THREADS), WIN_THREADS, 0, st>>>(
                    nullptr, nullptr, static_cast<const scalar_t *>(offset), static_cast<const scalar_t *>(grad_out), dense, nullptr,
                    static_cast<scalar_t *>(ddense), nullptr, static_cast<scalar_t *>(grad_offset), nullptr, taps, tap_count, B, Cq, H, W, P, G);
            else
                deform_window_bwd_kernel<scalar_t, 0, BWD_QK><<<grid_1d(total, WIN_THREADS), WIN_THREADS, 0, st>>>(
                    nullptr, nullptr, static_cast<const scalar_t *>(offset), static_cast<const scalar_t *>(grad_out), dense, nullptr,
                    static_cast<scalar_t *>(ddense), nullptr, static_cast<scalar_t *>(grad_offset), nullptr, taps, tap_count, B, Cq, H, W, P, G);
            return check_launch("deform_window_bwd_kernel<qk>");
        }))
        return e;
    if (int e = run_agg(ddense, key, grad_query, B * G, Cq / G, H, W, 5, 2, dtype, st)) return e;       // dQ
    if (int e = run_gath(query, ddense, grad_key, B * G, Cq / G, H, W, 5, 2, dtype, st)) return e;      // dKey
    if (dtype == SAPA_F32) {
        deform_outlier_bwd_kernel<float, float><<<148 * 8, 256, 0, st>>>(
            taps, tap_count, nullptr, static_cast<const float *>(query), static_cast<const float *>(key), nullptr,
            static_cast<const float *>(offset), static_cast<float *>(grad_query), static_cast<float *>(grad_key), nullptr,
            static_cast<float *>(grad_offset), Cq, Cq, H, W, P, G);
        return check_launch("deform_outlier_bwd_kernel");
    }
    const size_t n_k = (size_t)B * Cq * H * W;
    float *side_k = reinterpret_cast<float *>(static_cast<char *>(workspace) + side_off);
    if (int e = memset_async(side_k, n_k * sizeof(float), st, fn)) return e;
    return SAPA_DISPATCH_FAST(dtype, [&] {
        deform_outlier_bwd_kernel<scalar_t, float><<<148 * 8, 256, 0, st>>>(
            taps, tap_count, nullptr, static_cast<const scalar_t *>(query), static_cast<const scalar_t *>(key), nullptr,
            static_cast<const scalar_t *>(offset), static_cast<scalar_t *>(grad_query), side_k, nullptr,
            static_cast<scalar_t *>(grad_offset), Cq, Cq, H, W, P, G);
        if (int e = check_launch("deform_outlier_bwd_kernel")) return e;
        deform_add_scatter_kernel<scalar_t><<<148 * 8, 256, 0, st>>>(tap_count, static_cast<scalar_t *>(grad_key), side_k, n_k,
                                                                    static_cast<scalar_t *>(nullptr), nullptr, 0);
        return check_launch("deform_add_scatter_kernel");
    });
}

}  // extern "C"
