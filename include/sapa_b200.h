/* sapa_b200.h — C ABI of libsapa_b200.so: SAPA upsampling kernels for NVIDIA B200 (sm_100a).
 *
 * Every entry point replaces one function of the reference's pybind11 extension modules and follows
 * their ownership rule: the CALLER allocates every tensor, the library allocates nothing, keeps no
 * reference and writes results in place.  What differs from the reference:
 *   - plain device pointers + sizes + a dtype code + a CUDA stream instead of at::Tensor;
 *   - launches go to the stream passed in (the reference uses the legacy default stream);
 *   - an int status is returned and the text is available from sapa_last_error(); the process is
 *     never terminated (the reference calls exit(-1) on a launch error, qk_cuda_kernel.cu:92-96);
 *   - gradient outputs are OVERWRITTEN (the reference accumulates with atomics into buffers the caller
 *     must have zeroed); zeroing them first is unnecessary but harmless.
 *
 * Layout: all tensors are dense NCHW, as the reference requires (CHECK_CONTIGUOUS, qk_cuda.cpp:34-39).
 * H and W are always the LOW-resolution (key / value) height and width; query, attention, offset and
 * output tensors are s*H x s*W.  Window slot k = dy*K+dx addresses the low-res neighbour
 * (ph/s - (K-1)/2 + dy, pw/s - (K-1)/2 + dx); neighbours outside the image contribute zero
 * (qk_cuda_kernel.cu:50-66, av_cuda_kernel.cu:57-61).
 *
 * Pointers must be aligned to the element size; the fast kernels additionally need 16-byte alignment (what any
 * allocator returns).  The separate ops and sapa_fused_backward send a tensor view whose storage offset breaks that
 * alignment to the scalar generic kernels (the reference accepts such views too); the fused forward entry points
 * return SAPA_ERR_ALIGNMENT for it.  `stream` is a cudaStream_t passed as void* (NULL = default
 * stream).  The current CUDA device must be the one that owns the pointers.  Functions are re-entrant
 * and do not synchronise.
 */
#ifndef SAPA_B200_H_
#define SAPA_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* dtype codes (element type of every tensor of a call) */
#define SAPA_F32  0
#define SAPA_F16  1
#define SAPA_BF16 2
#define SAPA_F64  3   /* generic kernels only; kept so that float64 gradcheck scripts run (grad_check.py:17-22) */

/* status codes */
#define SAPA_OK               0
#define SAPA_ERR_ARGUMENT    -1   /* null pointer, non-positive size, even K, d % G != 0 ... */
#define SAPA_ERR_DTYPE       -2
#define SAPA_ERR_ALIGNMENT   -3
#define SAPA_ERR_LAUNCH      -4   /* cudaGetLastError() after the launch; text in sapa_last_error() */
#define SAPA_ERR_UNSUPPORTED -5   /* no kernel for this (K, s, P) in the fused path: use the separate ops */
#define SAPA_ERR_WORKSPACE   -6   /* workspace missing or too small */

/* Text of the last error raised on the calling thread ("" if none). */
const char *sapa_last_error(void);
/* Names of the kernels the most recent entry-point call of the process launched (on whichever thread: PyTorch runs
 * the backward of an autograd Function on a worker thread), comma separated and in launch order, e.g.
 * "sapa_tma_fused_f32_kernel<bwd>,sapa_gath_mma_kernel,sapa_gath_mma_kernel"; "" before the first call.  A host-side
 * record (no device work) meant for tests and diagnostics: they assert which kernel a shape exercised, so that a
 * silent fall-back to a slower kernel cannot pass unnoticed.  With several threads calling at once it describes
 * whichever call started last.  The returned string is valid until the calling thread asks again.
 * No counterpart in the reference. */
const char *sapa_last_kernels(void);
/* ABI version of this header (bumped on any signature change). */
int sapa_abi_version(void);
/* The TMA kernels never spin without a limit: a wait on a shared-memory barrier that gives up (which only a
 * malfunction can cause) makes the kernel return early and sets a flag on the device.  This reads the flags of the
 * current device: 0 = no wait ever gave up, bit 0 = fused forward / backward stage 1, bit 1 = gradient gather,
 * bit 2 = projection GEMM,
 * -1 = the flags could not be read.  Reading a raised flag clears it and resets the tile schedulers of that kernel
 * family (a CTA that gave up leaves its scheduler counters dirty), so the library is usable again afterwards.
 * It synchronises the device; meant for tests and for diagnosing wrong results, not for the hot path.
 * Graph replays: a launch captured into a CUDA graph keeps its scheduler counters for every replay; replays of
 * graphs holding these kernels must not overlap each other on one device (ordinary launches on other streams may
 * overlap them freely).  No counterpart in the reference. */
int sapa_wait_timeout_flags(void);
/* Self-test of that mechanism: launches one small kernel whose bounded wait is certain to give up (it waits a few
 * dozen tries on a barrier that nothing signals, then raises the flag and returns normally; nothing hangs or faults).
 * Afterwards sapa_wait_timeout_flags() reports bit 0 once, and the library works as before. */
int sapa_selftest_wait_timeout(void *stream);

/* ------------------------------------------------------------------ SAPA-B, separate ops ------------- */

/* sim: out[B,K*K,sH,sW] = local query.key similarity.
 * Replaces qk_forward(features=key, masks=query, K, s, output)  — sapa/sapa/src/qk_ext.cpp:22-34,
 * qk_forward_cuda qk_cuda.cpp:41-60, QKForwardLauncher qk_cuda_kernel.cu:71-99. d = query channels. */
int sapa_qk_forward(const void *query, const void *key, void *out,
                    int B, int d, int H, int W, int K, int s, int dtype, void *stream);

/* Gradients of sim.  Replaces qk_backward(top_grad, key, query, K, s, grad_key, grad_query)
 * — qk_ext.cpp:36-50, qk_backward_cuda qk_cuda.cpp:62-84, QKBackwardLauncher qk_cuda_kernel.cu:139-171.
 * Deterministic (gather form, no atomics). */
int sapa_qk_backward(const void *grad_out, const void *query, const void *key,
                     void *grad_query, void *grad_key,
                     int B, int d, int H, int W, int K, int s, int dtype, void *stream);

/* atn: out[B,C,sH,sW] = attention-weighted sum over the K x K value window.
 * Replaces av_forward(features=value, masks=attn, K, s, output) — sapa/sapa/src/av_ext.cpp:18-30,
 * av_forward_cuda av_cuda.cpp:28-47, AVForwardLauncher av_cuda_kernel.cu:77-101. */
int sapa_av_forward(const void *attn, const void *value, void *out,
                    int B, int C, int H, int W, int K, int s, int dtype, void *stream);

/* Gradients of atn.  Replaces av_backward(top_grad, value, attn, K, s, grad_value, grad_attn)
 * — av_ext.cpp:32-46, av_backward_cuda av_cuda.cpp:49-70, AVBackwardLauncher av_cuda_kernel.cu:150-181.
 * Deterministic (gather form, no atomics). */
int sapa_av_backward(const void *grad_out, const void *attn, const void *value,
                     void *grad_attn, void *grad_value,
                     int B, int C, int H, int W, int K, int s, int dtype, void *stream);

/* ------------------------------------------------------------------ SAPA-B, fused --------------------- */

/* out = atn(softmax_k(sim(query, key)), value) in one kernel: what SAPA.attention computes with three
 * launches and two HBM round trips of the attention map (sapa_base.py:38-40).  `attn` may be NULL
 * (inference); when given, the [B,K*K,sH,sW] softmax output is also stored for the backward pass.
 * Returns SAPA_ERR_UNSUPPORTED for (K, s) without a fused kernel (supported: K in {3,5}, s = 2, and
 * dtype != SAPA_F64). */
int sapa_fused_forward(const void *query, const void *key, const void *value, void *out, void *attn,
                       int B, int d, int C, int H, int W, int K, int s, int dtype, void *stream);

/* Row-slab form of sapa_fused_forward for one spatial shard of a larger image: key and value hold
 * `halo_top` extra low-res rows above and `halo_bottom` below the H rows whose outputs are produced
 * (so they are [B, ., halo_top+H+halo_bottom, W]); rows beyond those halos read as zero.  With a halo of
 * (K-1)/2 rows taken from the neighbouring shards the result equals the matching rows of the unsharded
 * call.  No counterpart in the reference (it has no multi-device code). */
int sapa_fused_forward_slab(const void *query, const void *key, const void *value, void *out, void *attn,
                            int B, int d, int C, int H, int W, int halo_top, int halo_bottom,
                            int K, int s, int dtype, void *stream);

/* sapa_fused_forward_slab restricted to the band [row_begin, row_end) of the slab's H low-res rows (output rows
 * 2*row_begin .. 2*row_end-1 of `out`, which is still the slab's whole [B,C,2H,2W] tensor, like `query`).  A sharded
 * caller launches the rows that need no halo first and the border bands once the halos have arrived.  Partial bands
 * need K = 5 and rows of 16 bytes (otherwise SAPA_ERR_UNSUPPORTED: call the band [0, H)).  No counterpart in the
 * reference. */
int sapa_fused_forward_slab_rows(const void *query, const void *key, const void *value, void *out, void *attn,
                                 int B, int d, int C, int H, int W, int halo_top, int halo_bottom,
                                 int row_begin, int row_end, int K, int s, int dtype, void *stream);

/* Bytes of scratch sapa_fused_backward needs (grad of the logits, [B,K*K,sH,sW] elements of dtype). */
size_t sapa_fused_backward_workspace(int B, int H, int W, int K, int s, int dtype);

/* Gradients of the fused op with respect to query, key and value from grad_out and the attention map
 * saved by sapa_fused_forward: the chain AVBackward -> softmax backward -> QKBackward of the reference
 * (sapa_func.py:80-93, 35-48).  Works for every odd K and s >= 1.  Deterministic. */
int sapa_fused_backward(const void *grad_out, const void *query, const void *key, const void *value,
                        const void *attn, void *grad_query, void *grad_key, void *grad_value,
                        void *workspace, size_t workspace_bytes,
                        int B, int d, int C, int H, int W, int K, int s, int dtype, void *stream);

/* Same gradients as sapa_fused_backward for callers that cannot allocate device memory where they call it
 * (engines that run under a memory plan fixed when they were built, plugin hosts whose allocator the op cannot
 * reach, real-time loops that forbid cudaMalloc after start-up because it synchronises the device).  It has no counterpart in the reference.
 * The scratch for the logit gradients is a 16 MiB array built into the library, so:
 *   - every GPU that loads the library holds those 16 MiB until the process exits;
 *   - problems whose scratch (sapa_fused_backward_workspace) exceeds sapa_fused_backward_static_capacity()
 *     are refused with SAPA_ERR_WORKSPACE (B=8, 64x64 -> 128x128 in float32 needs 13.1 MB and fits);
 *   - the first call on each device looks the array's address up (cudaGetSymbolAddress, with that device
 *     current); make that first call before any stream capture begins.  The address is cached for the life of the
 *     process: it assumes the device's primary context is never reset (cudaDeviceReset) while the library is loaded;
 *   - all calls share the one array, which keeps the previous call's contents (nothing needs clearing: it is
 *     fully rewritten before it is read), so two calls that overlap on the GPU (different streams) race.
 * Neither this function nor anything it calls allocates or frees memory. */
size_t sapa_fused_backward_static_capacity(void);
int sapa_fused_backward_static(const void *grad_out, const void *query, const void *key, const void *value,
                               const void *attn, void *grad_query, void *grad_key, void *grad_value,
                               int B, int d, int C, int H, int W, int K, int s, int dtype, void *stream);

/* ------------------------------------------------------------------ SAPA-D (deformable) -------------- */
/* offset is [B, G*P*2, sH, sW]; channel 2*(g*P+p) is the x (w) offset and 2*(g*P+p)+1 the y (h) offset,
 * in low-res pixels, added to the integer parent index (qh/s, qw/s) (deform_qk_cuda_kernel.cu:172-183).
 * Sampling is bilinear with zero outside the image; a point outside (-1,H)x(-1,W) contributes nothing. */

/* out[B,G,P,sH,sW].  Replaces deform_qk_forward(query,key,offset,P,s,G,output) — deformsapa/deformsapa/
 * src/deform_qk.cpp:32-48, deform_qk_forward_cuda deform_qk_cuda.cpp:45-68, launcher
 * deform_qk_cuda_kernel.cu:199-230.  Cq = number of query/key channels (all groups). */
int sapa_deform_qk_forward(const void *query, const void *key, const void *offset, void *out,
                           int B, int Cq, int H, int W, int P, int s, int G, int dtype, void *stream);

/* Replaces deform_qk_backward(top_grad,query,key,offset,P,s,G,grad_query,grad_key,grad_offset)
 * — deform_qk.cpp:50-70, deform_qk_cuda.cpp:70-100, launcher deform_qk_cuda_kernel.cu:298-337.
 * grad_query and grad_key are accumulated with atomics (data-dependent scatter), so for SAPA_F16 /
 * SAPA_BF16 they must be FLOAT32 buffers of the same shape (the caller casts afterwards); grad_offset
 * has the call's dtype.  All three are overwritten. */
int sapa_deform_qk_backward(const void *grad_out, const void *query, const void *key, const void *offset,
                            void *grad_query, void *grad_key, void *grad_offset,
                            int B, int Cq, int H, int W, int P, int s, int G, int dtype, void *stream);

/* out[B,C,sH,sW].  Replaces deform_av_forward(attn,value,offset,P,s,G,output) — deform_av.cpp:32-48,
 * deform_av_cuda.cpp:45-68, launcher deform_av_cuda_kernel.cu:197-228. */
int sapa_deform_av_forward(const void *attn, const void *value, const void *offset, void *out,
                           int B, int C, int H, int W, int P, int s, int G, int dtype, void *stream);

/* Replaces deform_av_backward(top_grad,attn,value,offset,P,s,G,grad_attn,grad_value,grad_offset)
 * — deform_av.cpp:50-70, deform_av_cuda.cpp:70-100, launcher deform_av_cuda_kernel.cu:294-333.
 * grad_value is a scatter target: FLOAT32 buffer for SAPA_F16 / SAPA_BF16.  All three are overwritten. */
int sapa_deform_av_backward(const void *grad_out, const void *attn, const void *value, const void *offset,
                            void *grad_attn, void *grad_value, void *grad_offset,
                            int B, int C, int H, int W, int P, int s, int G, int dtype, void *stream);

/* out = deform_av(softmax_p(deform_qk(query, key, offset)), value, offset) in one kernel — what
 * SAPADeform.attention computes with three launches (sapa_deform.py:51-53).  `attn` ([B,G,P,sH,sW]) may
 * be NULL.  Supported: P <= 16, dtype != SAPA_F64; otherwise SAPA_ERR_UNSUPPORTED. */
int sapa_deform_fused_forward(const void *query, const void *key, const void *value, const void *offset,
                              void *out, void *attn,
                              int B, int Cq, int C, int H, int W, int P, int s, int G, int dtype, void *stream);

/* The same result as sapa_deform_fused_forward by way of the SAPA-B kernels, for s = 2 and float32 (float16 / bfloat16
 * too when W is a multiple of 8: 16-bit operands, float32 similarity in the workspace): with offsets inside
 * [-2, 2) low-res pixels every sampling point falls into the 5 x 5 window of the pixel's parent, so the logits are
 * bilinear combinations of the dense 25-slot similarity of each group (one call of the sim kernel with the B x G
 * groups as images) and the aggregation is the 5 x 5 aggregation with per-group window weights (one call of the agg
 * kernel); a small kernel in between forms the softmax over the points and the window weights and lists the points
 * that leave the window, and a last one adds the listed points to the output, one read-modify-write per output element
 * and no atomics, so the result is deterministic (any offset is handled, large ones just cost more).  Several times faster than sapa_deform_fused_forward at B=8, C=256, 64x64 -> 128x128.
 * `workspace` holds the dense similarity, the window weights and the list: sapa_deform_fused_forward_workspace()
 * bytes, 16-byte aligned, owned by the caller.  `attn` (optional) receives the attention over the points.  Other
 * configurations return SAPA_ERR_UNSUPPORTED (the workspace query returns 0 for them).
 * No counterpart in the reference. */
size_t sapa_deform_fused_forward_workspace(int B, int H, int W, int P, int s, int G, int dtype);
int sapa_deform_fused_forward_dense(const void *query, const void *key, const void *value, const void *offset,
                                    void *out, void *attn, void *workspace, size_t workspace_bytes,
                                    int B, int Cq, int C, int H, int W, int P, int s, int G, int dtype, void *stream);

/* sapa_deform_fused_forward_dense for one row slab of a larger image (row-slab sharding of SAPA-D across GPUs): `key` and
 * `value` hold halo_top + H + halo_bottom low-res rows per plane - the slab's own H rows with the neighbouring slabs'
 * rows above and below (zeros where the image ends) - while `query`, `offset`, `out` and `attn` hold only the slab's own
 * s*H high-res rows.  Exact when no sampling point of the slab reaches further than the halo (the caller derives the
 * halo depth from max |offset_y|; rows beyond it read as outside the image).  Workspace as for H rows.
 * No counterpart in the reference. */
int sapa_deform_fused_forward_slab(const void *query, const void *key, const void *value, const void *offset,
                                   void *out, void *attn, void *workspace, size_t workspace_bytes,
                                   int B, int Cq, int C, int H, int W, int halo_top, int halo_bottom,
                                   int P, int s, int G, int dtype, void *stream);

/* sapa_deform_qk_forward and sapa_deform_av_forward by way of the dense 5 x 5 window (s = 2; float32, or float16 /
 * bfloat16 with W a multiple of 8): the two halves of
 * sapa_deform_fused_forward_dense with the reference's op boundaries - raw logits out (deform_qk_cuda_kernel.cu:139-197)
 * and attention in (deform_av_cuda_kernel.cu:139-195).  Same results as the gather kernels; `workspace`:
 * sapa_deform_fused_forward_workspace() bytes, 16-byte aligned. */
int sapa_deform_qk_forward_dense(const void *query, const void *key, const void *offset, void *out, void *workspace,
                                 size_t workspace_bytes, int B, int Cq, int H, int W, int P, int s, int G, int dtype,
                                 void *stream);
int sapa_deform_av_forward_dense(const void *attn, const void *value, const void *offset, void *out, void *workspace,
                                 size_t workspace_bytes, int B, int C, int H, int W, int P, int s, int G, int dtype,
                                 void *stream);

/* sapa_deform_av_backward and sapa_deform_qk_backward by way of the dense 5 x 5 window (s = 2; float32, or float16 /
 * bfloat16 with W a multiple of 8): the two halves of sapa_deform_fused_backward_dense without the softmax between them
 * (deform_av_cuda_kernel.cu:230-292, deform_qk_cuda_kernel.cu:233-296).  All gradients have the type and the shapes of
 * their inputs and are overwritten; `workspace`: sapa_deform_fused_backward_workspace() bytes, 16-byte aligned, for 16-bit
 * tensors rounded up to 16 plus sapa_deform_fused_backward_scatter_bytes(B, 0, C, ...) (av) or (B, Cq, 0, ...) (qk). */
int sapa_deform_av_backward_dense(const void *grad_out, const void *attn, const void *value, const void *offset,
                                  void *grad_attn, void *grad_value, void *grad_offset, void *workspace,
                                  size_t workspace_bytes, int B, int C, int H, int W, int P, int s, int G, int dtype,
                                  void *stream);
int sapa_deform_qk_backward_dense(const void *grad_out, const void *query, const void *key, const void *offset,
                                  void *grad_query, void *grad_key, void *grad_offset, void *workspace,
                                  size_t workspace_bytes, int B, int Cq, int H, int W, int P, int s, int G, int dtype,
                                  void *stream);

/* The same gradients as sapa_deform_fused_backward by way of the SAPA-B kernels, for s = 2 and float32 (the backward
 * counterpart of sapa_deform_fused_forward_dense): two similarity launches (Q x Key and dOut x Value per group), one
 * per-pixel kernel (softmax backward over the points, logit-gradient and weight windows, offset gradients), one
 * aggregation launch (dQ) and two gather launches (dKey, dV) - deterministic for every point inside the 5 x 5 window;
 * the points outside it are listed and added by a last kernel with atomics.  All four gradients have the type and the
 * shapes of their inputs and are overwritten.  float16 / bfloat16 (W a multiple of 8): 16-bit operands in the tensor-core
 * kernels, float32 similarities in the workspace, 16-bit gradients (the listed points then add with 16-bit atomics).  `workspace`: sapa_deform_fused_backward_workspace() bytes, 16-byte
 * aligned.  Other configurations: SAPA_ERR_UNSUPPORTED (the workspace query returns 0).  No counterpart in the reference. */
size_t sapa_deform_fused_backward_workspace(int B, int H, int W, int P, int s, int G, int dtype);
/* float16 / bfloat16 only (0 otherwise): bytes of the float32 side buffers in which the key / value gradients of the
 * listed points are collected.  sapa_deform_fused_backward_dense then needs a workspace of
 * round_up(sapa_deform_fused_backward_workspace(), 16) + sapa_deform_fused_backward_scatter_bytes() bytes. */
size_t sapa_deform_fused_backward_scatter_bytes(int B, int Cq, int C, int H, int W, int dtype);
int sapa_deform_fused_backward_dense(const void *grad_out, const void *query, const void *key, const void *value,
                                     const void *offset, const void *attn, void *grad_query, void *grad_key, void *grad_value,
                                     void *grad_offset, void *workspace, size_t workspace_bytes, int B, int Cq, int C, int H,
                                     int W, int P, int s, int G, int dtype, void *stream);

/* Backward of sapa_fused_forward_slab for one row slab (multi-GPU row sharding; no counterpart in the reference).
 * grad_out / query / attn are the slab's own rows; key / value are the padded slabs of the forward
 * [B, *, halo_top + H + halo_bottom, W]; grad_query [B, d, sH, sW]; grad_key / grad_value come out in the same padded
 * frame as key / value: rows [halo_top, halo_top + H) are the slab's contribution to its own rows, the halo rows its
 * contribution to the neighbouring slabs' edge rows - the caller sends those to the neighbours and adds what it
 * receives to its own first / last rows.  Workspace as for sapa_fused_backward (sized for the slab).  Needs K = 5,
 * s = 2 and rows of 16 bytes (SAPA_ERR_UNSUPPORTED otherwise).  Deterministic. */
int sapa_fused_backward_slab(const void *grad_out, const void *query, const void *key, const void *value, const void *attn,
                             void *grad_query, void *grad_key, void *grad_value, void *workspace, size_t workspace_bytes,
                             int B, int d, int C, int H, int W, int halo_top, int halo_bottom, int K, int s, int dtype,
                             void *stream);

/* sapa_fused_forward for channels-last tensors: query [B, sH, sW, d], key [B, H, W, d], value [B, H, W, C] ->
 * out [B, sH, sW, C]; `attn` (optional) receives the attention as [B, sH, sW, K*K].  Same arithmetic and border rule as
 * the channels-first entry point (sapa_base.py:38-40).  Needs K <= 5, d and C multiples of 16 bytes worth of elements and
 * 16-byte aligned tensors (SAPA_ERR_UNSUPPORTED / SAPA_ERR_ALIGNMENT otherwise); float32, float16, bfloat16; forward only.
 * No counterpart in the reference, whose tensors are channels-first throughout. */
int sapa_fused_forward_nhwc(const void *query, const void *key, const void *value, void *out, void *attn,
                            int B, int d, int C, int H, int W, int K, int s, int dtype, void *stream);

/* GroupNorm followed by the 1 x 1 projection that produces the query or the key (reference: sapa_base.py:27-34,
 * sapa_deform.py:35-42 - `self.q(self.norm_y(y))`, `self.k(self.norm_x(x))`), forward only:
 *   out[b, j, p] = bias[j] + sum_c weight[j, c] * (gamma[c] * (x[b, c, p] - mean[b, g(c)]) * rstd[b, g(c)] + beta[c])
 * x [B, C, HW], weight [d, C], bias [d] or NULL, gamma / beta [C], out [B, d, HW]; `groups` = number of GroupNorm groups
 * (32 in the reference modules), 0 = no normalisation (gamma, beta ignored; `norm=False`).  The statistics take one pass
 * over x, the normalisation is folded into per-image weights, and the product runs as one tcgen05 GEMM that reads x once
 * more: the normalised tensor is never written.  float32 is evaluated as a three-term tf32 product (float32 accuracy).
 * `workspace`: sapa_project_workspace() bytes, 256-byte aligned, owned by the caller.  Needs d % 16 == 0, d <= 256,
 * HW * esize and C * esize multiples of 16 and, with groups > 0, C % groups == 0; otherwise SAPA_ERR_UNSUPPORTED (the
 * workspace query returns 0) and the caller uses its own GroupNorm + convolution.  No counterpart in the reference's
 * extensions (the reference runs these as torch modules). */
size_t sapa_project_workspace(int B, int C, int HW, int d, int groups, int dtype);
int sapa_project_forward(const void *x, const void *gamma, const void *beta, const void *weight, const void *bias, void *out,
                         void *workspace, size_t workspace_bytes, int B, int C, int HW, int d, int groups, float eps,
                         int dtype, void *stream);

/* Gradients of sapa_deform_fused_forward with respect to query, key, value and offset from grad_out and the
 * attention map it saved, in one kernel: the chain DeformAVBackward -> softmax backward over the points ->
 * DeformQKBackward of the reference (deform_av_cuda_kernel.cu:230-292, sapa_deform.py:52, deform_qk_cuda_kernel.cu:
 * 233-296) with the offsets and the attention read once and the two offset gradients added in the kernel (autograd
 * adds them in the reference, because the offset feeds both ops).  grad_key and grad_value are scatter targets
 * (float atomics): FLOAT32 buffers for SAPA_F16 / SAPA_BF16, like grad_query (FLOAT64 for SAPA_F64); grad_offset has the
 * call's dtype.  All four are overwritten.  Supported: P <= 16; otherwise SAPA_ERR_UNSUPPORTED. */
int sapa_deform_fused_backward(const void *grad_out, const void *query, const void *key, const void *value,
                               const void *offset, const void *attn,
                               void *grad_query, void *grad_key, void *grad_value, void *grad_offset,
                               int B, int Cq, int C, int H, int W, int P, int s, int G, int dtype, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SAPA_B200_H_ */
