"""The benchmark configurations at FULL size against the CPU oracle (the oracle only ever sees the part of a
configuration it can finish in seconds: one image of a batch, or a band of rows with the halo it depends on).

config 2: B=8, C=256, d=64, 64^2 -> 128^2, 16-bit element types, forward and backward (float32 is in test_parity_gpu.py)
config 3: SAPA-D, B=8, C=256, 4 groups x 9 points, offsets ~ N(0, 0.5^2): backward in float32 and forward in bfloat16
config 5a: B=64, C=256, 128^2 -> 256^2, bfloat16 (the batch-sharded scaling workload)
config 5b: B=1, C=256, 1024^2 -> 2048^2, bfloat16, as two row slabs with real halos (the row-sharded scaling workload);
           its tensors pass 2^31 bytes, which is what the 64-bit indexing of the kernels is for.
Tolerances: 1e-2 forward / 3e-2 backward for 16-bit types against the oracle on the rounded inputs, 2e-5 for float32
gradients (norm-relative error max|a-b| / max|b|)."""
import numpy as np
import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def sp():
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    import sapa_b200
    return sapa_b200


def host64(t):
    return t.detach().double().cpu().numpy()


def f32(t):
    return t.detach().float().cpu().numpy()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_config2_16bit_full_size_vs_oracle(sp, oracle, dtype):
    from sapa_b200 import _lib
    B, d, C, H, W, K, s = 8, 64, 256, 64, 64, 5, 2
    g = torch.Generator().manual_seed(1)
    q, k, v, go = (torch.randn(*sh, generator=g).to(dtype) for sh in
                   ((B, d, s * H, s * W), (B, d, H, W), (B, C, H, W), (B, C, s * H, s * W)))
    want = oracle.sapa_forward(f32(q), f32(k), f32(v), K, s)                    # float32 oracle on the rounded inputs
    wq, wk, wv = oracle.sapa_backward(f32(go), f32(q), f32(k), f32(v), K, s)
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = sp.sapa_fused(qd, kd, vd, K, s)
    torch.cuda.synchronize()
    assert _lib.last_kernels() == ["sapa_tma_fused_16_kernel<fwd>"]
    assert rel_err(host64(out), want) < 1e-2
    fq, fk, fv = torch.autograd.grad(out, (qd, kd, vd), go.to(DEV))
    torch.cuda.synchronize()
    assert _lib.last_kernels() == ["sapa_tma_fused_16_kernel<bwd>", "sapa_gath_mma_kernel", "sapa_gath_mma_kernel"]
    for got, ref in ((fq, wq), (fk, wk), (fv, wv)):
        assert rel_err(host64(got), ref) < 3e-2


def test_config3_full_size_backward_and_bf16_vs_oracle(sp, oracle):
    B, Cq, C, H, W, P, G, s = 8, 64, 256, 64, 64, 9, 4, 2
    g = torch.Generator().manual_seed(3)
    q = torch.randn(B, Cq, s * H, s * W, generator=g)
    k = torch.randn(B, Cq, H, W, generator=g)
    v = torch.randn(B, C, H, W, generator=g)
    off = torch.randn(B, G * P * 2, s * H, s * W, generator=g) * 0.5
    go = torch.randn(B, C, s * H, s * W, generator=g)
    img = 5
    t = [x.to(DEV).requires_grad_() for x in (q, k, v, off)]
    out = sp.deform_sapa_fused(*t, P, s, G)
    grads = torch.autograd.grad(out, t, go.to(DEV))
    one = [x[img:img + 1].numpy() for x in (q, k, v, off)]
    want = oracle.deform_sapa_backward(go[img:img + 1].numpy(), *one, P, s, G)    # images are independent
    for got, ref in zip(grads, want):
        assert rel_err(host64(got[img:img + 1]), ref) < 2e-5
    # bfloat16 forward and backward of the same image, against the float32 oracle on the rounded inputs
    tb = [x[img:img + 1].to(torch.bfloat16) for x in (q, k, v, off)]
    rb = [f32(x) for x in tb]
    gob = go[img:img + 1].to(torch.bfloat16)
    td = [x.to(DEV).requires_grad_() for x in tb]
    outb = sp.deform_sapa_fused(*td, P, s, G)
    assert rel_err(host64(outb), oracle.deform_sapa_forward(*rb, P, s, G)) < 1e-2
    gb = torch.autograd.grad(outb, td, gob.to(DEV))
    wb = oracle.deform_sapa_backward(f32(gob), *rb, P, s, G)
    for got, ref in zip(gb, wb):
        assert rel_err(host64(got), ref) < 3e-2


def test_config5a_batch_of_64_bf16_one_image_vs_oracle(sp, oracle):
    from sapa_b200.functions import fused_forward_raw
    B, d, C, H, W, K, s = 64, 64, 256, 128, 128, 5, 2
    g = torch.Generator().manual_seed(5)
    q = torch.randn(B, d, s * H, s * W, generator=g, dtype=torch.bfloat16).to(DEV)
    k = torch.randn(B, d, H, W, generator=g, dtype=torch.bfloat16).to(DEV)
    v = torch.randn(B, C, H, W, generator=g, dtype=torch.bfloat16).to(DEV)
    out, _ = fused_forward_raw(q, k, v, K, s, False)
    for img in (0, 37, 63):      # first, one in the middle, last (the last image ends 3.2 GB into the output)
        want = oracle.sapa_forward(f32(q[img:img + 1]), f32(k[img:img + 1]), f32(v[img:img + 1]), K, s)
        assert rel_err(host64(out[img:img + 1]), want) < 1e-2


def test_config5b_2048_square_row_slabs_with_real_halos_vs_oracle(sp, oracle):
    """One 1024^2 -> 2048^2 image as two slabs of 512 low-res rows, each with the r = 2 halo rows of its neighbour (what
    the halo exchange delivers) and zero rows at the image border; three bands of output rows are compared with the
    oracle run on the rows they depend on: the top border, the slab boundary and the bottom border."""
    from sapa_b200.functions import fused_forward_raw
    B, d, C, H, W, K, s, r = 1, 64, 256, 1024, 1024, 5, 2, 2
    g = torch.Generator().manual_seed(6)
    q = torch.randn(B, d, s * H, s * W, generator=g, dtype=torch.bfloat16).to(DEV)
    k = torch.randn(B, d, H, W, generator=g, dtype=torch.bfloat16).to(DEV)
    v = torch.randn(B, C, H, W, generator=g, dtype=torch.bfloat16).to(DEV)
    kp, vp = (torch.nn.functional.pad(x, (0, 0, r, r)) for x in (k, v))
    half = H // 2
    slabs = []
    for a in (0, half):
        o, _ = fused_forward_raw(q[:, :, s * a:s * (a + half)].contiguous(), kp[:, :, a:a + half + 2 * r].contiguous(),
                                 vp[:, :, a:a + half + 2 * r].contiguous(), K, s, False, halo=(r, r))
        slabs.append(o)
    out = torch.cat(slabs, dim=2)
    assert out.shape == (B, C, s * H, s * W) and out.numel() * out.element_size() >= 2 ** 31

    def band(a, b):
        lo, hi = max(a - r, 0), min(b + r, H)           # rows the band depends on (zero padding beyond the image)
        want = oracle.sapa_forward(f32(q[:, :, s * lo:s * hi]), f32(k[:, :, lo:hi]), f32(v[:, :, lo:hi]), K, s)
        return rel_err(host64(out[:, :, s * a:s * b]), want[:, :, s * (a - lo):s * (b - lo)])

    assert band(0, 6) < 1e-2
    assert band(half - 4, half + 4) < 1e-2
    assert band(H - 6, H) < 1e-2


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_row_slab_backward_of_two_slabs_sums_to_the_unsharded_gradients(dtype, tol):
    """sapa_fused_backward_slab on the two halves of an image (halos copied from the other half, as the exchange would):
    grad_query of each half equals the unsharded rows bit for bit; the key / value gradients, with the halo rows of each
    half added to the other half's edge rows, equal the unsharded gradients to rounding."""
    import sapa_b200
    from sapa_b200 import _lib, sharding
    dev = torch.device("cuda:0")
    B, d, C, H, W, K, s, r = 2, 32, 48, 24, 40, 5, 2, 2
    g = torch.Generator().manual_seed(23)
    q, k, v, go = (torch.randn(*sh, generator=g).to(dev, dtype) for sh in
                   ((B, d, s * H, s * W), (B, d, H, W), (B, C, H, W), (B, C, s * H, s * W)))
    qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))
    gq, gk, gv = torch.autograd.grad(sapa_b200.sapa_fused(qf, kf, vf, K, s), (qf, kf, vf), go)
    kp, vp = (torch.nn.functional.pad(t, (0, 0, r, r)) for t in (k, v))
    sum_k, sum_v = torch.zeros_like(kp, dtype=torch.float32), torch.zeros_like(vp, dtype=torch.float32)
    hl = H // 2
    for half in range(2):
        rows, hi = slice(half * hl, (half + 1) * hl), slice(s * half * hl, s * (half + 1) * hl)
        slab = sharding.RowSlab(B, d, C, hl, W, dtype, dev, K, s)
        slab.key_padded.copy_(kp[:, :, half * hl:half * hl + hl + 2 * r])
        slab.value_padded.copy_(vp[:, :, half * hl:half * hl + hl + 2 * r])
        ql = q[:, :, hi].contiguous()
        out = slab.forward(ql, keep_attn=True)
        code = _lib.dtype_code(ql)
        mq = torch.empty_like(ql)
        mk, mv = torch.empty_like(slab.key_padded), torch.empty_like(slab.value_padded)
        nb = _lib.fused_backward_workspace(B, hl, W, K, s, code)
        ws = torch.empty(nb, dtype=torch.uint8, device=dev)
        _lib.call("sapa_fused_backward_slab", dev, go[:, :, hi].contiguous(), ql, slab.key_padded, slab.value_padded, slab.attn,
                  mq, mk, mv, ws, nb, B, d, C, hl, W, r, r, K, s, code)
        assert _lib.last_kernels() == [f"sapa_tma_fused_{'f32' if dtype == torch.float32 else '16'}_kernel<bwd>",
                                       "sapa_gath_mma_kernel", "sapa_gath_mma_kernel"]
        assert torch.equal(mq, gq[:, :, hi])
        sum_k[:, :, half * hl:half * hl + hl + 2 * r] += mk.float()
        sum_v[:, :, half * hl:half * hl + hl + 2 * r] += mv.float()
    for got, want in ((sum_k[:, :, r:r + H], gk), (sum_v[:, :, r:r + H], gv)):
        assert float((got - want.float()).abs().max()) <= tol * float(want.float().abs().max())


DEFORM_SHAPES = [
    # B, Cq, C, H, W, P, G, sigma
    (1, 8, 8, 5, 8, 1, 1, 0.5),          # one point, one group
    (2, 16, 24, 7, 12, 4, 2, 0.8),       # rows of 16 bytes (tensor-map kernels), four points
    (1, 12, 20, 6, 9, 9, 4, 0.5),        # odd width: the tiled / generic SAPA-B kernels under the dense path
    (2, 32, 32, 8, 16, 16, 4, 2.5),      # the largest point count, most points outside the window
    (1, 16, 16, 4, 4, 9, 2, 6.0),        # offsets that leave the image
]


@pytest.mark.parametrize("shape", DEFORM_SHAPES, ids=lambda s: "B%d_q%d_c%d_%dx%d_P%d_G%d_s%g" % s)
def test_dense_window_deform_matches_the_separate_ops(shape):
    """SAPA-D fused forward and backward (dense 5x5 window path for s = 2) against the chain of separate ops, which the
    golden tests pin to the reference: outputs and all four gradients, ragged shapes, every point count, offsets from
    well inside the window to far outside the image."""
    import sapa_b200
    from sapa_b200 import _lib
    B, Cq, C, H, W, P, G, sigma = shape
    dev, s = torch.device("cuda:0"), 2
    g = torch.Generator().manual_seed(31)
    q, k, v, off, go = (torch.randn(*sh, generator=g).to(dev) for sh in
                        ((B, Cq, s * H, s * W), (B, Cq, H, W), (B, C, H, W), (B, G * P * 2, s * H, s * W), (B, C, s * H, s * W)))
    off = off * sigma
    a = [t.clone().requires_grad_() for t in (q, k, v, off)]
    out = sapa_b200.deform_sapa_fused(*a, P, s, G)
    assert "deform_window_kernel" in _lib.last_kernels()
    grads = torch.autograd.grad(out, a, go)
    assert "deform_window_bwd_kernel" in _lib.last_kernels()
    b = [t.clone().requires_grad_() for t in (q, k, v, off)]
    ref = sapa_b200.deform_av(torch.softmax(sapa_b200.deform_qk(b[0], b[1], b[3], P, s, G), dim=2), b[2], b[3], P, s, G)
    ref_grads = torch.autograd.grad(ref, b, go)
    for got, want in [(out.detach(), ref.detach())] + list(zip(grads, ref_grads)):
        scale = float(want.abs().max())
        assert float((got - want).abs().max()) <= 1e-5 * max(scale, 1e-30)
    assert _lib.wait_timeout_flags(dev) == 0


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 3e-2), (torch.float16, 4e-3)])
@pytest.mark.parametrize("sigma", [0.5, 1.5])
def test_deform_16bit_dense_window_forward_and_backward(sp, dtype, tol, sigma):
    """float16 / bfloat16 SAPA-D with rows of 16 bytes runs the dense-window chain natively (16-bit operands, float32
    similarities, 16-bit window weights; the scattered gradients of far points are collected in float32): output and all
    four gradients against the float32 chain on the same rounded inputs, also with a quarter of the points far."""
    from sapa_b200 import _lib
    B, d, C, H, W, G, P, s = 2, 32, 64, 20, 24, 4, 9, 2
    g = torch.Generator(device=DEV).manual_seed(43)
    shapes = ((B, d, s * H, s * W), (B, d, H, W), (B, C, H, W), (B, 2 * G * P, s * H, s * W), (B, C, s * H, s * W))
    q, k, v, off, go = (torch.randn(*sh, generator=g, device=DEV) for sh in shapes)
    t16 = [t.to(dtype).requires_grad_() for t in (q, k, v, sigma * off)]
    t32 = [t.detach().float().requires_grad_() for t in t16]
    go16 = go.to(dtype)
    out = sp.deform_sapa_fused(*t16, P, s, G)
    assert _lib.last_kernels()[0] == "sapa_tma_fused_16_kernel<sim>"
    got = torch.autograd.grad(out, t16, go16)
    kernels = _lib.last_kernels()
    assert kernels[:2] == ["sapa_tma_fused_16_kernel<sim>"] * 2 and kernels[-1] == "deform_add_scatter_kernel"
    ref_out = sp.deform_sapa_fused(*t32, P, s, G)
    ref = torch.autograd.grad(ref_out, t32, go16.float())
    for a, b in [(out, ref_out)] + list(zip(got, ref)):
        assert a.dtype == dtype
        assert rel_err(f32(a), f32(b)) < tol
    assert _lib.wait_timeout_flags(torch.device(DEV)) == 0


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 3e-2), (torch.float16, 4e-3)])
def test_deform_16bit_separate_ops_through_the_window(sp, dtype, tol):
    """deform_qk / deform_av and their backward in float16 / bfloat16 (rows of 16 bytes) run through the dense window like
    float32; results and gradients against the float32 ops on the same rounded inputs (sigma = 1: a quarter of the
    points leave the window, so the float32 side buffers of the scattered gradients are exercised)."""
    from sapa_b200 import _lib
    B, d, C, H, W, G, P, s = 2, 32, 64, 20, 24, 4, 9, 2
    g = torch.Generator(device=DEV).manual_seed(47)
    shapes = ((B, d, s * H, s * W), (B, d, H, W), (B, C, H, W), (B, 2 * G * P, s * H, s * W), (B, G, P, s * H, s * W),
              (B, C, s * H, s * W))
    q, k, v, off, gs, go = (torch.randn(*sh, generator=g, device=DEV) for sh in shapes)
    q16, k16, v16, o16 = (t.to(dtype).requires_grad_() for t in (q, k, v, off))
    q32, k32, v32, o32 = (t.detach().float().requires_grad_() for t in (q16, k16, v16, o16))
    sim = sp.deform_qk(q16, k16, o16, P, s, G)
    assert _lib.last_kernels() == ["sapa_tma_fused_16_kernel<sim>", "deform_window_kernel<logits>"]
    got = torch.autograd.grad(sim, (q16, k16, o16), gs.to(dtype))
    assert _lib.last_kernels()[-1] == "deform_add_scatter_kernel"
    sim32 = sp.deform_qk(q32, k32, o32, P, s, G)
    ref = torch.autograd.grad(sim32, (q32, k32, o32), gs.to(dtype).float())
    for a, b in [(sim, sim32)] + list(zip(got, ref)):
        assert a.dtype == dtype and rel_err(f32(a), f32(b)) < tol
    a16 = torch.softmax(sim32.detach(), dim=2).to(dtype).requires_grad_()
    a32 = a16.detach().float().requires_grad_()
    out = sp.deform_av(a16, v16, o16, P, s, G)
    assert _lib.last_kernels()[:2] == ["deform_window_kernel<weights>", "sapa_tma_fused_16_kernel<agg>"]
    got = torch.autograd.grad(out, (a16, v16, o16), go.to(dtype))
    assert _lib.last_kernels()[-1] == "deform_add_scatter_kernel"
    out32 = sp.deform_av(a32, v32, o32, P, s, G)
    ref = torch.autograd.grad(out32, (a32, v32, o32), go.to(dtype).float())
    for a, b in [(out, out32)] + list(zip(got, ref)):
        assert a.dtype == dtype and rel_err(f32(a), f32(b)) < tol
    assert _lib.wait_timeout_flags(torch.device(DEV)) == 0


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("sigma,halo", [(0.5, None), (1.5, None), (0.2, 2)])
def test_deform_row_slabs_with_halos_equal_the_unsharded_rows(sp, sigma, halo, dtype, tol):
    """sapa_deform_fused_forward_slab on three row slabs of one image (key / value padded with the neighbours' rows, zeros
    at the image's top and bottom; halo depth from max |offset_y|, or a given bound) against the unsharded fused op:
    far points included (sigma = 1.5 sends a quarter of the points out of the 5 x 5 window)."""
    from sapa_b200 import _lib, sharding
    B, d, C, H, W, G, P, s = 2, 32, 64, 36, 24, 4, 9, 2
    g = torch.Generator(device=DEV).manual_seed(41)
    q = torch.randn(B, d, s * H, s * W, generator=g, device=DEV).to(dtype)
    k = torch.randn(B, d, H, W, generator=g, device=DEV).to(dtype)
    v = torch.randn(B, C, H, W, generator=g, device=DEV).to(dtype)
    off = sigma * torch.randn(B, 2 * G * P, s * H, s * W, generator=g, device=DEV)
    if halo is not None:
        off = off.clamp(-halo + 0.05, halo - 0.05)
    off = off.to(dtype)
    full = sp.deform_sapa_fused(q, k, v, off, P, s, G)
    code = _lib.dtype_code(q)
    depth = sharding.deform_halo_rows(off) if halo is None else halo
    assert depth >= int(off[:, 1::2].abs().max()) + 1 and (halo is not None or depth == int(off[:, 1::2].abs().max()) + 1)
    hl = H // 3
    assert depth <= hl
    kp = torch.nn.functional.pad(k, (0, 0, depth, depth))
    vp = torch.nn.functional.pad(v, (0, 0, depth, depth))
    for r in range(3):
        lo, hi = slice(r * hl, (r + 1) * hl), slice(s * r * hl, s * (r + 1) * hl)
        ks = kp[:, :, r * hl:(r + 1) * hl + 2 * depth].contiguous()
        vs = vp[:, :, r * hl:(r + 1) * hl + 2 * depth].contiguous()
        qs, os_ = q[:, :, hi].contiguous(), off[:, :, hi].contiguous()
        nbytes = int(_lib.lib().sapa_deform_fused_forward_workspace(B, hl, W, P, s, G, code))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
        out = torch.empty(B, C, s * hl, s * W, device=DEV, dtype=dtype)
        _lib.call("sapa_deform_fused_forward_slab", q.device, qs, ks, vs, os_, out, None, ws, nbytes, B, d, C, hl, W, depth, depth,
                  P, s, G, code)
        assert "deform_window_kernel" in _lib.last_kernels()
        assert rel_err(f32(out), f32(full[:, :, hi])) < tol, r


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2), (torch.float16, 2e-3)])
@pytest.mark.parametrize("shape", [(2, 16, 24, 9, 13, 5, 2), (1, 8, 8, 1, 1, 5, 2), (2, 32, 64, 7, 6, 3, 2), (1, 8, 16, 5, 4, 5, 4),
                                   (1, 16, 16, 6, 6, 1, 1), (3, 64, 256, 16, 16, 5, 2)],
                         ids=lambda s: "B%d_d%d_C%d_%dx%d_K%d_s%d" % s)
def test_channels_last_forward_matches_channels_first(shape, dtype, tol, oracle):
    """sapa_fused_forward_nhwc against the CPU oracle (through the permuted tensors) and against the channels-first fused
    op: outputs and attention, odd sizes, window sizes 1 / 3 / 5, scale factors 1 / 2 / 4."""
    import sapa_b200
    from sapa_b200 import _lib
    B, d, C, H, W, K, s = shape
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(41)
    q, k, v = (torch.randn(*sh, generator=g).to(dtype) for sh in ((B, d, s * H, s * W), (B, d, H, W), (B, C, H, W)))
    ql, kl, vl = (t.permute(0, 2, 3, 1).contiguous().to(dev) for t in (q, k, v))
    out, attn = sapa_b200.sapa_fused_nhwc(ql, kl, vl, K, s, return_attn=True)
    assert _lib.last_kernels() == ["sapa_nhwc_fwd_kernel"]
    want = oracle.sapa_forward(q.double().numpy(), k.double().numpy(), v.double().numpy(), K, s)
    got = out.permute(0, 3, 1, 2).double().cpu().numpy()
    assert float(np.abs(got - want).max() / np.abs(want).max()) < tol
    if sapa_b200.functions.fused_supported(K, s, dtype):
        from sapa_b200.functions import fused_forward_raw
        ref_out, ref_attn = fused_forward_raw(q.to(dev), k.to(dev), v.to(dev), K, s, True)
        assert float((attn.permute(0, 3, 1, 2).float() - ref_attn.float()).abs().max()) < (1e-5 if dtype == torch.float32 else 1e-2)
    with pytest.raises(NotImplementedError):
        sapa_b200.sapa_fused_nhwc(ql.clone().requires_grad_(), kl, vl, K, s, return_attn=True)
    # gradients: the channels-last forward with the channels-first backward behind it, against the channels-first op
    if sapa_b200.functions.fused_supported(K, s, dtype):
        go = torch.randn(B, s * H, s * W, C, generator=g).to(dtype).to(dev)
        a = [t.clone().requires_grad_() for t in (ql, kl, vl)]
        got = torch.autograd.grad(sapa_b200.sapa_fused_nhwc(*a, K, s), a, go)
        b = [t.to(dev).requires_grad_() for t in (q, k, v)]
        ref = torch.autograd.grad(sapa_b200.sapa_fused(*b, K, s), b, go.permute(0, 3, 1, 2).contiguous())
        for x, y in zip(got, ref):
            assert x.shape == y.permute(0, 2, 3, 1).shape and torch.equal(x, y.permute(0, 2, 3, 1))
