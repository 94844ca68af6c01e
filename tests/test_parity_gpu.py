"""Parity of the CUDA kernels (reached through the C ABI) with the CPU oracle, the committed golden
vectors of the reference, and - when its compiled extensions are present - the reference's own kernels.

Tolerances (norm-relative error max|a-b| / max|b|):
  float32: 1e-5      float64: 1e-11      float16 / bfloat16: 1e-2 (against the oracle on the rounded inputs)
"""
import os
import sys

import numpy as np
import pytest
import torch

from conftest import (ROOT, Golden, expected_agg, expected_fused_backward, expected_fused_forward, expected_sim,
                      golden_cases, rel_err)

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.float64: 1e-11, torch.float16: 1e-2, torch.bfloat16: 1e-2}
DEV = "cuda:0"


@pytest.fixture(scope="module")
def sp():
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    import sapa_b200
    return sapa_b200


def dev(a, dtype):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV, dtype)


def host64(t):
    return t.detach().double().cpu().numpy()


def grads(out, inputs, grad_out):
    return torch.autograd.grad(out, inputs, grad_out)


DTYPE_NAME = {torch.float32: "f32", torch.float64: "f64", torch.float16: "f16", torch.bfloat16: "bf16"}


def ran():
    """Kernels of the most recent entry-point call (host-side record of the library; the backward of an autograd
    Function runs on PyTorch's worker thread, the record is process-wide)."""
    from sapa_b200 import _lib
    torch.cuda.synchronize()
    return _lib.last_kernels()


# ------------------------------------------------------------------ golden vectors, SAPA-B

@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("name", golden_cases("b_"))
def test_sapa_b_golden(sp, name, dtype):
    g = Golden(name)
    K, s = g.meta["K"], g.meta["s"]
    tol = TOL[dtype]
    x = {k: dev(v, dtype) for k, v in g.inputs.items()}
    q, k, v, a = (x[n].clone().requires_grad_() for n in ("query", "key", "value", "attn"))
    sim = sp.qk(q, k, K, s)
    assert rel_err(host64(sim), g.expected["sim"]) < tol
    gq, gk = grads(sim, (q, k), x["grad_sim"])
    assert rel_err(host64(gq), g.expected["sim_dquery"]) < tol
    assert rel_err(host64(gk), g.expected["sim_dkey"]) < tol
    agg = sp.av(a, v, K, s)
    assert rel_err(host64(agg), g.expected["agg"]) < tol
    ga, gv = grads(agg, (a, v), x["grad_out"])
    assert rel_err(host64(ga), g.expected["agg_dattn"]) < tol
    assert rel_err(host64(gv), g.expected["agg_dvalue"]) < tol
    q2, k2, v2 = (x[n].clone().requires_grad_() for n in ("query", "key", "value"))
    full = sp.sapa_fused(q2, k2, v2, K, s)
    assert rel_err(host64(full), g.expected["full"]) < tol
    fq, fk, fv = grads(full, (q2, k2, v2), x["grad_out"])
    assert rel_err(host64(fq), g.expected["full_dquery"]) < 2 * tol
    assert rel_err(host64(fk), g.expected["full_dkey"]) < 2 * tol
    assert rel_err(host64(fv), g.expected["full_dvalue"]) < 2 * tol


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("name", ["b_fwdcheck", "b_wide", "b_k3s1", "b_k7s2"])
def test_sapa_b_half_precision(sp, oracle, name, dtype):
    g = Golden(name)
    K, s = g.meta["K"], g.meta["s"]
    x = {k: dev(v, dtype) for k, v in g.inputs.items()}
    r = {k: host64(v) for k, v in x.items()}           # the rounded inputs, as float64
    q, k, v = (x[n].clone().requires_grad_() for n in ("query", "key", "value"))
    assert rel_err(host64(sp.qk(x["query"], x["key"], K, s)), oracle.qk_forward(r["query"], r["key"], K, s)) < 1e-2
    assert rel_err(host64(sp.av(x["attn"], x["value"], K, s)), oracle.av_forward(r["attn"], r["value"], K, s)) < 1e-2
    full = sp.sapa_fused(q, k, v, K, s)
    assert full.dtype == dtype
    assert rel_err(host64(full), oracle.sapa_forward(r["query"], r["key"], r["value"], K, s)) < 1e-2
    fq, fk, fv = grads(full, (q, k, v), x["grad_out"])
    wq, wk, wv = oracle.sapa_backward(r["grad_out"], r["query"], r["key"], r["value"], K, s)
    assert rel_err(host64(fq), wq) < 2e-2 and rel_err(host64(fk), wk) < 2e-2 and rel_err(host64(fv), wv) < 2e-2


def test_config1_single_op_forward(sp):
    g = Golden("cfg1")
    X, Y, Wq, Wk = (dev(g.inputs[k], torch.float32) for k in ("X", "Y", "Wq", "Wk"))
    q = torch.einsum("oc,bchw->bohw", Wq, Y).contiguous()
    k = torch.einsum("oc,bchw->bohw", Wk, X).contiguous()
    out = sp.sapa_fused(q, k, X, 5, 2)
    assert out.shape == (1, 64, 32, 32)
    assert rel_err(host64(out), g.expected["full"]) < 1e-5
    sep = sp.av(torch.softmax(sp.qk(q, k, 5, 2), dim=1), X, 5, 2)
    assert rel_err(host64(sep), g.expected["full"]) < 1e-5


# ------------------------------------------------------------------ golden vectors, SAPA-D

@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("name", golden_cases("d_"))
def test_sapa_d_golden(sp, name, dtype):
    g = Golden(name)
    P, s, G = g.meta["P"], g.meta["s"], g.meta["G"]
    tol = TOL[dtype]
    x = {k: dev(v, dtype) for k, v in g.inputs.items()}
    q, k, v, a, o = (x[n].clone().requires_grad_() for n in ("query", "key", "value", "attn", "offset"))
    sim = sp.deform_qk(q, k, o, P, s, G)
    assert sim.shape == x["attn"].shape
    assert rel_err(host64(sim), g.expected["sim"]) < tol
    gq, gk, go = grads(sim, (q, k, o), x["grad_sim"])
    assert rel_err(host64(gq), g.expected["sim_dquery"]) < tol
    assert rel_err(host64(gk), g.expected["sim_dkey"]) < tol
    assert rel_err(host64(go), g.expected["sim_doffset"]) < tol
    agg = sp.deform_av(a, v, o, P, s, G)
    assert rel_err(host64(agg), g.expected["agg"]) < tol
    ga, gv, go = grads(agg, (a, v, o), x["grad_out"])
    assert rel_err(host64(ga), g.expected["agg_dattn"]) < tol
    assert rel_err(host64(gv), g.expected["agg_dvalue"]) < tol
    assert rel_err(host64(go), g.expected["agg_doffset"]) < tol
    q2, k2, v2, o2 = (x[n].clone().requires_grad_() for n in ("query", "key", "value", "offset"))
    full = sp.deform_sapa_fused(q2, k2, v2, o2, P, s, G)
    assert rel_err(host64(full), g.expected["full"]) < tol
    fq, fk, fv, fo = grads(full, (q2, k2, v2, o2), x["grad_out"])
    for got, key in ((fq, "full_dquery"), (fk, "full_dkey"), (fv, "full_dvalue"), (fo, "full_doffset")):
        assert rel_err(host64(got), g.expected[key]) < 2 * tol, key


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("name", ["d_fwdcheck", "d_p9g4"])
def test_sapa_d_half_precision(sp, oracle, name, dtype):
    g = Golden(name)
    P, s, G = g.meta["P"], g.meta["s"], g.meta["G"]
    x = {k: dev(v, dtype) for k, v in g.inputs.items()}
    r = {k: host64(v) for k, v in x.items()}
    q, k, v, o = (x[n].clone().requires_grad_() for n in ("query", "key", "value", "offset"))
    full = sp.deform_sapa_fused(q, k, v, o, P, s, G)
    assert rel_err(host64(full), oracle.deform_sapa_forward(r["query"], r["key"], r["value"], r["offset"], P, s, G)) < 1e-2
    sep = sp.deform_av(torch.softmax(sp.deform_qk(x["query"], x["key"], x["offset"], P, s, G), dim=2), x["value"],
                       x["offset"], P, s, G)
    assert rel_err(host64(sep), host64(full)) < 1e-2
    fq, fk, fv, fo = grads(full, (q, k, v, o), x["grad_out"])
    wq, wk, wv, wo = oracle.deform_sapa_backward(r["grad_out"], r["query"], r["key"], r["value"], r["offset"], P, s, G)
    for got, want in ((fq, wq), (fk, wk), (fv, wv), (fo, wo)):
        assert rel_err(host64(got), want) < 3e-2


# ------------------------------------------------------------------ seeded cases against the C oracle

SHAPES_B = [  # B, d, C, H, W: tile overhang in both directions, channel-chunk tails, a single pixel
    (2, 64, 48, 9, 40), (1, 7, 5, 4, 33), (3, 2, 1, 1, 1), (1, 13, 9, 17, 3), (1, 32, 256, 8, 64),
    (4, 16, 40, 64, 64),   # 512 tiles: persistent CTAs take several tiles, 3 stages per tile against a ring of 4
    (1, 8, 24, 6, 10),     # even width that is not a multiple of 4: cp.async forward, tensor-core gather with a ragged tile
    (2, 5, 7, 2, 4),       # an image smaller than one TMA box in both directions
]


@pytest.mark.parametrize("K", [5, 3])
@pytest.mark.parametrize("shape", SHAPES_B)
def test_sapa_b_seeded_vs_oracle(sp, oracle, shape, K):
    B, d, C, H, W = shape
    s = 2
    g = torch.Generator().manual_seed(1234 + H * W + K)
    q = torch.randn(B, d, s * H, s * W, generator=g)
    k = torch.randn(B, d, H, W, generator=g)
    v = torch.randn(B, C, H, W, generator=g)
    go = torch.randn(B, C, s * H, s * W, generator=g)
    want, want_p = oracle.sapa_forward(q.double().numpy(), k.double().numpy(), v.double().numpy(), K, s, return_attn=True)
    wq, wk, wv = oracle.sapa_backward(go.double().numpy(), q.double().numpy(), k.double().numpy(), v.double().numpy(), K, s)
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = sp.sapa_fused(qd, kd, vd, K, s)
    assert ran() == expected_fused_forward(K, s, W, "f32")          # no silent fall-back to a slower kernel
    assert rel_err(host64(out), want) < 1e-5
    fq, fk, fv = grads(out, (qd, kd, vd), go.to(DEV))
    assert ran() == expected_fused_backward(K, s, W, "f32")
    assert rel_err(host64(fq), wq) < 2e-5 and rel_err(host64(fk), wk) < 2e-5 and rel_err(host64(fv), wv) < 2e-5
    # separate path: same numbers from three launches, attention rows sum to one
    sim = sp.qk(qd.detach(), kd.detach(), K, s)
    assert ran() == expected_sim(K, s, W, "f32")
    prob = torch.softmax(sim, dim=1)
    assert rel_err(host64(prob), want_p) < 1e-5
    sep = sp.av(prob, vd.detach(), K, s)
    assert ran() == expected_agg(K, s, W, "f32")
    assert rel_err(host64(sep), want) < 1e-5


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(2, 64, 48, 9, 40), (4, 16, 40, 64, 64), (1, 24, 72, 7, 8), (1, 8, 16, 5, 12), (2, 5, 7, 2, 8)])
def test_sapa_b_half_precision_fused_forward_vs_oracle(sp, oracle, shape, dtype):
    """16-bit fused forward (rows of 16 bytes: tensor-map kernel; W=12: cp.async kernel) against the float64 oracle
    evaluated on the same rounded inputs; tolerance 1e-2 (16-bit probabilities and outputs)."""
    from sapa_b200.functions import fused_forward_raw
    B, d, C, H, W = shape
    K, s = 5, 2
    g = torch.Generator().manual_seed(77 + H * W)
    q, k, v = (torch.randn(*sh, generator=g).to(dtype) for sh in ((B, d, s * H, s * W), (B, d, H, W), (B, C, H, W)))
    want, want_p = oracle.sapa_forward(q.double().numpy(), k.double().numpy(), v.double().numpy(), K, s, return_attn=True)
    out, attn = fused_forward_raw(q.to(DEV), k.to(DEV), v.to(DEV), K, s, True)
    assert ran() == expected_fused_forward(K, s, W, DTYPE_NAME[dtype])
    assert rel_err(host64(out), want) < 1e-2
    assert rel_err(host64(attn), want_p) < 1e-2
    out2, _ = fused_forward_raw(q.to(DEV), k.to(DEV), v.to(DEV), K, s, False)
    assert torch.equal(out, out2)
    # backward through the public op: tensor-core stage 1 (dS, dQ) and the gather kernels (dKey, dV); the oracle
    # differentiates the exact function, the kernels work with 16-bit probabilities and logit gradients
    go = torch.randn(B, C, s * H, s * W, generator=g).to(dtype)
    wq, wk, wv = oracle.sapa_backward(go.double().numpy(), q.double().numpy(), k.double().numpy(), v.double().numpy(), K, s)
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    fq, fk, fv = grads(sp.sapa_fused(qd, kd, vd, K, s), (qd, kd, vd), go.to(DEV))
    assert ran() == expected_fused_backward(K, s, W, DTYPE_NAME[dtype])
    for got, want_g in ((fq, wq), (fk, wk), (fv, wv)):
        assert rel_err(host64(got), want_g) < 3e-2


def test_sapa_b_config2_full_size_vs_oracle_float32(sp, oracle):
    """Benchmark configuration 2 at full size: B=8, C=256, 64^2 -> 128^2, d=64, K=5, s=2, forward and backward."""
    B, d, C, H, W, K, s = 8, 64, 256, 64, 64, 5, 2
    g = torch.Generator().manual_seed(0)
    q = torch.randn(B, d, s * H, s * W, generator=g)
    k = torch.randn(B, d, H, W, generator=g)
    v = torch.randn(B, C, H, W, generator=g)
    go = torch.randn(B, C, s * H, s * W, generator=g)
    want = oracle.sapa_forward(q.numpy(), k.numpy(), v.numpy(), K, s)             # float32 oracle (seconds)
    wq, wk, wv = oracle.sapa_backward(go.numpy(), q.numpy(), k.numpy(), v.numpy(), K, s)
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = sp.sapa_fused(qd, kd, vd, K, s)
    assert ran() == ["sapa_tma_fused_f32_kernel<fwd>"]
    assert rel_err(host64(out), want) < 1e-5
    fq, fk, fv = grads(out, (qd, kd, vd), go.to(DEV))
    assert ran() == ["sapa_tma_fused_f32_kernel<bwd>", "sapa_gath_mma_kernel", "sapa_gath_mma_kernel"]
    assert rel_err(host64(fq), wq) < 2e-5 and rel_err(host64(fk), wk) < 2e-5 and rel_err(host64(fv), wv) < 2e-5
    # size-independent properties
    sep = sp.av(torch.softmax(sp.qk(qd.detach(), kd.detach(), K, s), dim=1), vd.detach(), K, s)
    assert rel_err(host64(sep), host64(out)) < 1e-5                                # fused == separate
    one = sp.sapa_fused(qd[3:4].detach().contiguous(), kd[3:4].detach().contiguous(), vd[3:4].detach().contiguous(), K, s)
    assert torch.equal(one[0], out[3].detach())                                    # images are independent, bit-exact
    v2 = torch.randn(B, C, H, W, generator=g).to(DEV)
    lin = sp.sapa_fused(qd.detach(), kd.detach(), (0.5 * vd.detach() - 2.0 * v2).contiguous(), K, s)
    ref = 0.5 * out.detach() - 2.0 * sp.sapa_fused(qd.detach(), kd.detach(), v2, K, s)
    assert rel_err(host64(lin), host64(ref)) < 1e-5                                # linear in the value
    fq2, fk2, fv2 = grads(sp.sapa_fused(qd, kd, vd, K, s), (qd, kd, vd), go.to(DEV))
    assert torch.equal(fq, fq2) and torch.equal(fk, fk2) and torch.equal(fv, fv2)  # deterministic backward


def test_row_slab_equals_unsharded_rows_bit_exact(sp):
    from sapa_b200.functions import fused_forward_raw
    B, d, C, H, W, K, s = 2, 16, 32, 24, 40, 5, 2
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(*sh, generator=g).to(DEV) for sh in ((B, d, s * H, s * W), (B, d, H, W), (B, C, H, W)))
    full, _ = fused_forward_raw(q, k, v, K, s, False)
    r = 2
    kp, vp = (torch.nn.functional.pad(t, (0, 0, r, r)) for t in (k, v))
    for a, b in ((0, 8), (8, 20), (20, 24)):
        slab, _ = fused_forward_raw(q[:, :, s * a:s * b].contiguous(), kp[:, :, a:b + 2 * r].contiguous(),
                                    vp[:, :, a:b + 2 * r].contiguous(), K, s, False, halo=(r, r))
        assert torch.equal(slab, full[:, :, s * a:s * b])


# ------------------------------------------------------------------ SAPA-D seeded and full size

@pytest.mark.parametrize("cfg", [(2, 16, 32, 9, 11, 9, 4, 0.5), (1, 8, 8, 5, 40, 5, 2, 2.0), (1, 64, 64, 6, 6, 16, 4, 1.0)])
def test_sapa_d_seeded_vs_oracle(sp, oracle, cfg):
    B, Cq, C, H, W, P, G, sigma = cfg
    s = 2
    g = torch.Generator().manual_seed(99 + P)
    q = torch.randn(B, Cq, s * H, s * W, generator=g)
    k = torch.randn(B, Cq, H, W, generator=g)
    v = torch.randn(B, C, H, W, generator=g)
    off = torch.randn(B, G * P * 2, s * H, s * W, generator=g) * sigma
    go = torch.randn(B, C, s * H, s * W, generator=g)
    n = [t.double().numpy() for t in (q, k, v, off)]
    want = oracle.deform_sapa_forward(*n, P, s, G)
    wq, wk, wv, wo = oracle.deform_sapa_backward(go.double().numpy(), *n, P, s, G)
    t = [x.to(DEV).requires_grad_() for x in (q, k, v, off)]
    out = sp.deform_sapa_fused(*t, P, s, G)
    assert rel_err(host64(out), want) < 1e-5
    got = grads(out, t, go.to(DEV))
    for a, b in zip(got, (wq, wk, wv, wo)):
        assert rel_err(host64(a), b) < 2e-5
    sep = sp.deform_av(torch.softmax(sp.deform_qk(t[0], t[1], t[3], P, s, G), dim=2), t[2], t[3], P, s, G)
    assert rel_err(host64(sep), want) < 1e-5
    got = grads(sep, t, go.to(DEV))
    for a, b in zip(got, (wq, wk, wv, wo)):
        assert rel_err(host64(a), b) < 2e-5


def test_sapa_d_config3_full_size_properties(sp, oracle):
    """Benchmark configuration 3 at full size (q/k channels 64 = 16 per group): fused == separate, a 1-image slice of
    the batch against the oracle, and linearity in the value."""
    B, Cq, C, H, W, P, G, s = 8, 64, 256, 64, 64, 9, 4, 2
    g = torch.Generator().manual_seed(3)
    q = torch.randn(B, Cq, s * H, s * W, generator=g).to(DEV)
    k = torch.randn(B, Cq, H, W, generator=g).to(DEV)
    v = torch.randn(B, C, H, W, generator=g).to(DEV)
    off = (torch.randn(B, G * P * 2, s * H, s * W, generator=g) * 0.5).to(DEV)
    out = sp.deform_sapa_fused(q, k, v, off, P, s, G)
    sep = sp.deform_av(torch.softmax(sp.deform_qk(q, k, off, P, s, G), dim=2), v, off, P, s, G)
    assert rel_err(host64(sep), host64(out)) < 1e-5
    want = oracle.deform_sapa_forward(*(t[5:6].cpu().numpy() for t in (q, k, v, off)), P, s, G)
    assert rel_err(host64(out[5:6]), want) < 1e-5
    v2 = torch.randn(B, C, H, W, generator=g).to(DEV)
    lin = sp.deform_sapa_fused(q, k, (v + 3.0 * v2).contiguous(), off, P, s, G)
    assert rel_err(host64(lin), host64(out + 3.0 * sp.deform_sapa_fused(q, k, v2, off, P, s, G))) < 1e-5


# ------------------------------------------------------------------ against the reference's compiled kernels

def _reference_extensions():
    path = os.path.join(ROOT, "oracle", "_ref")
    if not all(os.path.exists(os.path.join(path, n + ".so")) for n in ("qk_ext", "av_ext", "dqk", "dav")):
        return None
    if path not in sys.path:
        sys.path.append(path)      # appended: the stand-ins of sapa_b200.compat are never shadowed by accident
    import importlib
    return tuple(importlib.import_module(n) for n in ("qk_ext", "av_ext", "dqk", "dav"))


def test_against_reference_cuda_extensions_float32(sp):
    """Same seeded float32 inputs through the reference's own kernels and through this library.
    The reference's float32 backward sums in atomic order, so its own distance to its float64 run sets
    the bar where that is larger than 1e-5."""
    ref = _reference_extensions()
    if ref is None:
        pytest.skip("oracle/_ref is not built (python oracle/build_ref.py)")
    qk_ext, av_ext, dqk, dav = ref
    B, d, C, H, W, K, s = 2, 32, 64, 24, 40, 5, 2
    g = torch.Generator().manual_seed(11)
    q, k, v = (torch.randn(*sh, generator=g).to(DEV) for sh in ((B, d, s * H, s * W), (B, d, H, W), (B, C, H, W)))
    attn = torch.softmax(torch.randn(B, K * K, s * H, s * W, generator=g).to(DEV), dim=1)
    gs = torch.randn(B, K * K, s * H, s * W, generator=g).to(DEV)
    go = torch.randn(B, C, s * H, s * W, generator=g).to(DEV)

    def ref_run(dt):
        qq, kk, vv, aa, gss, goo = (t.to(dt) for t in (q, k, v, attn, gs, go))
        sim = torch.zeros(B, K * K, s * H, s * W, device=DEV, dtype=dt)
        qk_ext.forward(kk, qq, K, s, sim)
        gq, gk = torch.zeros_like(qq), torch.zeros_like(kk)
        qk_ext.backward(gss, kk, qq, K, s, gk, gq)
        agg = torch.zeros(B, C, s * H, s * W, device=DEV, dtype=dt)
        av_ext.forward(vv, aa, K, s, agg)
        ga, gv = torch.zeros_like(aa), torch.zeros_like(vv)
        av_ext.backward(goo, vv, aa, K, s, gv, ga)
        torch.cuda.synchronize()
        return dict(sim=sim, gq=gq, gk=gk, agg=agg, ga=ga, gv=gv)

    r32, r64 = ref_run(torch.float32), ref_run(torch.float64)
    qd, kd, vd, ad = (t.clone().requires_grad_() for t in (q, k, v, attn))
    sim = sp.qk(qd, kd, K, s)
    gq, gk = grads(sim, (qd, kd), gs)
    agg = sp.av(ad, vd, K, s)
    ga, gv = grads(agg, (ad, vd), go)
    mine = dict(sim=sim, gq=gq, gk=gk, agg=agg, ga=ga, gv=gv)
    for key in mine:
        bar = max(1e-5, 2 * rel_err(host64(r32[key]), host64(r64[key])))
        assert rel_err(host64(mine[key]), host64(r64[key])) < bar, key

    # deformable pair
    P, G = 9, 4
    off = (torch.randn(B, G * P * 2, s * H, s * W, generator=g) * 0.7).to(DEV)
    dattn = torch.softmax(torch.randn(B, G, P, s * H, s * W, generator=g).to(DEV), dim=2)
    gds = torch.randn(B, G, P, s * H, s * W, generator=g).to(DEV)

    def ref_deform(dt):
        qq, kk, vv, oo, aa, gss, goo = (t.to(dt) for t in (q, k, v, off, dattn, gds, go))
        sim = torch.zeros(B, G, P, s * H, s * W, device=DEV, dtype=dt)
        dqk.forward(qq, kk, oo, P, s, G, sim)
        gq, gk, go1 = torch.zeros_like(qq), torch.zeros_like(kk), torch.zeros_like(oo)
        dqk.backward(gss, qq, kk, oo, P, s, G, gq, gk, go1)
        agg = torch.zeros(B, C, s * H, s * W, device=DEV, dtype=dt)
        dav.forward(aa, vv, oo, P, s, G, agg)
        ga, gv, go2 = torch.zeros_like(aa), torch.zeros_like(vv), torch.zeros_like(oo)
        dav.backward(goo, aa, vv, oo, P, s, G, ga, gv, go2)
        torch.cuda.synchronize()
        return dict(sim=sim, gq=gq, gk=gk, go1=go1, agg=agg, ga=ga, gv=gv, go2=go2)

    r32, r64 = ref_deform(torch.float32), ref_deform(torch.float64)
    qd, kd, vd, od, ad = (t.clone().requires_grad_() for t in (q, k, v, off, dattn))
    sim = sp.deform_qk(qd, kd, od, P, s, G)
    gq, gk, go1 = grads(sim, (qd, kd, od), gds)
    agg = sp.deform_av(ad, vd, od, P, s, G)
    ga, gv, go2 = grads(agg, (ad, vd, od), go)
    mine = dict(sim=sim, gq=gq, gk=gk, go1=go1, agg=agg, ga=ga, gv=gv, go2=go2)
    for key in mine:
        bar = max(1e-5, 2 * rel_err(host64(r32[key]), host64(r64[key])))
        assert rel_err(host64(mine[key]), host64(r64[key])) < bar, key


# ------------------------------------------------------------------ reference check scripts, re-run on this library

def test_gradcheck_float64_like_the_reference_scripts(sp):
    """sapa/sapa/grad_check.py:8-33 and deformsapa/deformsapa/grad_check.py:8-35: b=2, c=16, 3x4, float64."""
    from torch.autograd import gradcheck
    torch.manual_seed(0)
    b, h, w, c, K, s = 2, 3, 4, 16, 5, 2
    q = torch.rand(b, c, s * h, s * w, device=DEV, dtype=torch.float64, requires_grad=True)
    k = torch.rand(b, c, h, w, device=DEV, dtype=torch.float64, requires_grad=True)
    assert gradcheck(sp.qk, (q, k, K, s))
    a = torch.randn(b, K * K, s * h, s * w, device=DEV, dtype=torch.float64, requires_grad=True)
    v = torch.randn(b, c, h, w, device=DEV, dtype=torch.float64, requires_grad=True)
    assert gradcheck(sp.av, (a, v, K, s), eps=1e-4)
    assert gradcheck(sp.sapa_fused, (q, k, v, K, s))
    P, G = 5, 4
    o = torch.rand(b, G * P * 2, s * h, s * w, device=DEV, dtype=torch.float64, requires_grad=True)
    # key / value gradients are scattered with float atomics (as in the reference): summation order varies
    assert gradcheck(sp.deform_qk, (q, k, o, P, s, G), nondet_tol=1e-10)
    da = torch.randn(b, G, P, s * h, s * w, device=DEV, dtype=torch.float64, requires_grad=True)
    assert gradcheck(sp.deform_av, (da, v, o, P, s, G), nondet_tol=1e-10)


def test_forward_check_like_the_reference_scripts(sp):
    """sapa/sapa/forward_check.py:27-47 with this repo's restatement of its PyTorch formulas, atol 1e-5."""
    from oracle import unfold_port as up
    torch.manual_seed(0)
    b, h, w, c, K, s = 4, 10, 12, 8, 5, 2
    q, k = torch.randn(b, c, s * h, s * w, device=DEV), torch.randn(b, c, h, w, device=DEV)
    assert torch.allclose(up.sim(q, k, K, s), sp.qk(q, k, K, s), atol=1e-5)
    a, v = torch.randn(b, K * K, s * h, s * w, device=DEV), torch.randn(b, c, h, w, device=DEV)
    assert torch.allclose(up.atn(a, v, K, s), sp.av(a, v, K, s), atol=1e-5)
    P, G = 5, 4
    o = torch.randn(b, G * P * 2, s * h, s * w, device=DEV)
    assert torch.allclose(up.deform_sim(q, k, o, P, s, G), sp.deform_qk(q, k, o, P, s, G), atol=1e-5)
    da = torch.randn(b, G, P, s * h, s * w, device=DEV)
    assert torch.allclose(up.deform_atn(da, v, o, P, s, G), sp.deform_av(da, v, o, P, s, G), atol=1e-5)


# ------------------------------------------------------------------ modules and error behaviour on the GPU

def test_modules_fused_equals_separate_and_train(sp):
    torch.manual_seed(0)
    x = torch.randn(2, 64, 4, 6, device=DEV)
    y = torch.randn(2, 64, 8, 12, device=DEV)
    m = sp.SAPA(64).to(DEV)
    out = m(y, x)
    assert out.shape == (2, 64, 8, 12)
    m.impl = "separate"
    assert rel_err(host64(m(y, x)), host64(out)) < 1e-5
    m.impl = "fused"
    out.sum().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in m.parameters())
    xd, yd = torch.randn(2, 16, 4, 6, device=DEV), torch.randn(2, 16, 8, 12, device=DEV)
    md = sp.SAPADeform(16).to(DEV)
    torch.nn.init.normal_(md.offset.weight, std=0.5)
    outd = md(yd, xd)
    assert outd.shape == (2, 16, 8, 12)
    md.impl = "separate"
    assert rel_err(host64(md(yd, xd)), host64(outd)) < 1e-5
    md.impl = "fused"
    outd.square().mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in md.parameters())
    low = sp.SAPADeform(16, high_offset=False, norm=False).to(DEV)
    assert low(yd, xd).shape == (2, 16, 8, 12)


def test_error_behaviour_on_cuda_tensors(sp):
    q = torch.randn(1, 4, 8, 8, device=DEV)
    k = torch.randn(1, 4, 4, 4, device=DEV)
    with pytest.raises(RuntimeError, match="contiguous"):
        sp.qk(q.transpose(2, 3), k, 5, 2)
    with pytest.raises(RuntimeError, match="dtype"):
        sp.qk(q.half(), k, 5, 2)
    with pytest.raises(AssertionError):
        sp.qk(q, k, 5, 1)
    from sapa_b200 import _lib
    out = torch.empty(1, 49, 8, 8, device=DEV)
    with pytest.raises(RuntimeError, match="UNSUPPORTED|no fused kernel"):
        _lib.call("sapa_fused_forward", q.device, q, k, k, out, None, 1, 4, 4, 4, 4, 7, 2, 0)
    # K = 7 still works through the public op (separate kernels behind the same function)
    v = torch.randn(1, 3, 4, 4, device=DEV)
    assert sp.sapa_fused(q, k, v, 7, 2).shape == (1, 3, 8, 8)


def test_config4_decoder_pyramid_bf16_forward(sp):
    """Benchmark configuration 4 (stand-in wiring, random init): encoder features of 64/128/320/512 channels at
    128^2/64^2/32^2/16^2 are projected to 256 channels and upsampled 16^2 -> 32^2 -> 64^2 -> 128^2 by three
    chained SAPA modules (d=32, K=5), bf16, forward only.  Checked against the same modules in float32 on the
    separate-op path (1e-2 of the output range; batch 2 instead of 16 keeps the test small)."""
    torch.manual_seed(0)
    B = 2
    feats = [torch.randn(B, c, r, r, device=DEV) for c, r in ((64, 128), (128, 64), (320, 32), (512, 16))]
    proj = [torch.nn.Conv2d(c, 256, 1).to(DEV) for c in (64, 128, 320, 512)]
    ups = [sp.SAPA(256, embedding_dim=32).to(DEV) for _ in range(3)]

    def run(dtype, impl):
        with torch.no_grad():
            ys = [p.to(dtype)(f.to(dtype)) for p, f in zip(proj, feats)]
            x = ys[3]
            for level, m in zip((2, 1, 0), ups):
                m.impl = impl
                x = m.to(dtype)(ys[level], x)
            return x

    want = run(torch.float32, "separate")
    fused32 = run(torch.float32, "fused")
    got = run(torch.bfloat16, "fused")           # last: .to(bfloat16) rounds the modules' weights in place
    assert got.shape == (B, 256, 128, 128) and got.dtype == torch.bfloat16
    assert rel_err(host64(got), host64(want)) < 2e-2
    assert rel_err(host64(fused32), host64(want)) < 1e-5


def test_modules_under_autocast(sp):
    """Inside torch.autocast the projections are bfloat16 and the value float32: the modules cast to the autocast
    type and give the bfloat16 result (the reference modules have no autocast handling)."""
    torch.manual_seed(3)
    y, x = torch.randn(2, 64, 24, 32, device=DEV), torch.randn(2, 64, 12, 16, device=DEV)
    for m in (sp.SAPA(64, embedding_dim=16).to(DEV), sp.SAPADeform(64, embedding_dim=8).to(DEV)):
        with torch.no_grad():
            want = m(y, x)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                got = m(y, x)
        assert got.dtype == torch.bfloat16 and got.shape == want.shape
        assert rel_err(host64(got), host64(want)) < 3e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_forward_and_backward_replay_from_a_cuda_graph(sp, dtype):
    """The entry points neither synchronise nor allocate, so a stream capture of forward + backward replays to the
    same bits as the eager calls (new inputs are written into the captured buffers between replays)."""
    from sapa_b200 import _lib
    B, d, C, H, W, K, s = 2, 32, 48, 12, 24, 5, 2
    g = torch.Generator().manual_seed(11)
    mk = lambda *sh: torch.randn(*sh, generator=g).to(DEV, dtype)
    q, k, v, go = mk(B, d, s * H, s * W), mk(B, d, H, W), mk(B, C, H, W), mk(B, C, s * H, s * W)
    out, attn = torch.empty_like(go), torch.empty(B, K * K, s * H, s * W, device=DEV, dtype=dtype)
    gq, gk, gv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    code = _lib.dtype_code(q)
    nb = _lib.fused_backward_workspace(B, H, W, K, s, code)
    ws = torch.empty(nb, dtype=torch.uint8, device=DEV)

    def run():
        _lib.call("sapa_fused_forward", DEV, q, k, v, out, attn, B, d, C, H, W, K, s, code)
        _lib.call("sapa_fused_backward", DEV, go, q, k, v, attn, gq, gk, gv, ws, nb, B, d, C, H, W, K, s, code)

    run()                                   # warm-up outside the capture (tensor-map encoder lookup, function attributes)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            run()
    for seed in (21, 22):
        g2 = torch.Generator().manual_seed(seed)
        for t in (q, k, v, go):
            t.copy_(torch.randn(*t.shape, generator=g2).to(DEV, dtype))
        graph.replay()
        torch.cuda.synchronize()
        got = [t.clone() for t in (out, gq, gk, gv)]
        run()
        torch.cuda.synchronize()
        for a, b in zip(got, (out, gq, gk, gv)):
            assert torch.equal(a, b)


def test_no_barrier_wait_gave_up(sp):
    """Runs after the other tests of this file: every bounded mbarrier wait of the TMA kernels completed."""
    from sapa_b200 import _lib
    assert _lib.wait_timeout_flags(DEV) == 0
