"""The callers either side of the kernels, on the GPU: the ``SAPA`` / ``SAPADeform`` modules against golden outputs of
the REFERENCE's own module classes evaluated on the same ``state_dict`` (tests/golden/make_golden.py modules), the
import-compatible extension shims called with the reference's positional argument orders, and - where a reference
checkout is present next to a GPU - the reference's check scripts run unmodified on top of those shims."""
import importlib
import os
import runpy
import sys

import numpy as np
import pytest
import torch

from conftest import GOLDEN, ROOT, rel_err

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


MODULE_CASES = sorted(f[len("pyref_"):-4] for f in os.listdir(GOLDEN) if f.startswith("pyref_mod_"))


@pytest.mark.parametrize("impl", ["fused", "separate"])
@pytest.mark.parametrize("name", MODULE_CASES)
def test_modules_match_the_reference_modules_on_the_same_state_dict(sp, name, impl, monkeypatch):
    """sapa_base.py:26-40 / sapa_deform.py:34-53: GroupNorm, 1x1 projections, (offset conv + pixel_shuffle or nearest
    interpolation), attention.  float32 on the GPU against the reference classes in float64: 2e-5 of the output range
    (GroupNorm and the convolutions are torch float32 kernels)."""
    f = np.load(os.path.join(GOLDEN, f"pyref_{name}.npz"))
    # the 1x1 projections are torch convolutions: cuDNN would run them in TF32 by default (1e-3), which is not what is
    # being compared here
    monkeypatch.setattr(torch.backends.cudnn, "allow_tf32", False)
    monkeypatch.setattr(torch.backends.cuda.matmul, "allow_tf32", False)
    kwargs = {k[3:]: f[k].item() for k in f.files if k.startswith("kw_")}
    cls = getattr(sp, str(f["meta_class"]))
    mod = cls(**kwargs, impl=impl).to(DEV)
    state = {k[3:]: torch.from_numpy(f[k]) for k in f.files if k.startswith("sd_")}
    assert sorted(state) == sorted(mod.state_dict())          # same parameter names as the reference module
    mod.load_state_dict(state)
    x = torch.from_numpy(f["in_x"]).to(DEV).requires_grad_()
    y = torch.from_numpy(f["in_y"]).to(DEV).requires_grad_()
    out = mod(y, x)
    assert rel_err(host64(out), f["out_out"]) < 2e-5
    gx, gy = torch.autograd.grad(out, (x, y), torch.from_numpy(f["in_grad_out"]).to(DEV))
    assert rel_err(host64(gx), f["out_dx"]) < 5e-5
    assert rel_err(host64(gy), f["out_dy"]) < 5e-5


@pytest.fixture()
def compat(sp):
    sys.path.insert(0, sp.compat_path())
    saved = {n: sys.modules.pop(n, None) for n in ("qk_ext", "av_ext", "dqk", "dav", "sapa", "deformsapa")}
    try:
        yield {n: importlib.import_module(n) for n in ("qk_ext", "av_ext", "dqk", "dav")}
    finally:
        sys.path.remove(sp.compat_path())
        for n, m in saved.items():
            sys.modules.pop(n, None)
            if m is not None:
                sys.modules[n] = m


def test_extension_shims_with_the_reference_positional_orders(sp, compat, oracle):
    """qk_ext.forward(key, query, K, s, out), qk_ext.backward(dS, key, query, K, s, grad_key, grad_query),
    av_ext.forward(value, attn, K, s, out), av_ext.backward(dOut, value, attn, K, s, grad_value, grad_attn)
    (sapa/sapa/sapa_func.py:26, 44-46, 71, 89-91) and the dqk / dav equivalents (deform_func.py): outputs are written
    in place into caller-allocated (here: pre-zeroed, as the reference does) buffers."""
    B, d, C, H, W, K, s = 2, 12, 20, 7, 12, 5, 2
    g = torch.Generator().manual_seed(31)
    mk = lambda *sh: torch.randn(*sh, generator=g)
    q, k, v, a = mk(B, d, s * H, s * W), mk(B, d, H, W), mk(B, C, H, W), mk(B, K * K, s * H, s * W)
    gs, go = mk(B, K * K, s * H, s * W), mk(B, C, s * H, s * W)
    n = {name: t.double().numpy() for name, t in dict(q=q, k=k, v=v, a=a, gs=gs, go=go).items()}
    qd, kd, vd, ad, gsd, god = (t.to(DEV) for t in (q, k, v, a, gs, go))
    sim = torch.zeros(B, K * K, s * H, s * W, device=DEV)
    assert compat["qk_ext"].forward(kd, qd, K, s, sim) == 1
    assert rel_err(host64(sim), oracle.qk_forward(n["q"], n["k"], K, s)) < 1e-5
    gk, gq = torch.zeros_like(kd), torch.zeros_like(qd)
    compat["qk_ext"].backward(gsd, kd, qd, K, s, gk, gq)
    wq, wk = oracle.qk_backward(n["gs"], n["q"], n["k"], K, s)
    assert rel_err(host64(gq), wq) < 1e-5 and rel_err(host64(gk), wk) < 1e-5
    out = torch.zeros(B, C, s * H, s * W, device=DEV)
    assert compat["av_ext"].forward(vd, ad, K, s, out) == 1
    assert rel_err(host64(out), oracle.av_forward(n["a"], n["v"], K, s)) < 1e-5
    gv, ga = torch.zeros_like(vd), torch.zeros_like(ad)
    compat["av_ext"].backward(god, vd, ad, K, s, gv, ga)
    wa, wv = oracle.av_backward(n["go"], n["a"], n["v"], K, s)
    assert rel_err(host64(ga), wa) < 1e-5 and rel_err(host64(gv), wv) < 1e-5
    # deformable pair
    P, G = 5, 4
    off, da, gds = mk(B, G * P * 2, s * H, s * W) * 0.7, mk(B, G, P, s * H, s * W), mk(B, G, P, s * H, s * W)
    no, nda, ngds = (t.double().numpy() for t in (off, da, gds))
    od, dad, gdsd = off.to(DEV), da.to(DEV), gds.to(DEV)
    dsim = torch.zeros(B, G, P, s * H, s * W, device=DEV)
    assert compat["dqk"].forward(qd, kd, od, P, s, G, dsim) == 1
    assert rel_err(host64(dsim), oracle.deform_qk_forward(n["q"], n["k"], no, P, s, G)) < 1e-5
    gq, gk, go1 = torch.zeros_like(qd), torch.zeros_like(kd), torch.zeros_like(od)
    compat["dqk"].backward(gdsd, qd, kd, od, P, s, G, gq, gk, go1)
    wq, wk, wo = oracle.deform_qk_backward(ngds, n["q"], n["k"], no, P, s, G)
    assert rel_err(host64(gq), wq) < 1e-5 and rel_err(host64(gk), wk) < 1e-5 and rel_err(host64(go1), wo) < 1e-5
    dout = torch.zeros(B, C, s * H, s * W, device=DEV)
    assert compat["dav"].forward(dad, vd, od, P, s, G, dout) == 1
    assert rel_err(host64(dout), oracle.deform_av_forward(nda, n["v"], no, P, s, G)) < 1e-5
    ga, gv, go2 = torch.zeros_like(dad), torch.zeros_like(vd), torch.zeros_like(od)
    compat["dav"].backward(god, dad, vd, od, P, s, G, ga, gv, go2)
    wa, wv, wo = oracle.deform_av_backward(n["go"], nda, n["v"], no, P, s, G)
    assert rel_err(host64(ga), wa) < 1e-5 and rel_err(host64(gv), wv) < 1e-5 and rel_err(host64(go2), wo) < 1e-5


REFERENCE = os.environ.get("SAPA_REFERENCE", "")
CHECK_SCRIPTS = ["sapa/sapa/forward_check.py", "sapa/sapa/grad_check.py",
                 "deformsapa/deformsapa/forward_check.py", "deformsapa/deformsapa/grad_check.py"]


@pytest.mark.parametrize("script", CHECK_SCRIPTS)
def test_reference_check_scripts_run_unmodified_on_the_shims(sp, compat, script, capsys):
    """The reference's own four check scripts, executed as they are (``__main__``), with ``qk_ext`` / ``av_ext`` /
    ``dqk`` / ``dav`` resolving to this library's shims.  Needs a checkout of the reference (SAPA_REFERENCE) on the
    machine that has the GPU; skipped otherwise."""
    path = os.path.join(REFERENCE, script)
    if not REFERENCE or not os.path.exists(path):
        pytest.skip("no reference checkout on this machine (set SAPA_REFERENCE)")
    here = os.path.dirname(path)
    sys.path.insert(1, here)                   # the scripts import sapa_func / deform_func from their own folder
    for m in ("sapa_func", "deform_func"):
        sys.modules.pop(m, None)
    try:
        runpy.run_path(path, run_name="__main__")
    finally:
        sys.path.remove(here)
        for m in ("sapa_func", "deform_func"):
            sys.modules.pop(m, None)
    printed = capsys.readouterr().out
    assert "False" not in printed            # forward_check prints allclose results, grad_check prints gradcheck results
