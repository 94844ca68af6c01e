"""Generate the golden vectors of ``tests/golden/*.npz`` from the REFERENCE's own code.

Three producers, all running reference code only (nothing from this repository's kernels or oracle):

``python tests/golden/make_golden.py cpu  [--reference /path/to/sapa]``
    imports the reference's PyTorch check functions (sapa/sapa/forward_check.py:9-24,
    deformsapa/deformsapa/forward_check.py:6-40), evaluates them in float64 on seeded inputs and takes
    gradients by autograd through them.  Runs without a GPU.  Writes ``pyref_<case>.npz``.

``python tests/golden/make_golden.py modules --reference /path/to/sapa``
    instantiates the reference's ``SAPA`` / ``SAPADeform`` modules on the CPU (float64, their attention evaluated with
    the same PyTorch check functions) and stores ``state_dict``, inputs, output and input gradients.  Writes
    ``pyref_mod_<case>.npz``.

``python tests/golden/make_golden.py cuda --out DIR``
    loads ``pyref_<case>.npz`` and feeds the same inputs to the reference's compiled CUDA extensions
    (``oracle/_ref/*.so`` built by ``oracle/build_ref.py``; positional conventions of sapa_func.py:26,44-46,
    71,89-91 and deform_func.py:29,50-52,84,105-107) in float64 and float32 on a GPU.  Writes
    ``cudaref_<case>.npz`` into DIR.  Needs no reference checkout, only the built extensions.

Inputs are drawn in float32 and stored as float32, so float32 kernels see bit-identical inputs; the
expected outputs are float64.  The reference has no stored vectors or seeds of its own
(its checks draw unseeded ``randn``), so these files are the pin.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))

# name -> dict(B, d (q/k channels), C (value channels), H, W, K, s)
SAPA_B_CASES = {
    "b_fwdcheck": dict(B=2, d=8, C=8, H=10, W=12, K=5, s=2),     # shapes of sapa/sapa/forward_check.py:27-47 (b halved)
    "b_gradcheck": dict(B=2, d=16, C=16, H=3, W=4, K=5, s=2),    # shapes of sapa/sapa/grad_check.py:8-33
    "b_k3s1": dict(B=1, d=5, C=3, H=6, W=5, K=3, s=1),
    "b_k7s2": dict(B=1, d=4, C=6, H=5, W=9, K=7, s=2),
    "b_k5s4": dict(B=2, d=3, C=5, H=4, W=3, K=5, s=4),
    "b_k1s2": dict(B=1, d=4, C=4, H=3, W=3, K=1, s=2),
    "b_wide": dict(B=1, d=6, C=10, H=5, W=21, K=5, s=2),         # W not a multiple of any vector width
}
# name -> dict(B, Cq, C, H, W, P, s, G, sigma of offsets)
SAPA_D_CASES = {
    "d_fwdcheck": dict(B=1, Cq=8, C=8, H=10, W=12, P=5, s=2, G=4, sigma=1.0),   # deformsapa forward_check.py:43-65 (b=1)
    "d_gradcheck": dict(B=2, Cq=16, C=16, H=3, W=4, P=5, s=2, G=4, sigma=0.5),  # deformsapa grad_check.py:8-35
    "d_p9g4": dict(B=1, Cq=16, C=32, H=6, W=7, P=9, s=2, G=4, sigma=0.5),
    "d_far": dict(B=1, Cq=4, C=8, H=5, W=6, P=3, s=2, G=2, sigma=4.0),          # many samples outside the image
    "d_s1g1": dict(B=1, Cq=3, C=5, H=4, W=5, P=4, s=1, G=1, sigma=1.0),
}
# benchmark configuration 1: the CPU-runnable single-op case (1x1 projections, then SAPA-B attention)
CFG1 = dict(B=1, Cx=64, Cy=64, H=16, W=16, d=32, K=5, s=2)


def _randn(gen, *shape, scale=1.0):
    return (torch.randn(*shape, generator=gen, dtype=torch.float32) * scale)


def sapa_b_inputs(cfg, seed):
    g = torch.Generator().manual_seed(seed)
    B, d, C, H, W, K, s = (cfg[k] for k in "B d C H W K s".split())
    return dict(
        query=_randn(g, B, d, s * H, s * W), key=_randn(g, B, d, H, W), value=_randn(g, B, C, H, W),
        attn=_randn(g, B, K * K, s * H, s * W),          # a free (un-normalised) attention, as in forward_check
        grad_sim=_randn(g, B, K * K, s * H, s * W), grad_out=_randn(g, B, C, s * H, s * W))


def sapa_d_inputs(cfg, seed):
    g = torch.Generator().manual_seed(seed)
    B, Cq, C, H, W, P, s, G = (cfg[k] for k in "B Cq C H W P s G".split())
    return dict(
        query=_randn(g, B, Cq, s * H, s * W), key=_randn(g, B, Cq, H, W), value=_randn(g, B, C, H, W),
        offset=_randn(g, B, G * P * 2, s * H, s * W, scale=cfg["sigma"]),
        attn=_randn(g, B, G, P, s * H, s * W),
        grad_sim=_randn(g, B, G, P, s * H, s * W), grad_out=_randn(g, B, C, s * H, s * W))


def _np(d):
    return {k: v.detach().cpu().numpy() for k, v in d.items()}


def _save(path, meta, inputs, outputs):
    arrs = {"in_" + k: v for k, v in _np(inputs).items()}
    arrs.update({"out_" + k: v for k, v in _np(outputs).items()})
    arrs.update({"meta_" + k: np.asarray(v) for k, v in meta.items()})
    np.savez_compressed(path, **arrs)


# ------------------------------------------------------------------ producer 1: reference Python (CPU)

def make_cpu(reference: str):
    sys.path.insert(0, HERE)
    import _ref_import
    fb, fd = _ref_import.load(reference)
    for i, (name, cfg) in enumerate(SAPA_B_CASES.items()):
        t = {k: v.double() for k, v in sapa_b_inputs(cfg, 100 + i).items()}
        K, s = cfg["K"], cfg["s"]
        q, k, v, a = (t[n].clone().requires_grad_() for n in ("query", "key", "value", "attn"))
        sim = fb.qk_pytorch(q, k, K, s)
        gq, gk = torch.autograd.grad(sim, (q, k), t["grad_sim"])
        agg = fb.av_pytorch(a, v, K, s)
        ga, gv = torch.autograd.grad(agg, (a, v), t["grad_out"])
        # whole attention: av(softmax(qk), v) as in sapa_base.py:38-40
        q2, k2, v2 = (t[n].clone().requires_grad_() for n in ("query", "key", "value"))
        prob = torch.softmax(fb.qk_pytorch(q2, k2, K, s), dim=1)
        full = fb.av_pytorch(prob, v2, K, s)
        fq, fk, fv = torch.autograd.grad(full, (q2, k2, v2), t["grad_out"])
        _save(os.path.join(HERE, f"pyref_{name}.npz"), cfg, {n: x.float() for n, x in t.items()},
              dict(sim=sim, sim_dquery=gq, sim_dkey=gk, agg=agg, agg_dattn=ga, agg_dvalue=gv,
                   full=full, full_prob=prob, full_dquery=fq, full_dkey=fk, full_dvalue=fv))
        print("wrote", name)
    for i, (name, cfg) in enumerate(SAPA_D_CASES.items()):
        t = {k: v.double() for k, v in sapa_d_inputs(cfg, 200 + i).items()}
        P, s, G = cfg["P"], cfg["s"], cfg["G"]
        q, k, v, a, o = (t[n].clone().requires_grad_() for n in ("query", "key", "value", "attn", "offset"))
        sim = fd.deform_qk_pytorch(q, k, o, P, s, G)
        gq, gk, go1 = torch.autograd.grad(sim, (q, k, o), t["grad_sim"])
        agg = fd.deform_av_pytorch(a, v, o, P, s, G)
        ga, gv, go2 = torch.autograd.grad(agg, (a, v, o), t["grad_out"])
        q2, k2, v2, o2 = (t[n].clone().requires_grad_() for n in ("query", "key", "value", "offset"))
        prob = torch.softmax(fd.deform_qk_pytorch(q2, k2, o2, P, s, G), dim=2)
        full = fd.deform_av_pytorch(prob, v2, o2, P, s, G)
        fq, fk, fv, fo = torch.autograd.grad(full, (q2, k2, v2, o2), t["grad_out"])
        _save(os.path.join(HERE, f"pyref_{name}.npz"), cfg, {n: x.float() for n, x in t.items()},
              dict(sim=sim, sim_dquery=gq, sim_dkey=gk, sim_doffset=go1,
                   agg=agg, agg_dattn=ga, agg_dvalue=gv, agg_doffset=go2,
                   full=full, full_prob=prob, full_dquery=fq, full_dkey=fk, full_dvalue=fv, full_doffset=fo))
        print("wrote", name)
    # config 1: X, Y ~ N(0,1) seed 0; 1x1 projections with N(0, 0.02^2) weights and zero bias (sapa_base.py:42-46)
    c = CFG1
    g = torch.Generator().manual_seed(0)
    X = _randn(g, c["B"], c["Cx"], c["H"], c["W"])
    Y = _randn(g, c["B"], c["Cy"], c["s"] * c["H"], c["s"] * c["W"])
    Wq = _randn(g, c["d"], c["Cy"], scale=0.02)
    Wk = _randn(g, c["d"], c["Cx"], scale=0.02)
    q = torch.einsum("oc,bchw->bohw", Wq.double(), Y.double())
    k = torch.einsum("oc,bchw->bohw", Wk.double(), X.double())
    out = fb.av_pytorch(torch.softmax(fb.qk_pytorch(q, k, c["K"], c["s"]), dim=1), X.double(), c["K"], c["s"])
    _save(os.path.join(HERE, "pyref_cfg1.npz"), c, dict(X=X, Y=Y, Wq=Wq, Wk=Wk), dict(full=out.float()))
    print("wrote cfg1")


# ------------------------------------------------------------------ producer 1b: the reference's nn.Modules (CPU)

# name -> (class, constructor kwargs, low-res size, offset-projection std); dim_y / dim_x are multiples of 32 (GroupNorm(32, .))
MODULE_CASES = {
    "mod_sapa": ("SAPA", dict(dim_y=64, dim_x=96, embedding_dim=16), (2, 6, 8), None),
    "mod_sapa_nonorm": ("SAPA", dict(dim_y=32, embedding_dim=8, norm=False, qkv_bias=False), (1, 5, 12), None),
    "mod_deform": ("SAPADeform", dict(dim_y=32, dim_x=64, embedding_dim=8, norm=True), (2, 6, 8), 0.3),
    "mod_deform_low": ("SAPADeform", dict(dim_y=32, num_point=5, groups=2, embedding_dim=4, high_offset=False), (1, 4, 8), 0.3),
}


def make_modules(reference: str):
    """Instantiates the reference's own ``SAPA`` / ``SAPADeform`` classes (sapa_base.py:7-49, sapa_deform.py:7-62) on
    the CPU in float64, with ``sapa.qk/av`` and ``deformsapa.deform_qk/deform_av`` bound to the reference's PyTorch
    check functions (its CUDA ops need a GPU), and stores state_dict, inputs, output and input gradients (computed in float64, stored as float32)."""
    import importlib.util
    import types
    sys.path.insert(0, HERE)
    import _ref_import
    fb, fd = _ref_import.load(reference)
    stub_b, stub_d = types.ModuleType("sapa"), types.ModuleType("deformsapa")
    stub_b.qk, stub_b.av = fb.qk_pytorch, fb.av_pytorch
    stub_d.deform_qk, stub_d.deform_av = fd.deform_qk_pytorch, fd.deform_av_pytorch
    sys.modules["sapa"], sys.modules["deformsapa"] = stub_b, stub_d
    classes = {}
    for cls, rel in (("SAPA", "sapa_base.py"), ("SAPADeform", "sapa_deform.py")):
        spec = importlib.util.spec_from_file_location("ref_" + cls, os.path.join(reference, rel))
        m = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(m)
        classes[cls] = getattr(m, cls)
    for i, (name, (cls, kwargs, (B, H, W), off_std)) in enumerate(MODULE_CASES.items()):
        torch.manual_seed(300 + i)
        mod = classes[cls](**kwargs)
        g = torch.Generator().manual_seed(400 + i)
        with torch.no_grad():      # make every parameter non-trivial (the default affine GroupNorm is the identity)
            for pname, p in mod.named_parameters():
                if pname.startswith("norm"):
                    p.add_(_randn(g, *p.shape, scale=0.3))
                elif pname.endswith("bias"):
                    p.copy_(_randn(g, *p.shape, scale=0.1))
                elif pname.startswith("offset") and off_std is not None:
                    p.copy_(_randn(g, *p.shape, scale=off_std / (p.shape[1] ** 0.5)))
                else:
                    p.copy_(_randn(g, *p.shape, scale=0.2))
        s = mod.up_factor
        dim_y, dim_x = kwargs["dim_y"], kwargs.get("dim_x") or kwargs["dim_y"]
        x = _randn(g, B, dim_x, H, W)
        y = _randn(g, B, dim_y, s * H, s * W)
        grad_out = _randn(g, B, dim_x, s * H, s * W)
        mod = mod.double()
        xd, yd = x.double().requires_grad_(), y.double().requires_grad_()
        out = mod(yd, xd)
        gx, gy = torch.autograd.grad(out, (xd, yd), grad_out.double())
        arrs = {"sd_" + k: v.detach().float().numpy() for k, v in mod.state_dict().items()}
        arrs.update(in_x=x.numpy(), in_y=y.numpy(), in_grad_out=grad_out.numpy(),
                    out_out=out.detach().float().numpy(), out_dx=gx.float().numpy(), out_dy=gy.float().numpy())
        arrs["meta_class"] = np.asarray(cls)
        arrs.update({"kw_" + k: np.asarray(v) for k, v in kwargs.items()})
        np.savez_compressed(os.path.join(HERE, f"pyref_{name}.npz"), **arrs)
        print("wrote", name)


# ------------------------------------------------------------------ producer 2: reference CUDA extensions (GPU)

def make_cuda(out_dir: str):
    sys.path.insert(0, os.path.join(REPO, "oracle", "_ref"))
    import av_ext
    import dav
    import dqk
    import qk_ext
    os.makedirs(out_dir, exist_ok=True)
    dev = torch.device("cuda:0")

    def z(*shape, like):
        return torch.zeros(*shape, dtype=like.dtype, device=dev)

    for name, cfg in list(SAPA_B_CASES.items()) + list(SAPA_D_CASES.items()):
        f = np.load(os.path.join(HERE, f"pyref_{name}.npz"))
        res = {}
        for tag, dt in (("f64", torch.float64), ("f32", torch.float32)):
            t = {k[3:]: torch.from_numpy(f[k]).to(dev, dt) for k in f.files if k.startswith("in_")}
            s = cfg["s"]
            if name.startswith("b_"):
                K = cfg["K"]
                B, d, Hs, Ws = t["query"].shape
                sim = z(B, K * K, Hs, Ws, like=t["query"])
                qk_ext.forward(t["key"], t["query"], K, s, sim)
                gq, gk = torch.zeros_like(t["query"]), torch.zeros_like(t["key"])
                qk_ext.backward(t["grad_sim"], t["key"], t["query"], K, s, gk, gq)
                agg = z(B, cfg["C"], Hs, Ws, like=t["query"])
                av_ext.forward(t["value"], t["attn"], K, s, agg)
                ga, gv = torch.zeros_like(t["attn"]), torch.zeros_like(t["value"])
                av_ext.backward(t["grad_out"], t["value"], t["attn"], K, s, gv, ga)
                prob = torch.softmax(sim, dim=1)
                full = z(B, cfg["C"], Hs, Ws, like=t["query"])
                av_ext.forward(t["value"], prob, K, s, full)
                r = dict(sim=sim, sim_dquery=gq, sim_dkey=gk, agg=agg, agg_dattn=ga, agg_dvalue=gv,
                         full=full, full_prob=prob)
            else:
                P, G = cfg["P"], cfg["G"]
                B, Cq, Hs, Ws = t["query"].shape
                sim = z(B, G, P, Hs, Ws, like=t["query"])
                dqk.forward(t["query"], t["key"], t["offset"], P, s, G, sim)
                gq, gk, go1 = (torch.zeros_like(t[n]) for n in ("query", "key", "offset"))
                dqk.backward(t["grad_sim"], t["query"], t["key"], t["offset"], P, s, G, gq, gk, go1)
                agg = z(B, cfg["C"], Hs, Ws, like=t["query"])
                dav.forward(t["attn"], t["value"], t["offset"], P, s, G, agg)
                ga, gv, go2 = (torch.zeros_like(t[n]) for n in ("attn", "value", "offset"))
                dav.backward(t["grad_out"], t["attn"], t["value"], t["offset"], P, s, G, ga, gv, go2)
                prob = torch.softmax(sim, dim=2)
                full = z(B, cfg["C"], Hs, Ws, like=t["query"])
                dav.forward(prob, t["value"], t["offset"], P, s, G, full)
                r = dict(sim=sim, sim_dquery=gq, sim_dkey=gk, sim_doffset=go1,
                         agg=agg, agg_dattn=ga, agg_dvalue=gv, agg_doffset=go2, full=full, full_prob=prob)
            torch.cuda.synchronize()
            if tag == "f64":
                res.update({f"f64_{k}": v.cpu().numpy() for k, v in r.items()})
            else:   # float32 run: keep only its distance to the float64 run, max|a-b| / max|b|
                for k, v in r.items():
                    ref = torch.from_numpy(res[f"f64_{k}"]).to(dev)
                    res[f"f32err_{k}"] = np.asarray(
                        ((v.double() - ref).abs().max() / ref.abs().max().clamp_min(1e-30)).item())
        np.savez_compressed(os.path.join(out_dir, f"cudaref_{name}.npz"), **res)
        print("wrote", name)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("which", choices=["cpu", "modules", "cuda"])
    ap.add_argument("--reference", default=os.environ.get("SAPA_REFERENCE"),
                    help="path of a tiny-smart/sapa checkout (or set SAPA_REFERENCE); needed by `cpu` and `modules`")
    ap.add_argument("--out", default=HERE)
    a = ap.parse_args()
    if a.which in ("cpu", "modules") and not a.reference:
        ap.error("--reference (or SAPA_REFERENCE) is required")
    if a.which == "cpu":
        make_cpu(a.reference)
    elif a.which == "modules":
        make_modules(a.reference)
    else:
        make_cuda(a.out)


if __name__ == "__main__":
    main()
