"""GroupNorm + 1x1 projection (``sapa_project_forward``: statistics pass, fold, tcgen05 GEMM) against torch's own
GroupNorm and convolution evaluated in float64 on the same (rounded) inputs and parameters, and the modules' no-grad
path, which uses it, against the goldens made from the reference modules (sapa_base.py:26-40, sapa_deform.py:34-53)."""
import os

import numpy as np
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def sp():
    import sapa_b200
    return sapa_b200


def _case(B, C, H, W, d, groups, dtype, bias=True, mean=0.0, seed=1):
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(B, C, H, W, generator=g) + mean).to(dev).to(dtype)
    norm = nn.GroupNorm(groups, C).to(dev) if groups else None
    conv = nn.Conv2d(C, d, 1, bias=bias).to(dev)
    with torch.no_grad():
        conv.weight.normal_(0, 0.05, generator=None)
        if bias:
            conv.bias.normal_(0, 0.5)
        if norm is not None:
            norm.weight.normal_(1, 0.3)
            norm.bias.normal_(0, 0.3)
    conv = conv.to(dtype)
    norm = norm.to(dtype) if norm is not None else None
    with torch.no_grad():
        ref = x.double()
        if norm is not None:
            ref = F.group_norm(ref, groups, norm.weight.double(), norm.bias.double(), norm.eps)
        ref = F.conv2d(ref, conv.weight.double(), conv.bias.double() if bias else None)
    return x, norm, conv, ref


SHAPES = [
    # B, C, H, W, d, groups, bias, mean
    (2, 64, 8, 16, 32, 32, True, 0.0),        # one 128-pixel tile per image
    (2, 64, 8, 16, 32, 0, True, 0.0),         # norm=False
    (2, 96, 9, 12, 48, 32, False, 0.0),       # ragged tile (108 pixels), channel tail (96 = 3 x 32), no bias
    (3, 320, 20, 20, 32, 32, True, 3.0),      # several tiles per image + a tail, non-zero group means
    (1, 32, 2, 2, 16, 32, True, 0.0),         # four pixels, one channel per group
    (2, 128, 24, 24, 256, 32, True, 0.0),     # widest accumulator (all 512 TMEM columns, two stages)
    (5, 256, 32, 32, 64, 32, True, 0.0),      # more tiles than one wave of the smaller grids
]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2), (torch.float16, 2e-3)])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "B%d_C%d_%dx%d_d%d_g%d" % s[:6])
def test_projection_matches_groupnorm_plus_conv(sp, shape, dtype, tol):
    from sapa_b200 import _lib
    from sapa_b200.projection import project, project_supported
    B, C, H, W, d, groups, bias, mean = shape
    x, norm, conv, ref = _case(B, C, H, W, d, groups, dtype, bias, mean)
    if (H * W * x.element_size()) % 16 != 0:          # a pixel row of the tensor map must be a multiple of 16 bytes
        assert not project_supported(x, norm, conv)
        return
    assert project_supported(x, norm, conv)
    out = project(x, norm, conv)
    torch.cuda.synchronize()
    kernels = _lib.last_kernels()
    assert kernels[-1] == "sapa_proj_umma_kernel" and kernels[-2] == "gn_fold_kernel"
    assert ("gn_partial_kernel" in kernels) == bool(groups)
    err = float((out.double() - ref).abs().max() / ref.abs().max())
    assert err < tol, err
    assert _lib.wait_timeout_flags(x.device) == 0


def test_projection_full_size_and_determinism(sp):
    """The q projection of BASELINE config 2 (B=8, C=256 -> d=64 at 128 x 128): float32 accuracy, run twice bit-equal."""
    from sapa_b200.projection import project
    x, norm, conv, ref = _case(8, 256, 128, 128, 64, 32, torch.float32)
    a = project(x, norm, conv)
    b = project(x, norm, conv)
    assert torch.equal(a, b)
    assert float((a.double() - ref).abs().max() / ref.abs().max()) < 1e-5


def test_projection_refuses_what_the_kernel_cannot_take(sp):
    from sapa_b200.projection import project, project_supported
    dev = torch.device("cuda:0")
    conv = nn.Conv2d(64, 8, 1).to(dev)                     # d = 8 is not a multiple of 16
    x = torch.randn(1, 64, 4, 4, device=dev)
    assert not project_supported(x, None, conv)
    with pytest.raises(NotImplementedError):
        project(x, None, conv)
    assert not project_supported(torch.randn(1, 64, 3, 3, device=dev), None, nn.Conv2d(64, 16, 1).to(dev))     # 9 pixels: rows of 36 bytes
    assert not project_supported(x.double(), None, nn.Conv2d(64, 16, 1).to(dev).double())
    assert not project_supported(x, None, nn.Conv2d(64, 16, 3, padding=1).to(dev))


MODULE_CASES = sorted(f[len("pyref_"):-4] for f in os.listdir(GOLDEN) if f.startswith("pyref_mod_"))


@pytest.mark.parametrize("name", MODULE_CASES)
def test_modules_without_grad_match_the_reference_modules(sp, name, monkeypatch):
    """Inference path of the modules (fused projection where its shape rules allow, fused attention) against the outputs
    of the reference modules on the same state_dict."""
    f = np.load(os.path.join(GOLDEN, f"pyref_{name}.npz"))
    monkeypatch.setattr(torch.backends.cudnn, "allow_tf32", False)
    monkeypatch.setattr(torch.backends.cuda.matmul, "allow_tf32", False)
    kwargs = {k[3:]: f[k].item() for k in f.files if k.startswith("kw_")}
    cls = getattr(sp, str(f["meta_class"]))
    dev = torch.device("cuda:0")
    m = cls(**kwargs).to(dev)
    m.load_state_dict({k[3:]: torch.from_numpy(f[k]) for k in f.files if k.startswith("sd_")})
    m = m.eval()
    x = torch.from_numpy(f["in_x"]).to(dev)
    y = torch.from_numpy(f["in_y"]).to(dev)
    with torch.no_grad():
        out = m(y, x)
    want = f["out_out"]
    err = float(np.abs(out.double().cpu().numpy() - want).max() / np.abs(want).max())
    assert err < 2e-5, err


def test_graphed_pyramid_replays_bit_equal(sp):
    """Three chained SAPA modules (GroupNorm + projections on the GEMM kernel, fused attention) captured into one CUDA
    graph: replays on new inputs equal the eager calls bit for bit."""
    dev = torch.device("cuda:0")
    torch.manual_seed(3)
    ups = [sp.SAPA(64, embedding_dim=32).to(dev, torch.bfloat16).eval() for _ in range(3)]

    def pyramid(f0, f1, f2, f3):
        x = f3
        for y, m in zip((f2, f1, f0), ups):
            x = m(y, x)
        return x

    def feats(seed):
        g = torch.Generator().manual_seed(seed)
        return [torch.randn(2, 64, r, r, generator=g).to(dev, torch.bfloat16) for r in (64, 32, 16, 8)]

    graphed = sp.GraphedForward(pyramid, feats(0))
    for seed in (1, 2):
        f = feats(seed)
        with torch.no_grad():
            want = pyramid(*f)
        got = graphed(*f)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    from sapa_b200 import _lib
    assert _lib.wait_timeout_flags(dev) == 0


def test_projection_random_shapes(sp):
    """Seeded sweep over channel counts, pixel counts, output widths and batch sizes (float32, 1e-5)."""
    from sapa_b200.projection import project, project_supported
    rng = np.random.RandomState(5)
    done = 0
    for _ in range(40):
        B = int(rng.randint(1, 5))
        C = 32 * int(rng.randint(1, 11))
        H, W = int(rng.randint(1, 40)), 4 * int(rng.randint(1, 12))
        d = 16 * int(rng.randint(1, 9))
        groups = 32 if rng.rand() < 0.7 else 0
        x, norm, conv, ref = _case(B, C, H, W, d, groups, torch.float32, bias=bool(rng.rand() < 0.5), seed=int(rng.randint(1 << 30)))
        if not project_supported(x, norm, conv):
            continue
        out = project(x, norm, conv)
        err = float((out.double() - ref).abs().max() / ref.abs().max())
        assert err < 1e-5, (B, C, H, W, d, groups, err)
        done += 1
    assert done >= 30
