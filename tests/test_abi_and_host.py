"""CPU-side checks of the drop-in boundary: the C-ABI library loads and exports what the header declares,
argument validation answers without touching a GPU, and the Python layer keeps the reference's error
behaviour.  No kernel is launched here."""
import ctypes
import os
import re
import sys

import pytest
import torch

from conftest import ROOT


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "sapa_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sapa_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from sapa_b200 import _lib
    handle = _lib.lib()
    names = _declared_functions()
    assert len(names) >= 15
    for name in names:
        assert hasattr(handle, name), f"{name} is declared in include/sapa_b200.h but not exported"
    assert sorted(_lib.EXPORTS) == names
    assert handle.sapa_abi_version() == _lib.ABI_VERSION


def test_argument_validation_needs_no_gpu():
    from sapa_b200 import _lib
    h = _lib.lib()
    null = ctypes.c_void_p(0)
    ok = ctypes.c_void_p(4096)          # never dereferenced: validation fails first
    # NULL pointer
    assert h.sapa_qk_forward(null, ok, ok, 1, 4, 4, 4, 5, 2, 0, null) == -1
    assert b"NULL" in h.sapa_last_error()
    # even kernel size
    assert h.sapa_qk_forward(ok, ok, ok, 1, 4, 4, 4, 4, 2, 0, null) == -1
    assert b"odd" in h.sapa_last_error()
    # unknown dtype
    assert h.sapa_av_forward(ok, ok, ok, 1, 4, 4, 4, 5, 2, 9, null) == -2
    # a pointer that is not aligned to the element size; the fused forward needs 16 bytes (views with an odd storage
    # offset go to the generic kernels in the separate ops, which cannot be shown without a GPU)
    assert h.sapa_av_forward(ctypes.c_void_p(4098), ok, ok, 1, 4, 4, 4, 5, 2, 0, null) == -3
    assert h.sapa_fused_forward(ctypes.c_void_p(4100), ok, ok, ok, null, 1, 4, 4, 4, 4, 5, 2, 0, null) == -3
    # fused: unsupported configurations are reported, not silently run elsewhere
    assert h.sapa_fused_forward(ok, ok, ok, ok, null, 1, 4, 4, 4, 4, 7, 2, 0, null) == -5
    assert h.sapa_fused_forward(ok, ok, ok, ok, null, 1, 4, 4, 4, 4, 5, 2, 3, null) == -5
    # deform: channels not divisible by groups
    assert h.sapa_deform_qk_forward(ok, ok, ok, ok, 1, 6, 4, 4, 5, 2, 4, 0, null) == -1
    # backward without workspace
    assert h.sapa_fused_backward(ok, ok, ok, ok, ok, ok, ok, ok, null, 0, 1, 4, 4, 4, 4, 5, 2, 0, null) == -6
    assert h.sapa_fused_backward_workspace(8, 64, 64, 5, 2, 0) == 8 * 25 * 128 * 128 * 4


def test_cpu_tensors_raise_not_implemented_like_the_reference():
    import sapa_b200 as sp
    q, k, v = torch.randn(1, 4, 4, 4), torch.randn(1, 4, 2, 2), torch.randn(1, 3, 2, 2)
    with pytest.raises(NotImplementedError):
        sp.qk(q, k, 5, 2)
    with pytest.raises(NotImplementedError):
        sp.av(torch.randn(1, 25, 4, 4), v, 5, 2)
    with pytest.raises(NotImplementedError):
        sp.sapa_fused(q, k, v, 5, 2)
    off = torch.randn(1, 2 * 3 * 2, 4, 4)
    with pytest.raises(NotImplementedError):
        sp.deform_qk(q, k, off, 3, 2, 2)
    with pytest.raises(NotImplementedError):
        sp.deform_av(torch.randn(1, 2, 3, 4, 4), torch.randn(1, 4, 2, 2), off, 3, 2, 2)


def test_shape_assertions_match_the_reference():
    import sapa_b200 as sp
    with pytest.raises(AssertionError):      # query is not scale x key
        sp.qk(torch.randn(1, 4, 5, 4), torch.randn(1, 4, 2, 2), 5, 2)
    with pytest.raises(AssertionError):      # even kernel
        sp.qk(torch.randn(1, 4, 4, 4), torch.randn(1, 4, 2, 2), 4, 2)
    with pytest.raises(AssertionError):      # attention channels != K*K
        sp.av(torch.randn(1, 24, 4, 4), torch.randn(1, 3, 2, 2), 5, 2)
    with pytest.raises(AssertionError):      # offset channels != G*P*2
        sp.deform_qk(torch.randn(1, 4, 4, 4), torch.randn(1, 4, 2, 2), torch.randn(1, 10, 4, 4), 3, 2, 2)
    with pytest.raises(AssertionError):      # deform: q and k channel counts differ
        sp.deform_qk(torch.randn(1, 4, 4, 4), torch.randn(1, 6, 2, 2), torch.randn(1, 12, 4, 4), 3, 2, 2)


def test_modules_keep_reference_parameter_names_and_init():
    import sapa_b200 as sp
    m = sp.SAPA(64, dim_x=96, embedding_dim=32)
    assert sorted(m.state_dict()) == sorted(
        ["norm_y.weight", "norm_y.bias", "norm_x.weight", "norm_x.bias", "q.weight", "q.bias", "k.weight", "k.bias"])
    assert m.q.weight.shape == (32, 64, 1, 1) and m.k.weight.shape == (32, 96, 1, 1)
    assert float(m.q.bias.abs().max()) == 0.0 and 0.005 < float(m.q.weight.std()) < 0.04
    d = sp.SAPADeform(16, up_factor=2, num_point=9, groups=4, embedding_dim=8)
    assert sorted(d.state_dict()) == sorted(["q.weight", "q.bias", "k.weight", "k.bias", "offset.weight", "offset.bias"])
    assert d.q.weight.shape[0] == 32 and d.offset.weight.shape[0] == 4 * 9 * 2 * 4
    assert sp.SAPADeform(16, high_offset=False).offset.weight.shape[0] == 4 * 9 * 2
    with pytest.raises(ValueError):
        sp.SAPA(64, impl="triton")


def test_compat_packages_import_under_reference_names():
    import sapa_b200 as sp
    sys.path.insert(0, sp.compat_path())
    try:
        import av_ext, dav, deformsapa, dqk, qk_ext, sapa  # noqa: F401,E401
        assert sapa.qk is sp.qk and sapa.av is sp.av
        assert deformsapa.deform_qk is sp.deform_qk and deformsapa.deform_av is sp.deform_av
        for mod in (qk_ext, av_ext, dqk, dav):
            assert callable(mod.forward) and callable(mod.backward)
        with pytest.raises(RuntimeError):    # CHECK_CUDA of the reference: CPU tensors are a RuntimeError here
            qk_ext.forward(torch.randn(1, 4, 2, 2), torch.randn(1, 4, 4, 4), 5, 2, torch.zeros(1, 25, 4, 4))
    finally:
        sys.path.remove(sp.compat_path())


def test_product_package_never_touches_the_oracle():
    """The oracle is test infrastructure: no file of the product package may import, load or name it."""
    pkg = os.path.join(ROOT, "sapa_b200")
    pattern = re.compile(r"import\s+oracle|from\s+oracle|oracle[/.]|libsapa_oracle")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert not pattern.search(text), os.path.join(dirpath, f)
