import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def golden_cases(prefix):
    """Names of the golden cases whose reference-Python file exists, e.g. prefix 'b_' or 'd_'."""
    names = sorted(f[len("pyref_"):-4] for f in os.listdir(GOLDEN) if f.startswith("pyref_" + prefix) and f.endswith(".npz"))
    return names


class Golden:
    """One golden case: inputs (float32), metadata and the expected float64 outputs of the reference."""

    def __init__(self, name, source="pyref"):
        f = np.load(os.path.join(GOLDEN, f"pyref_{name}.npz"))
        self.name = name
        self.inputs = {k[3:]: f[k] for k in f.files if k.startswith("in_")}
        self.meta = {k[5:]: f[k].item() for k in f.files if k.startswith("meta_")}
        self.expected = {k[4:]: f[k] for k in f.files if k.startswith("out_")}
        self.cuda = None
        path = os.path.join(GOLDEN, f"cudaref_{name}.npz")
        if os.path.exists(path):
            c = np.load(path)
            self.cuda = {k: c[k] for k in c.files}


def rel_err(got, want):
    """max|got - want| / max|want| (norm-relative error used throughout the parity tests)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


@pytest.fixture(scope="session")
def oracle():
    from oracle import c_oracle
    c_oracle.build()
    return c_oracle


# ------------------------------------------------------------------ which kernel must serve which call
# Mirrors the dispatch rules of csrc/sapa_b.cu so that a silent fall-back to a slower kernel fails a test instead of
# passing on the fall-back's (correct) numbers.  W = low-res width; `wide` = 16-bit element types.

def _tensor_map_rows(W, wide):
    """Rows of every tensor on a 16-byte boundary: what the tensor-map (TMA) kernels need."""
    return W % (8 if wide else 4) == 0


def expected_fused_forward(K, s, W, dtype_name):
    wide = dtype_name in ("f16", "bf16")
    if s != 2 or K not in (3, 5) or dtype_name == "f64":
        return None                                   # no fused kernel: the separate ops run
    if K == 5 and dtype_name == "f32" and W % 4 == 0:
        return ["sapa_tma_fused_f32_kernel<fwd>"]
    if K == 5 and wide and W % 8 == 0:
        return ["sapa_tma_fused_16_kernel<fwd>"]
    if K == 5 and (dtype_name == "f32" or W % 2 == 0):
        return ["sapa_mma_fused_kernel"]
    return ["sapa_tile_kernel<fused>"]


def _gath(K, s, W, dtype_name):
    wide = dtype_name in ("f16", "bf16")
    if K == 5 and s == 2 and dtype_name != "f64" and W % (4 if wide else 2) == 0:
        return "sapa_gath_mma_kernel"
    if s == 2 and K in (3, 5) and dtype_name != "f64":
        return "sapa_gath_kernel"
    return "gath_generic_kernel"


def expected_fused_backward(K, s, W, dtype_name):
    wide = dtype_name in ("f16", "bf16")
    tiled = s == 2 and K in (3, 5) and dtype_name != "f64"
    if K == 5 and s == 2 and dtype_name != "f64" and _tensor_map_rows(W, wide):
        stage1 = ["sapa_tma_fused_16_kernel<bwd>" if wide else "sapa_tma_fused_f32_kernel<bwd>"]
    elif tiled:
        stage1 = ["sapa_tile_kernel<bwd>"]
    else:
        stage1 = ["sim_generic_kernel", "softmax_bwd_generic_kernel", "agg_generic_kernel"]
    return stage1 + [_gath(K, s, W, dtype_name)] * 2


def expected_sim(K, s, W, dtype_name):
    wide = dtype_name in ("f16", "bf16")
    if K == 5 and s == 2 and dtype_name != "f64" and _tensor_map_rows(W, wide):
        return ["sapa_tma_fused_16_kernel<sim>" if wide else "sapa_tma_fused_f32_kernel<sim>"]
    if s == 2 and K in (3, 5) and dtype_name != "f64":
        return ["sapa_tile_kernel<sim>"]
    return ["sim_generic_kernel"]


def expected_agg(K, s, W, dtype_name):
    wide = dtype_name in ("f16", "bf16")
    if K == 5 and s == 2 and dtype_name != "f64" and _tensor_map_rows(W, wide):
        return ["sapa_tma_fused_16_kernel<agg>" if wide else "sapa_tma_fused_f32_kernel<agg>"]
    if s == 2 and K in (3, 5) and dtype_name != "f64":
        return ["sapa_tile_kernel<agg>"]
    return ["agg_generic_kernel"]
