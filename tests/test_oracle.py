"""The CPU oracle against the reference: golden vectors made by the reference's own code, plus
hand-computable cases.  No GPU, no product code."""
import numpy as np
import pytest
import torch

from conftest import Golden, golden_cases, rel_err

TOL64 = 1e-12   # float64 oracle vs float64 reference Python functions
TOLCUDA = 1e-11  # float64 oracle vs float64 run of the reference's CUDA kernels (atomics reorder sums)


@pytest.mark.parametrize("name", golden_cases("b_"))
def test_c_oracle_sapa_b_matches_reference_python(oracle, name):
    g = Golden(name)
    K, s = g.meta["K"], g.meta["s"]
    x = {k: v.astype(np.float64) for k, v in g.inputs.items()}
    assert rel_err(oracle.qk_forward(x["query"], x["key"], K, s), g.expected["sim"]) < TOL64
    gq, gk = oracle.qk_backward(x["grad_sim"], x["query"], x["key"], K, s)
    assert rel_err(gq, g.expected["sim_dquery"]) < TOL64 and rel_err(gk, g.expected["sim_dkey"]) < TOL64
    assert rel_err(oracle.av_forward(x["attn"], x["value"], K, s), g.expected["agg"]) < TOL64
    ga, gv = oracle.av_backward(x["grad_out"], x["attn"], x["value"], K, s)
    assert rel_err(ga, g.expected["agg_dattn"]) < TOL64 and rel_err(gv, g.expected["agg_dvalue"]) < TOL64
    out, prob = oracle.sapa_forward(x["query"], x["key"], x["value"], K, s, return_attn=True)
    assert rel_err(out, g.expected["full"]) < TOL64 and rel_err(prob, g.expected["full_prob"]) < TOL64
    fq, fk, fv = oracle.sapa_backward(x["grad_out"], x["query"], x["key"], x["value"], K, s)
    assert rel_err(fq, g.expected["full_dquery"]) < 1e-11
    assert rel_err(fk, g.expected["full_dkey"]) < 1e-11
    assert rel_err(fv, g.expected["full_dvalue"]) < 1e-11


@pytest.mark.parametrize("name", golden_cases("d_"))
def test_c_oracle_sapa_d_matches_reference_python(oracle, name):
    g = Golden(name)
    P, s, G = g.meta["P"], g.meta["s"], g.meta["G"]
    x = {k: v.astype(np.float64) for k, v in g.inputs.items()}
    assert rel_err(oracle.deform_qk_forward(x["query"], x["key"], x["offset"], P, s, G), g.expected["sim"]) < TOL64
    gq, gk, go = oracle.deform_qk_backward(x["grad_sim"], x["query"], x["key"], x["offset"], P, s, G)
    assert rel_err(gq, g.expected["sim_dquery"]) < TOL64
    assert rel_err(gk, g.expected["sim_dkey"]) < TOL64
    assert rel_err(go, g.expected["sim_doffset"]) < TOL64
    assert rel_err(oracle.deform_av_forward(x["attn"], x["value"], x["offset"], P, s, G), g.expected["agg"]) < TOL64
    ga, gv, go = oracle.deform_av_backward(x["grad_out"], x["attn"], x["value"], x["offset"], P, s, G)
    assert rel_err(ga, g.expected["agg_dattn"]) < TOL64
    assert rel_err(gv, g.expected["agg_dvalue"]) < TOL64
    assert rel_err(go, g.expected["agg_doffset"]) < TOL64
    out, prob = oracle.deform_sapa_forward(x["query"], x["key"], x["value"], x["offset"], P, s, G, return_attn=True)
    assert rel_err(out, g.expected["full"]) < TOL64 and rel_err(prob, g.expected["full_prob"]) < TOL64
    fq, fk, fv, fo = oracle.deform_sapa_backward(x["grad_out"], x["query"], x["key"], x["value"], x["offset"], P, s, G)
    for got, key in ((fq, "full_dquery"), (fk, "full_dkey"), (fv, "full_dvalue"), (fo, "full_doffset")):
        assert rel_err(got, g.expected[key]) < 1e-11, key


@pytest.mark.parametrize("name", golden_cases("b_") + golden_cases("d_"))
def test_c_oracle_matches_reference_cuda_kernels(oracle, name):
    """Vectors produced by the reference's compiled CUDA extensions on a B200 (float64 run)."""
    g = Golden(name)
    if g.cuda is None:
        pytest.skip("no cudaref vector for this case")
    x = {k: v.astype(np.float64) for k, v in g.inputs.items()}
    s = g.meta["s"]
    if name.startswith("b_"):
        K = g.meta["K"]
        got = dict(sim=oracle.qk_forward(x["query"], x["key"], K, s), agg=oracle.av_forward(x["attn"], x["value"], K, s))
        got["sim_dquery"], got["sim_dkey"] = oracle.qk_backward(x["grad_sim"], x["query"], x["key"], K, s)
        got["agg_dattn"], got["agg_dvalue"] = oracle.av_backward(x["grad_out"], x["attn"], x["value"], K, s)
        got["full"], got["full_prob"] = oracle.sapa_forward(x["query"], x["key"], x["value"], K, s, return_attn=True)
    else:
        P, G = g.meta["P"], g.meta["G"]
        got = dict(sim=oracle.deform_qk_forward(x["query"], x["key"], x["offset"], P, s, G),
                   agg=oracle.deform_av_forward(x["attn"], x["value"], x["offset"], P, s, G))
        got["sim_dquery"], got["sim_dkey"], got["sim_doffset"] = oracle.deform_qk_backward(
            x["grad_sim"], x["query"], x["key"], x["offset"], P, s, G)
        got["agg_dattn"], got["agg_dvalue"], got["agg_doffset"] = oracle.deform_av_backward(
            x["grad_out"], x["attn"], x["value"], x["offset"], P, s, G)
        got["full"], got["full_prob"] = oracle.deform_sapa_forward(x["query"], x["key"], x["value"], x["offset"], P, s, G,
                                                                   return_attn=True)
    for key, val in got.items():
        assert rel_err(val, g.cuda["f64_" + key]) < TOLCUDA, key


@pytest.mark.parametrize("name", golden_cases("b_"))
def test_unfold_port_matches_reference_python(name):
    from oracle import unfold_port as up
    g = Golden(name)
    K, s = g.meta["K"], g.meta["s"]
    x = {k: torch.from_numpy(v).double() for k, v in g.inputs.items()}
    assert rel_err(up.sim(x["query"], x["key"], K, s).numpy(), g.expected["sim"]) < TOL64
    assert rel_err(up.atn(x["attn"], x["value"], K, s).numpy(), g.expected["agg"]) < TOL64
    assert rel_err(up.sapa(x["query"], x["key"], x["value"], K, s).numpy(), g.expected["full"]) < TOL64


@pytest.mark.parametrize("name", golden_cases("d_"))
def test_unfold_port_deform_matches_reference_python(name):
    from oracle import unfold_port as up
    g = Golden(name)
    P, s, G = g.meta["P"], g.meta["s"], g.meta["G"]
    x = {k: torch.from_numpy(v).double() for k, v in g.inputs.items()}
    assert rel_err(up.deform_sim(x["query"], x["key"], x["offset"], P, s, G).numpy(), g.expected["sim"]) < TOL64
    assert rel_err(up.deform_atn(x["attn"], x["value"], x["offset"], P, s, G).numpy(), g.expected["agg"]) < TOL64
    assert rel_err(up.deform_sapa(x["query"], x["key"], x["value"], x["offset"], P, s, G).numpy(), g.expected["full"]) < TOL64


def test_config1_single_op_forward(oracle):
    """Benchmark configuration 1 (the CPU-runnable single-op case): B=1, X 64x16x16, Y 64x32x32, 1x1 projections to d=32, K=5, s=2, float32."""
    g = Golden("cfg1")
    X, Y, Wq, Wk = (g.inputs[k] for k in ("X", "Y", "Wq", "Wk"))
    q = np.einsum("oc,bchw->bohw", Wq, Y).astype(np.float32)
    k = np.einsum("oc,bchw->bohw", Wk, X).astype(np.float32)
    out = oracle.sapa_forward(q, k, X, 5, 2)
    assert out.shape == (1, 64, 32, 32) and out.dtype == np.float32
    assert rel_err(out, g.expected["full"]) < 1e-5      # float32 arithmetic vs the float64 reference run


def test_border_slots_are_zero_logits_and_keep_their_softmax_weight(oracle):
    """A key outside the image gives logit exactly 0 (not -inf) and the softmax still spans all K*K slots."""
    q = np.ones((1, 1, 2, 2), np.float64)
    k = np.full((1, 1, 1, 1), 3.0, np.float64)
    sim = oracle.qk_forward(q, k, 3, 2)              # single low-res pixel: only the centre slot is inside
    assert sim.shape == (1, 9, 2, 2)
    centre = sim[0, 4]
    assert np.all(centre == 3.0)
    assert np.all(np.delete(sim[0], 4, axis=0) == 0.0)
    prob = oracle.softmax(sim, 1)
    want_centre = np.exp(3.0) / (np.exp(3.0) + 8.0)
    assert np.allclose(prob[0, 4], want_centre, rtol=1e-14)
    out = oracle.av_forward(prob, k, 3, 2)           # value outside the image contributes nothing
    assert np.allclose(out, 3.0 * want_centre, rtol=1e-14)


def test_hand_computed_window_order(oracle):
    """Slot k = dy*K+dx addresses neighbour (y-r+dy, x-r+dx): row-major like F.unfold."""
    key = np.arange(9, dtype=np.float64).reshape(1, 1, 3, 3)
    q = np.ones((1, 1, 3, 3), np.float64)
    sim = oracle.qk_forward(q, key, 3, 1)
    assert np.array_equal(sim[0, :, 1, 1], np.arange(9.0))          # centre pixel sees the whole image in order
    assert np.array_equal(sim[0, :, 0, 0], [0, 0, 0, 0, 0, 1, 0, 3, 4])


def test_deform_zero_offset_reads_parent_pixel(oracle):
    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, 2, 4, 6))
    k = rng.standard_normal((1, 2, 2, 3))
    off = np.zeros((1, 2 * 1 * 2, 4, 6))
    sim = oracle.deform_qk_forward(q, k, off, 1, 2, 2)
    up = np.repeat(np.repeat(k, 2, axis=2), 2, axis=3)
    assert np.allclose(sim[:, :, 0], q * up, rtol=1e-14)


def test_float32_and_float64_variants_agree(oracle):
    g = Golden("b_gradcheck")
    K, s = g.meta["K"], g.meta["s"]
    q, k = g.inputs["query"], g.inputs["key"]
    a = oracle.qk_forward(q, k, K, s)
    b = oracle.qk_forward(q.astype(np.float64), k.astype(np.float64), K, s)
    assert a.dtype == np.float32 and rel_err(a, b) < 1e-6
