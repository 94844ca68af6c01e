"""The allocation-free backward entry point, sapa_fused_backward_static.

It serves callers that cannot allocate device memory at the call site (engines with a fixed memory plan, plugin hosts
without a reachable allocator, real-time loops that may not call cudaMalloc), so the test reaches it the way they would: through the C
ABI, with every buffer allocated beforehand.  Its gradients must equal those of the ordinary entry point, which
gets a caller-provided workspace, on two calls in a row (the built-in scratch keeps the first call's contents).
Collected last on purpose: a failure here must not hide the results of the other tests in a -x run.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _problem(seed, B, d, C, H, W, K, s, dtype):
    from sapa_b200.functions import fused_forward_raw
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, d, s * H, s * W, generator=g).to(DEV, dtype)
    k = torch.randn(B, d, H, W, generator=g).to(DEV, dtype)
    v = torch.randn(B, C, H, W, generator=g).to(DEV, dtype)
    go = torch.randn(B, C, s * H, s * W, generator=g).to(DEV, dtype)
    _, attn = fused_forward_raw(q, k, v, K, s, True)
    return q, k, v, go, attn


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_backward_matches_workspace_backward_twice(dtype):
    from sapa_b200 import _lib
    code = {torch.float32: 0, torch.bfloat16: 2}[dtype]
    K, s = 5, 2
    tol = 0.0   # both entry points run the same deterministic kernels: bit-identical results
    for call, (B, d, C, H, W) in enumerate(((2, 16, 24, 12, 20), (1, 8, 40, 9, 33))):   # second call: other sizes
        q, k, v, go, attn = _problem(40 + call, B, d, C, H, W, K, s, dtype)
        want = [torch.empty_like(t) for t in (q, k, v)]
        nbytes = _lib.fused_backward_workspace(B, H, W, K, s, code)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
        _lib.call("sapa_fused_backward", q.device, go, q, k, v, attn, *want, ws, nbytes, B, d, C, H, W, K, s, code)
        got = [torch.full_like(t, float("nan")) for t in (q, k, v)]
        # a first call on this device: it loads the kernels and looks up the scratch array's address (set-up, not part of
        # the promise); from then on the device's free memory, as the driver reports it, must not move across a call
        # (torch's own counters would not see a cudaMalloc inside the library)
        _lib.call("sapa_fused_backward_static", q.device, go, q, k, v, attn, *got, B, d, C, H, W, K, s, code)
        torch.cuda.synchronize()
        for t in got:
            t.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(torch.device(DEV))[0]
        _lib.call("sapa_fused_backward_static", q.device, go, q, k, v, attn, *got, B, d, C, H, W, K, s, code)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(torch.device(DEV))[0] == free_before
        for a, b in zip(got, want):
            assert torch.isfinite(a).all()
            assert float((a.float() - b.float()).abs().max()) <= tol


def test_static_scratch_rejects_problems_beyond_its_capacity():
    from sapa_b200 import _lib
    cap = int(_lib.lib().sapa_fused_backward_static_capacity())
    assert cap == 16 << 20
    B, d, C, H, W, K, s = 16, 4, 4, 64, 64, 5, 2            # 16*25*128*128*4 B = 26 MB of scratch
    assert _lib.fused_backward_workspace(B, H, W, K, s, 0) > cap
    t = torch.zeros(16, device=DEV)                           # never touched: the size check comes first
    with pytest.raises(RuntimeError, match="built-in buffer"):
        _lib.call("sapa_fused_backward_static", t.device, t, t, t, t, t, t, t, t, B, d, C, H, W, K, s, 0)


def test_zzz_bounded_wait_gives_up_and_the_library_recovers():
    """A kernel whose bounded barrier wait runs out (a barrier that nothing signals, a limit of a few dozen tries) raises
    the device flag and returns; reading the flag clears it, and the next fused forward is correct."""
    import torch
    import sapa_b200
    from sapa_b200 import _lib
    dev = torch.device("cuda:0")
    assert _lib.wait_timeout_flags(dev) == 0
    _lib.call("sapa_selftest_wait_timeout", dev)
    assert _lib.last_kernels() == ["sapa_wait_selftest_kernel"]
    assert _lib.wait_timeout_flags(dev) == 1          # bit 0: the tensor-map kernels' flag
    assert _lib.wait_timeout_flags(dev) == 0          # reading cleared it (and reset the tile schedulers)
    g = torch.Generator().manual_seed(5)
    q, k, v = torch.randn(1, 16, 16, 32, generator=g), torch.randn(1, 16, 8, 16, generator=g), torch.randn(1, 32, 8, 16, generator=g)
    out = sapa_b200.sapa_fused(q.to(dev), k.to(dev), v.to(dev), 5, 2)
    ref = sapa_b200.av(torch.softmax(sapa_b200.qk(q.to(dev), k.to(dev), 5, 2), dim=1), v.to(dev), 5, 2)
    assert _lib.wait_timeout_flags(dev) == 0
    assert float((out - ref).abs().max()) < 1e-5
