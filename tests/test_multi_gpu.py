"""Row-slab sharding on real GPUs: two NCCL ranks (one process per GPU) exchange their halo rows and must reproduce the
rows of the unsharded op bit for bit.  Needs two GPUs; skipped on a single-GPU machine."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, dtype_name, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import sapa_b200
        from sapa_b200 import sharding
        dtype = {"f32": torch.float32, "bf16": torch.bfloat16}[dtype_name]
        B, d, C, H, W, K, s = 2, 32, 64, 40, 48, 5, 2
        g = torch.Generator().manual_seed(17)
        q, k, v = (torch.randn(*sh, generator=g).to(dev, dtype) for sh in ((B, d, s * H, s * W), (B, d, H, W), (B, C, H, W)))
        full = sapa_b200.sapa_fused(q, k, v, K, s)
        rows = sharding.row_slice(H, world, rank)
        mine = sharding.sapa_fused_row_sharded(q[:, :, s * rows.start:s * rows.stop].contiguous(),
                                               k[:, :, rows].contiguous(), v[:, :, rows].contiguous(), K, s)
        torch.cuda.synchronize()
        ok = bool(torch.equal(mine, full[:, :, s * rows.start:s * rows.stop]))
        # backward of the row-sharded op: the rank's rows of the unsharded gradients (the edge rows of the key / value
        # gradients are sums over two ranks, so they agree to rounding, everything else bit for bit)
        go = torch.randn(B, C, s * H, s * W, generator=g).to(dev, dtype)
        qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))
        gq, gk, gv = torch.autograd.grad(sapa_b200.sapa_fused(qf, kf, vf, K, s), (qf, kf, vf), go)
        slab = sharding.RowSlab(B, d, C, rows.stop - rows.start, W, dtype, dev, K, s)
        slab.key.copy_(k[:, :, rows]); slab.value.copy_(v[:, :, rows])
        hi = slice(s * rows.start, s * rows.stop)
        ql = q[:, :, hi].contiguous()
        slab.forward(ql, keep_attn=True)
        mq, mk, mv = slab.backward(go[:, :, hi].contiguous(), ql)
        torch.cuda.synchronize()
        tol = 1e-5 if dtype == torch.float32 else 2e-2

        def close(a, b):
            return float((a.float() - b.float()).abs().max()) <= tol * float(b.float().abs().max())
        ok = ok and bool(torch.equal(mq, gq[:, :, hi])) and close(mk, gk[:, :, rows]) and close(mv, gv[:, :, rows])
        # the same through autograd
        ql2, kl2, vl2 = (t.clone().requires_grad_() for t in (ql, k[:, :, rows].contiguous(), v[:, :, rows].contiguous()))
        aq, ak, av = torch.autograd.grad(sharding.sapa_fused_row_sharded(ql2, kl2, vl2, K, s), (ql2, kl2, vl2),
                                         go[:, :, hi].contiguous())
        torch.cuda.synchronize()
        ok = ok and bool(torch.equal(aq, mq)) and bool(torch.equal(ak, mk)) and bool(torch.equal(av, mv))
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("dtype_name", ["f32", "bf16"])
def test_row_sharded_equals_unsharded_rows_on_two_gpus(dtype_name):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(2, port, dtype_name, ret), nprocs=2, join=True)
        assert dict(ret) == {0: True, 1: True}


def _worker_deform(rank, world, port, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import sapa_b200
        from sapa_b200 import sharding
        B, d, C, H, W, G, P, s = 2, 32, 64, 48, 32, 4, 9, 2
        g = torch.Generator().manual_seed(29)
        q, k, v, off, go = (torch.randn(*sh, generator=g).to(dev) for sh in (
            (B, d, s * H, s * W), (B, d, H, W), (B, C, H, W), (B, 2 * G * P, s * H, s * W), (B, C, s * H, s * W)))
        off = 0.5 * off
        full_in = [t.clone().requires_grad_() for t in (q, k, v, off)]
        full = sapa_b200.deform_sapa_fused(*full_in, P, s, G)
        grads = torch.autograd.grad(full, full_in, go)
        rows = sharding.row_slice(H, world, rank)
        hi = slice(s * rows.start, s * rows.stop)
        mine_in = [q[:, :, hi], k[:, :, rows], v[:, :, rows], off[:, :, hi]]
        mine_in = [t.contiguous().requires_grad_() for t in mine_in]
        depth = sharding.deform_halo_rows(mine_in[3])
        mine = sharding.sapa_deform_row_sharded(*mine_in, P, s, G)
        mine_grads = torch.autograd.grad(mine, mine_in, go[:, :, hi].contiguous())
        torch.cuda.synchronize()

        def close(a, b, tol=2e-5):
            return float((a - b).abs().max()) <= tol * float(b.abs().max())
        ok = depth == int(off[:, 1::2].abs().max()) + 1 and close(mine, full[:, :, hi])
        with torch.no_grad():       # inference: the slab form of the kernels, no padded query / offsets
            fast = sharding.sapa_deform_row_sharded(*[t.detach() for t in mine_in], P, s, G)
        ok = ok and "deform_window_kernel" in sapa_b200._lib.last_kernels() and close(fast, full[:, :, hi])
        # resident slab: halo rows exchanged in place; first with the measured depth, then with a larger given bound
        slab = sharding.DeformRowSlab(B, d, C, rows.stop - rows.start, W, depth + 2, dev, P, G)
        slab.key.copy_(k[:, :, rows]); slab.value.copy_(v[:, :, rows])
        qd, od = mine_in[0].detach(), mine_in[3].detach()
        ok = ok and close(slab.forward(qd, od), full[:, :, hi]) and close(slab.forward(qd, od, halo=depth + 1), full[:, :, hi])
        try:
            slab.forward(qd, od, halo=depth + 3)
            ok = False
        except ValueError:
            pass
        # the same in bfloat16 (16-bit operands, float32 similarities), against the unsharded bfloat16 op
        h = [t.detach().to(torch.bfloat16) for t in (q, k, v, off)]
        full16 = sapa_b200.deform_sapa_fused(*h, P, s, G)
        slab16 = sharding.DeformRowSlab(B, d, C, rows.stop - rows.start, W, depth + 2, dev, P, G, dtype=torch.bfloat16)
        slab16.key.copy_(h[1][:, :, rows]); slab16.value.copy_(h[2][:, :, rows])
        got16 = slab16.forward(h[0][:, :, hi].contiguous(), h[3][:, :, hi].contiguous())
        ok = ok and got16.dtype == torch.bfloat16 and close(got16.float(), full16[:, :, hi].float(), 1e-2)
        for got, want, sl in zip(mine_grads, grads, (hi, rows, rows, hi)):
            ok = ok and close(got, want[:, :, sl])
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


def test_deform_row_sharded_equals_unsharded_rows_on_two_gpus():
    """SAPA-D on two row slabs with the measured halo depth: output rows and the gradients of query, key, value and
    offsets equal the rows of the unsharded op (float32; sums over atomics, so to rounding)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker_deform, args=(2, port, ret), nprocs=2, join=True)
        assert dict(ret) == {0: True, 1: True}
