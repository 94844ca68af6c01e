"""Host logic of the multi-GPU paths on CPU: two gloo ranks exchange row halos and the padded slabs must
equal slices of the zero-padded full tensor; batch slices must tile the batch."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sapa_b200 import sharding


def test_batch_and_row_slices_tile_the_range():
    for total in (1, 7, 8, 64):
        for world in (1, 2, 3, 4, 8):
            got = []
            for r in range(world):
                sl = sharding.batch_slice(total, world, r)
                got += list(range(total))[sl]
            assert got == list(range(total))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, halo, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(7)
        H, W = 4 * world, 5
        key = torch.randn(2, 3, H, W, generator=g)
        value = torch.randn(2, 6, H, W, generator=g)
        rows = sharding.row_slice(H, world, rank)
        kp, vp = sharding.exchange_row_halo([key[:, :, rows].contiguous(), value[:, :, rows].contiguous()], halo)
        full_k = torch.nn.functional.pad(key, (0, 0, halo, halo))
        full_v = torch.nn.functional.pad(value, (0, 0, halo, halo))
        ok = torch.equal(kp, full_k[:, :, rows.start:rows.stop + 2 * halo]) and \
            torch.equal(vp, full_v[:, :, rows.start:rows.stop + 2 * halo])
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,halo", [(2, 2), (3, 1), (2, 0)])
def test_row_halo_exchange_gloo(world, halo):
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, halo, ret), nprocs=world, join=True)
        assert dict(ret) == {r: True for r in range(world)}


def _worker_uneven(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        H, W = 4, 5                                  # 4 rows over 3 ranks: shares (2, 1, 1), one below the halo of 2
        rows = sharding.row_slice(H, world, rank)
        key = torch.zeros(1, 2, rows.stop - rows.start, W)
        try:
            sharding.exchange_row_halo([key], 2)
            ret[rank] = "no error"
        except ValueError as exc:
            ret[rank] = "ValueError" if "shares [2, 1, 1]" in str(exc) else str(exc)
    finally:
        dist.destroy_process_group()


def test_uneven_split_below_the_halo_raises_on_every_rank_together():
    """A rank whose share is too small must not raise alone: its neighbour would wait in a receive for ever.  Every rank
    sees every share and all raise the same error before any point-to-point operation is posted."""
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker_uneven, args=(3, port, ret), nprocs=3, join=True)
        assert dict(ret) == {0: "ValueError", 1: "ValueError", 2: "ValueError"}


def _worker_resident(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(3)
        H, W, r = 5 * world, 8, 2
        key, value = torch.randn(1, 3, H, W, generator=g), torch.randn(1, 4, H, W, generator=g)
        rows = sharding.row_slice(H, world, rank)
        slab = sharding.RowSlab(1, 3, 4, rows.stop - rows.start, W, torch.float32, "cpu")
        ok = True
        for step in range(2):                        # the buffers are resident: a second step reuses them
            slab.key.copy_(key[:, :, rows] + step)
            slab.value.copy_(value[:, :, rows] - step)
            sharding._exchange_into([slab.key_padded, slab.value_padded], r)
            full_k = torch.nn.functional.pad(key + step, (0, 0, r, r))
            full_v = torch.nn.functional.pad(value - step, (0, 0, r, r))
            if rank == 0:                            # image border: the halo stays zero
                full_k[:, :, :r], full_v[:, :, :r] = 0, 0
            if rank == world - 1:
                full_k[:, :, -r:], full_v[:, :, -r:] = 0, 0
            ok = ok and torch.equal(slab.key_padded, full_k[:, :, rows.start:rows.stop + 2 * r]) and \
                torch.equal(slab.value_padded, full_v[:, :, rows.start:rows.stop + 2 * r])
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_resident_slab_exchanges_only_its_halo_rows_in_place():
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker_resident, args=(3, port, ret), nprocs=3, join=True)
        assert dict(ret) == {0: True, 1: True, 2: True}


def _worker_reduce(rank, world, port, halo, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # Every rank holds gradient contributions in its padded frame; the sum over the ranks, each placed at its
        # position in the padded full image, is what the reduction must reproduce on the ranks' own rows.
        H, W, hl = 4 * world, 3, 4
        g = torch.Generator().manual_seed(11)
        contrib = [[torch.randn(2, c, hl + 2 * halo, W, generator=g) for c in (3, 5)] for _ in range(world)]
        mine = [t.clone() for t in contrib[rank]]
        sharding._reduce_halo_grads(mine, halo)
        ok = True
        for ti, c in enumerate((3, 5)):
            full = torch.zeros(2, c, H + 2 * halo, W)
            for r in range(world):
                full[:, :, r * hl:r * hl + hl + 2 * halo] += contrib[r][ti]
            want = full[:, :, halo + rank * hl:halo + rank * hl + hl]
            got = mine[ti][:, :, halo:halo + hl]
            ok = ok and bool(torch.allclose(got, want, atol=1e-6))
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,halo", [(2, 2), (3, 2), (3, 1)])
def test_halo_gradient_reduction_gloo(world, halo):
    """Backward of the halo exchange: halo rows of the padded gradients go to the neighbours and are added to their edge
    rows; the ranks' own rows then hold the sum of every rank's contribution."""
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker_reduce, args=(world, port, halo, ret), nprocs=world, join=True)
        assert dict(ret) == {r: True for r in range(world)}


def _deform_case(world, hl, sigma):
    """One image split into ``world`` slabs of ``hl`` low-res rows: float64 so that the comparison can be tight."""
    g = torch.Generator().manual_seed(23)
    B, d, C, W, G, P, s = 1, 8, 8, 6, 2, 4, 2
    H = world * hl
    q = torch.randn(B, d, s * H, s * W, generator=g, dtype=torch.float64)
    k = torch.randn(B, d, H, W, generator=g, dtype=torch.float64)
    v = torch.randn(B, C, H, W, generator=g, dtype=torch.float64)
    off = sigma * torch.randn(B, 2 * G * P, s * H, s * W, generator=g, dtype=torch.float64)
    go = torch.randn(B, C, s * H, s * W, generator=g, dtype=torch.float64)
    return q, k, v, off, go, (P, s, G)


def _worker_deform(rank, world, port, sigma, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import unfold_port
        hl = 5
        q, k, v, off, go, (P, s, G) = _deform_case(world, hl, sigma)
        full = [t.clone().requires_grad_(True) for t in (q, k, v, off)]
        want = unfold_port.deform_sapa(*full, P, s, G)
        want.backward(go)
        lo, hi = slice(rank * hl, (rank + 1) * hl), slice(s * rank * hl, s * (rank + 1) * hl)
        mine = [q[:, :, hi].clone(), k[:, :, lo].clone(), v[:, :, lo].clone(), off[:, :, hi].clone()]
        mine = [t.requires_grad_(True) for t in mine]
        depth = sharding.deform_halo_rows(mine[3])
        got = sharding.sapa_deform_row_sharded(*mine, P, s, G, op=unfold_port.deform_sapa)
        got.backward(go[:, :, hi])
        ok = depth == int(off[:, 1::2].abs().max()) + 1 and depth <= hl
        ok = ok and bool(torch.allclose(got, want[:, :, hi], atol=1e-12))
        for t, f, rows in zip(mine, full, (hi, lo, lo, hi)):
            ok = ok and bool(torch.allclose(t.grad, f.grad[:, :, rows], atol=1e-12))
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,sigma", [(2, 0.5), (3, 1.0)])
def test_deform_row_sharding_equals_the_unsharded_rows_gloo(world, sigma):
    """SAPA-D on row slabs with a measured halo depth: output rows and all four gradients equal the unsharded op's
    (PyTorch transcription as the per-slab operator; the CUDA kernels take its place on GPUs)."""
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker_deform, args=(world, port, sigma, ret), nprocs=world, join=True)
        assert dict(ret) == {r: True for r in range(world)}


def _worker_deform_refuse(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import unfold_port
        q, k, v, off, _, (P, s, G) = _deform_case(world, 2, 0.1)
        off[0, 1, 0, 0] = 7.5            # one far point on rank 0: depth 8 > 2 rows per rank, seen by every rank
        lo, hi = slice(rank * 2, (rank + 1) * 2), slice(s * rank * 2, s * (rank + 1) * 2)
        try:
            sharding.sapa_deform_row_sharded(q[:, :, hi], k[:, :, lo], v[:, :, lo], off[:, :, hi], P, s, G,
                                             op=unfold_port.deform_sapa)
            ret[rank] = "no error"
        except ValueError:
            ret[rank] = "raised"
    finally:
        dist.destroy_process_group()


def test_deform_row_sharding_refuses_a_halo_deeper_than_a_slab_on_every_rank():
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker_deform_refuse, args=(2, port, ret), nprocs=2, join=True)
        assert dict(ret) == {0: "raised", 1: "raised"}
