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
