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
        ret[rank] = bool(torch.equal(mine, full[:, :, s * rows.start:s * rows.stop]))
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
