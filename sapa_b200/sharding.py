"""Multi-GPU sharding of the SAPA-B attention: one process per GPU, ``torch.distributed`` for the plumbing.

* Batch sharding needs no communication at all: images are independent in every kernel, so each rank runs
  the ordinary ops on its slice of the batch (:func:`batch_slice`).
* Row-slab sharding splits ONE image by low-res rows.  Output row ``ph`` reads key/value rows
  ``ph/s - r .. ph/s + r`` (r = (K-1)/2), so each rank needs r halo rows of key and value from each
  neighbour; the image's own top and bottom are zero padding.  The halos travel as one point-to-point
  message per neighbour (NCCL send/recv over NVLink on GPUs, gloo on CPU); the fused kernel then reads the
  padded slab through ``sapa_fused_forward_slab``.  Nothing spins on the device.

The reference has no multi-device code; this module has no counterpart there.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def batch_slice(batch: int, world_size: int, rank: int) -> slice:
    """Contiguous share of ``batch`` images for ``rank`` (sizes differ by at most one)."""
    base, extra = divmod(batch, world_size)
    start = rank * base + min(rank, extra)
    return slice(start, start + base + (1 if rank < extra else 0))


def row_slice(rows: int, world_size: int, rank: int) -> slice:
    """Contiguous share of ``rows`` low-res rows for ``rank``."""
    return batch_slice(rows, world_size, rank)


def exchange_row_halo(tensors, halo: int, group=None):
    """Pad each local slab [B,C,Hl,W] to [B,C,halo+Hl+halo,W] with rows of the neighbouring ranks.

    ``tensors`` is a list of slabs that share B, Hl, W, dtype and device (e.g. key and value); their halos are
    packed into ONE message per neighbour.  Rank 0's top halo and the last rank's bottom halo stay zero,
    which is the zero padding of the unsharded op.  Returns the list of padded slabs.
    """
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    first = tensors[0]
    B, _, Hl, W = first.shape
    if halo == 0:
        return list(tensors)
    if Hl < halo:
        raise ValueError(f"each rank needs at least {halo} rows, got {Hl}")
    chans = [t.size(1) for t in tensors]
    ctot = sum(chans)

    def pack(rows: slice) -> torch.Tensor:
        return torch.cat([t[:, :, rows, :] for t in tensors], dim=1).contiguous()

    padded = [t.new_zeros((B, c, Hl + 2 * halo, W)) for t, c in zip(tensors, chans)]
    for p, t in zip(padded, tensors):
        p[:, :, halo:halo + Hl, :] = t
    ops, from_up, from_down = [], None, None
    to_global = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)
    if rank > 0:
        from_up = first.new_empty((B, ctot, halo, W))
        ops.append(dist.P2POp(dist.isend, pack(slice(0, halo)), to_global(rank - 1), group))
        ops.append(dist.P2POp(dist.irecv, from_up, to_global(rank - 1), group))
    if rank < world - 1:
        from_down = first.new_empty((B, ctot, halo, W))
        ops.append(dist.P2POp(dist.isend, pack(slice(Hl - halo, Hl)), to_global(rank + 1), group))
        ops.append(dist.P2POp(dist.irecv, from_down, to_global(rank + 1), group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    c0 = 0
    for p, c in zip(padded, chans):
        if from_up is not None:
            p[:, :, :halo, :] = from_up[:, c0:c0 + c]
        if from_down is not None:
            p[:, :, halo + Hl:, :] = from_down[:, c0:c0 + c]
        c0 += c
    return padded


def sapa_fused_row_sharded(query, key, value, kernel_size=5, scale_factor=2, group=None):
    """Fused SAPA-B forward on this rank's row slab.

    ``query`` [B,d,s*Hl,s*W], ``key`` [B,d,Hl,W], ``value`` [B,C,Hl,W] hold the rank's rows of one larger
    image; the result equals the same rows of the unsharded ``sapa_fused``.  Forward only.
    """
    from .functions import fused_forward_raw, fused_supported

    if not fused_supported(kernel_size, scale_factor, value.dtype):
        raise NotImplementedError("row-slab sharding needs the fused kernel (K in {3,5}, s = 2, f32/f16/bf16)")
    halo = (kernel_size - 1) // 2
    key_p, value_p = exchange_row_halo([key, value], halo, group)
    out, _ = fused_forward_raw(query.contiguous(), key_p, value_p, kernel_size, scale_factor, False, halo=(halo, halo))
    return out
