"""Multi-GPU sharding of the SAPA-B attention: one process per GPU, ``torch.distributed`` for the plumbing.

* Batch sharding needs no communication at all: images are independent in every kernel, so each rank runs
  the ordinary ops on its slice of the batch (:func:`batch_slice`).
* Row-slab sharding splits ONE image by low-res rows.  Output row ``ph`` reads key/value rows
  ``ph/s - r .. ph/s + r`` (r = (K-1)/2), so each rank needs r halo rows of key and value from each
  neighbour; the image's own top and bottom are zero padding.  :class:`RowSlab` keeps a rank's key and value
  resident in padded buffers (the halo rows are part of the buffer, so nothing is copied but the halo itself),
  exchanges the 2 x r rows per step as one point-to-point message per neighbour (NCCL send/recv over NVLink on
  GPUs, gloo on CPU) on a side stream, and meanwhile computes the rows that need no halo; the two border bands
  follow when the halos have arrived.  Nothing spins on the device and no kernel reads another GPU's memory.

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


def check_row_split(local_rows: int, halo: int, group=None) -> None:
    """Every rank must own at least ``halo`` rows (a halo comes from the direct neighbour only).  The decision is
    taken from the shares of ALL ranks, so that either every rank raises or none does: a rank that raised alone
    would leave its neighbour waiting in a receive."""
    if not dist.is_initialized():
        return
    world = dist.get_world_size(group)
    if world == 1 or halo == 0:
        return
    shares = [None] * world
    dist.all_gather_object(shares, int(local_rows), group=group)
    if min(shares) < halo:
        raise ValueError(f"row-slab sharding with a halo of {halo} rows needs at least {halo} rows on every rank, "
                         f"got shares {shares}")


def _exchange_into(padded, halo: int, group=None) -> None:
    """Fill the halo rows of the padded slabs ``[B, C_i, halo + Hl + halo, W]`` in place: the top ``halo`` rows come
    from the rank above, the bottom ones from the rank below; the halos of the first / last rank at the image border
    are left as they are (zero).  The slabs' halos travel packed in ONE message per neighbour."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    if halo == 0 or world == 1:
        return
    first = padded[0]
    B, _, Hp, W = first.shape
    Hl = Hp - 2 * halo
    chans = [t.size(1) for t in padded]
    ctot = sum(chans)
    to_global = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)

    def pack(lo: int) -> torch.Tensor:        # rows lo .. lo+halo of every slab, channels concatenated
        return torch.cat([t[:, :, lo:lo + halo, :] for t in padded], dim=1).contiguous()

    ops, from_up, from_down = [], None, None
    if rank > 0:
        from_up = first.new_empty((B, ctot, halo, W))
        ops.append(dist.P2POp(dist.isend, pack(halo), to_global(rank - 1), group))
        ops.append(dist.P2POp(dist.irecv, from_up, to_global(rank - 1), group))
    if rank < world - 1:
        from_down = first.new_empty((B, ctot, halo, W))
        ops.append(dist.P2POp(dist.isend, pack(Hl), to_global(rank + 1), group))
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


def _reduce_halo_grads(padded, halo: int, group=None) -> None:
    """Backward counterpart of :func:`_exchange_into` for gradients in the padded frame ``[B, C_i, halo + Hl + halo, W]``:
    the halo rows hold this rank's contribution to the neighbours' edge rows.  They are sent to the neighbours (one
    message each) and what arrives from them is added to this rank's own first / last ``halo`` rows, in place."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    if halo == 0 or world == 1:
        return
    first = padded[0]
    B, _, Hp, W = first.shape
    Hl = Hp - 2 * halo
    chans = [t.size(1) for t in padded]
    ctot = sum(chans)
    to_global = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)

    def pack(lo: int) -> torch.Tensor:
        return torch.cat([t[:, :, lo:lo + halo, :] for t in padded], dim=1).contiguous()

    ops, from_up, from_down = [], None, None
    if rank > 0:
        from_up = first.new_empty((B, ctot, halo, W))
        ops.append(dist.P2POp(dist.isend, pack(0), to_global(rank - 1), group))           # my top halo -> its last rows
        ops.append(dist.P2POp(dist.irecv, from_up, to_global(rank - 1), group))
    if rank < world - 1:
        from_down = first.new_empty((B, ctot, halo, W))
        ops.append(dist.P2POp(dist.isend, pack(halo + Hl), to_global(rank + 1), group))   # my bottom halo -> its first rows
        ops.append(dist.P2POp(dist.irecv, from_down, to_global(rank + 1), group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    c0 = 0
    for p, c in zip(padded, chans):
        if from_up is not None:
            p[:, :, halo:2 * halo, :] += from_up[:, c0:c0 + c]
        if from_down is not None:
            p[:, :, Hl:Hl + halo, :] += from_down[:, c0:c0 + c]
        c0 += c


def exchange_row_halo(tensors, halo: int, group=None):
    """Pad each local slab [B,C,Hl,W] to [B,C,halo+Hl+halo,W] with rows of the neighbouring ranks.

    ``tensors`` is a list of slabs that share B, Hl, W, dtype and device (e.g. key and value).  Rank 0's top halo
    and the last rank's bottom halo stay zero, which is the zero padding of the unsharded op.  Returns the list of
    padded slabs.  This convenience form copies the slabs; a caller that runs many steps keeps its key / value in a
    :class:`RowSlab` instead, where only the halo rows move.
    """
    if halo == 0:
        return list(tensors)
    Hl = tensors[0].size(2)
    check_row_split(Hl, halo, group)
    padded = [_pad_rows(t, halo) for t in tensors]
    _exchange_into(padded, halo, group)
    return padded


def _pad_rows(t: torch.Tensor, halo: int) -> torch.Tensor:
    """[B,C,Hl,W] -> [B,C,halo+Hl+halo,W] with zero halo rows (only the halo rows are cleared: one pass over the slab)."""
    Hl = t.size(2)
    p = t.new_empty((t.size(0), t.size(1), Hl + 2 * halo, t.size(3)))
    p[:, :, :halo, :] = 0
    p[:, :, halo + Hl:, :] = 0
    p[:, :, halo:halo + Hl, :] = t
    return p


class RowSlab:
    """One rank's share of a row-sharded fused SAPA-B forward.

    ``key`` and ``value`` are views of the interior rows of padded buffers allocated once; whoever produces the key
    and value of this rank writes them there (no copy per step).  :meth:`forward` then
      1. starts the halo exchange on a side stream (pack 2 x r edge rows, one send + one receive per neighbour,
         unpack into the halo rows of the padded buffers),
      2. computes, on the caller's stream, the output rows whose windows stay inside the rank's own rows,
      3. waits for the exchange and computes the top and bottom bands.
    The result equals the matching rows of the unsharded ``sapa_fused`` bit for bit.

    :meth:`backward` (after a ``forward(..., keep_attn=True)``) returns the gradients of the rank's query, key and value
    rows: the slab backward kernel produces the key / value gradients in the padded frame, the halo rows (this rank's
    contribution to its neighbours' edge rows) travel to the neighbours and what arrives is added to the rank's own
    edge rows - a 2 x r row reduction per step.
    """

    BAND = 4          # low-res rows per border band (a multiple of the kernels' tile heights, >= the halo)

    def __init__(self, batch, channels_qk, channels_v, local_rows, width, dtype, device, kernel_size=5, scale_factor=2,
                 group=None):
        from .functions import fused_supported
        if not fused_supported(kernel_size, scale_factor, dtype):
            raise NotImplementedError("row-slab sharding needs the fused kernel (K in {3,5}, s = 2, f32/f16/bf16)")
        self.K, self.s, self.group = kernel_size, scale_factor, group
        self.halo = (kernel_size - 1) // 2
        self.B, self.d, self.C, self.Hl, self.W = batch, channels_qk, channels_v, local_rows, width
        check_row_split(local_rows, self.halo, group)
        rows = local_rows + 2 * self.halo
        self.key_padded = torch.zeros((batch, channels_qk, rows, width), dtype=dtype, device=device)
        self.value_padded = torch.zeros((batch, channels_v, rows, width), dtype=dtype, device=device)
        self.key = self.key_padded[:, :, self.halo:self.halo + local_rows, :]
        self.value = self.value_padded[:, :, self.halo:self.halo + local_rows, :]
        self._side = torch.cuda.Stream(device=device) if torch.device(device).type == "cuda" else None
        self._halo_done = torch.cuda.Event() if self._side is not None else None
        self.attn = None            # [B, K*K, s*Hl, s*W] of the last forward(keep_attn=True)

    def _launch(self, query, out, row_begin, row_end):
        from . import _lib
        return _lib.call("sapa_fused_forward_slab_rows", out.device, query, self.key_padded, self.value_padded, out, self.attn,
                         self.B, self.d, self.C, self.Hl, self.W, self.halo, self.halo, row_begin, row_end, self.K, self.s,
                         _lib.dtype_code(out), allow_unsupported=True)

    def forward(self, query, out=None, keep_attn=False):
        """``query`` [B, d, s*Hl, s*W] -> ``out`` [B, C, s*Hl, s*W] (allocated when not given).  ``keep_attn`` stores the
        attention map of the slab for :meth:`backward`."""
        from . import _lib
        s, Hl = self.s, self.Hl
        if keep_attn and self.attn is None:
            self.attn = torch.empty((self.B, self.K * self.K, s * Hl, s * self.W), dtype=self.value_padded.dtype,
                                    device=self.value_padded.device)
        elif not keep_attn:
            self.attn = None
        if out is None:
            out = torch.empty((self.B, self.C, s * Hl, s * self.W), dtype=self.value_padded.dtype, device=query.device)
        query = _lib.aligned(query.contiguous())
        band = self.BAND
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        overlap = self._side is not None and world > 1 and Hl > 2 * band
        if overlap:
            main = torch.cuda.current_stream(query.device)
            self._side.wait_stream(main)                        # key / value of this step are complete
            with torch.cuda.stream(self._side):
                _exchange_into([self.key_padded, self.value_padded], self.halo, self.group)
                self._halo_done.record(self._side)
            status = self._launch(query, out, band, Hl - band)  # rows that read no halo, under the exchange
            main.wait_event(self._halo_done)
            if status == 0:
                self._launch(query, out, 0, band)
                self._launch(query, out, Hl - band, Hl)
                return out
        elif world > 1:
            _exchange_into([self.key_padded, self.value_padded], self.halo, self.group)
        status = self._launch(query, out, 0, Hl)               # one launch over the whole slab
        if status != 0:
            raise RuntimeError("sapa_fused_forward_slab_rows: " + _lib.lib().sapa_last_error().decode("utf-8", "replace"))
        return out


    def backward(self, grad_out, query):
        """Gradients ``(grad_query, grad_key, grad_value)`` of this rank's rows from ``grad_out`` [B, C, s*Hl, s*W]; needs
        the attention map of ``forward(query, keep_attn=True)`` and the same key / value still in the slab."""
        from . import _lib
        if self.attn is None:
            raise RuntimeError("RowSlab.backward needs forward(..., keep_attn=True) first")
        query, grad_out = _lib.aligned(query.contiguous()), _lib.aligned(grad_out.contiguous())
        code = _lib.dtype_code(grad_out)
        grad_query = torch.empty_like(query)
        grad_key = torch.empty_like(self.key_padded)
        grad_value = torch.empty_like(self.value_padded)
        nbytes = _lib.fused_backward_workspace(self.B, self.Hl, self.W, self.K, self.s, code)
        workspace = torch.empty(nbytes, dtype=torch.uint8, device=grad_out.device)
        _lib.call("sapa_fused_backward_slab", grad_out.device, grad_out, query, self.key_padded, self.value_padded, self.attn,
                  grad_query, grad_key, grad_value, workspace, nbytes, self.B, self.d, self.C, self.Hl, self.W, self.halo,
                  self.halo, self.K, self.s, code)
        if dist.is_initialized():
            _reduce_halo_grads([grad_key, grad_value], self.halo, self.group)
        own = slice(self.halo, self.halo + self.Hl)
        return grad_query, grad_key[:, :, own, :], grad_value[:, :, own, :]


class _RowShardedFused(torch.autograd.Function):
    """Differentiable form of the row-sharded op: forward = halo exchange + slab kernel, backward = slab backward +
    reduction of the halo-row gradients across the neighbouring ranks."""

    @staticmethod
    def forward(ctx, query, key, value, kernel_size, scale_factor, group):
        slab = RowSlab(key.size(0), key.size(1), value.size(1), key.size(2), key.size(3), value.dtype, value.device,
                       kernel_size, scale_factor, group)
        slab.key.copy_(key)
        slab.value.copy_(value)
        need_grad = any(ctx.needs_input_grad[:3])
        out = slab.forward(query, keep_attn=need_grad)
        if need_grad:
            ctx.slab = slab
            ctx.save_for_backward(query)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (query,) = ctx.saved_tensors
        grad_query, grad_key, grad_value = ctx.slab.backward(grad_out, query)
        return grad_query, grad_key.contiguous(), grad_value.contiguous(), None, None, None


def sapa_fused_row_sharded(query, key, value, kernel_size=5, scale_factor=2, group=None):
    """Fused SAPA-B on this rank's row slab (one-shot form: builds a :class:`RowSlab` and copies key / value in).

    ``query`` [B,d,s*Hl,s*W], ``key`` [B,d,Hl,W], ``value`` [B,C,Hl,W] hold the rank's rows of one larger
    image; the result equals the same rows of the unsharded ``sapa_fused``, and so do the gradients (every rank must
    run the backward pass: it exchanges halo-row gradients with the neighbours).
    """
    return _RowShardedFused.apply(query, key, value, kernel_size, scale_factor, group)


# ---------------------------------------------------------------------------------------------- SAPA-D row slabs

class _HaloPad(torch.autograd.Function):
    """[B,C_i,Hl,W] slabs -> [B,C_i,halo+Hl+halo,W] with the neighbours' rows in the halos (zeros at the image border).
    Backward: the halo rows of the gradients go back to the neighbours and are added to their edge rows."""

    @staticmethod
    def forward(ctx, halo, group, *tensors):
        ctx.halo, ctx.group = halo, group
        padded = [_pad_rows(t, halo) for t in tensors]         # the caller has checked the shares of all ranks
        _exchange_into(padded, halo, group)
        return tuple(padded)

    @staticmethod
    def backward(ctx, *grads):
        halo = ctx.halo
        padded = [g.contiguous().clone() for g in grads]
        if dist.is_initialized():
            _reduce_halo_grads(padded, halo, ctx.group)
        Hl = padded[0].size(2) - 2 * halo
        return (None, None) + tuple(p[:, :, halo:halo + Hl, :].contiguous() for p in padded)


def deform_halo_rows(offset: torch.Tensor, group=None, local_rows=None) -> int:
    """Halo depth (low-res rows) that makes row-slab sharding of SAPA-D exact for these offsets.

    A sampling point of a pixel with parent row y lies at row y + oy and reads rows floor(y + oy) and floor(y + oy) + 1
    (deform_qk_cuda_kernel.cu:159-170 of the reference: bilinear corners of ``h = qh / s + offset_y``), so with
    m = max |oy| over every rank no tap leaves ``floor(m) + 1`` rows beyond a slab.  The y offsets are the odd
    channels of ``offset`` (x first, then y, per sampling point).  One device reduction, one MAX all-reduce and one
    host read: the depth must be the same on every rank.  With ``local_rows`` (this rank's share of rows) the same
    all-reduce also carries the smallest share, and a depth beyond it raises ``ValueError`` on every rank together
    (a halo comes from the direct neighbour only).
    """
    if offset.numel():
        lo, hi = torch.aminmax(offset.detach()[:, 1::2])            # one pass, no temporary
        m = torch.maximum(-lo, hi).to(torch.float32).reshape(1)
    else:
        m = offset.new_zeros(1, dtype=torch.float32)
    rows = m.new_full((1,), -float(local_rows) if local_rows is not None else -float("inf"))
    both = torch.cat([m, rows])                                     # MAX of (-rows) = -(smallest share)
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world > 1:
        dist.all_reduce(both, op=dist.ReduceOp.MAX, group=group)
    m, min_rows = float(both[0].item()), -float(both[1].item())
    if not m < float("inf"):
        raise ValueError("SAPA-D row-slab sharding: the offsets hold a non-finite value")
    depth = int(m) + 1
    if world > 1 and depth > min_rows:
        raise ValueError(f"SAPA-D row-slab sharding: the offsets reach {depth} rows beyond a slab but the smallest slab has "
                         f"{int(min_rows)} rows; shard by batch or gather the image instead")
    return depth


def _deform_slab_forward(query, key, value, offset, num_point, s, groups, halo, group):
    """Inference path of :func:`sapa_deform_row_sharded`: only key and value get halo rows, the kernels take the slab
    form (``sapa_deform_fused_forward_slab``), so query, offsets and output stay as they are and no row is computed
    twice.  Returns None when the dense-window kernels do not cover the configuration (the caller pads instead)."""
    from . import _lib
    from .deform_functions import _dense_workspace_bytes
    B, d, Hl, W = key.shape
    C = value.size(1)
    if not query.is_cuda:
        return None
    nbytes = _dense_workspace_bytes(query, B, Hl, W, num_point, s, groups, (key, value, offset))
    if not nbytes or (W * query.element_size()) % 16 != 0:
        return None
    key_p, value_p = _pad_rows(key, halo), _pad_rows(value, halo)
    _exchange_into([key_p, value_p], halo, group)
    query, offset = query.contiguous(), offset.contiguous()
    _lib.check_tensors(("query", query), ("key", key_p), ("value", value_p), ("offset", offset))
    out = torch.empty((B, C, s * Hl, s * W), dtype=value.dtype, device=value.device)
    workspace = torch.empty(nbytes, dtype=torch.uint8, device=query.device)
    _lib.call("sapa_deform_fused_forward_slab", query.device, query, key_p, value_p, offset, out, None, workspace, nbytes,
              B, d, C, Hl, W, halo, halo, num_point, s, groups, _lib.dtype_code(query))
    return out


def sapa_deform_row_sharded(query, key, value, offset, num_point=9, scale_factor=2, groups=4, group=None, halo=None,
                            op=None):
    """Fused SAPA-D on this rank's row slab of one larger image; equals the same rows of the unsharded op.

    ``query`` [B,d,s*Hl,s*W], ``key`` [B,d,Hl,W], ``value`` [B,C,Hl,W], ``offset`` [B,2*groups*num_point,s*Hl,s*W]
    hold the rank's rows.  The offsets are unbounded, so the halo depth is data-dependent: ``halo=None`` measures it
    (:func:`deform_halo_rows`, one host read per call); a caller that bounds its offsets passes the bound's depth
    instead.  Every rank must own at least ``halo`` rows (``ValueError`` on all ranks together otherwise: fall back to
    batch sharding or gather the image).  The slab, padded with the neighbours' rows - zeros at the image's own top
    and bottom, which sample exactly like the reference's dropped corners and its outside-the-image guard - goes to
    the kernels in one of two ways.  No gradient needed (float32, s = 2): the slab form of the dense-window kernels,
    where only key and value carry halo rows.  Otherwise the padded slab is run as an image of its own with zero
    query / offset rows over the halo, and the halo rows are cut from the result (2*halo / (Hl + 2*halo) of the work is
    thrown away, the price of reusing the single-GPU autograd function unchanged); the backward pass returns the
    halo-row gradients of key and value to the neighbours (every rank must run it).

    ``op`` replaces the per-slab operator (default :func:`sapa_b200.deform_sapa_fused`); the CPU tests pass a
    PyTorch transcription.
    """
    from .deform_functions import deform_sapa_fused
    if op is None:
        op = deform_sapa_fused
    s = scale_factor
    Hl = key.size(2)
    if halo is None:
        halo = deform_halo_rows(offset, group, local_rows=Hl)       # checks the shares of all ranks in the same all-reduce
    else:
        check_row_split(Hl, halo, group)
    if halo == 0 or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return op(query, key, value, offset, num_point, s, groups)
    if op is deform_sapa_fused and not (torch.is_grad_enabled() and any(t.requires_grad for t in (query, key, value, offset))):
        fast = _deform_slab_forward(query, key, value, offset, num_point, s, groups, halo, group)
        if fast is not None:
            return fast
    key_p, value_p = _HaloPad.apply(halo, group, key, value)
    pad = (0, 0, s * halo, s * halo)
    query_p = torch.nn.functional.pad(query, pad)
    offset_p = torch.nn.functional.pad(offset, pad)
    out = op(query_p.contiguous(), key_p, value_p, offset_p.contiguous(), num_point, s, groups)
    return out[:, :, s * halo:s * (halo + Hl), :]


class DeformRowSlab:
    """A rank's row slab of ONE image for repeated SAPA-D forward passes (inference): key and value live in buffers
    padded with ``max_halo`` rows above and below, so that a step moves nothing but the halo rows.

    ``slab.key`` [B,d,Hl,W] and ``slab.value`` [B,C,Hl,W] are views of the rank's own rows: the producer writes them
    in place.  :meth:`forward` exchanges ``halo`` rows with the neighbours (``halo=None``: measured from the offsets,
    one host read; a caller whose offsets are bounded - a clamp or a tanh in front of the op - passes the bound's depth
    and the step stays asynchronous), and runs the slab form of the dense-window kernels on the rank's own query /
    offset rows.  Every rank must own at least ``max_halo`` rows (checked once, here, on all ranks together); a step
    whose depth exceeds ``max_halo`` raises ``ValueError`` on every rank (the depth is the same everywhere).
    Scale factor 2; float32, or float16 / bfloat16 with rows of 16 bytes (the dense-window kernels).  The reference has
    no multi-device code.
    """

    def __init__(self, batch, channels_qk, channels_v, local_rows, width, max_halo, device, num_point=9, groups=4,
                 group=None, dtype=torch.float32):
        if max_halo < 2:
            raise ValueError("max_halo must be at least 2 (the 5 x 5 window of the dense similarity)")
        check_row_split(local_rows, max_halo, group)
        self.group, self.cap, self.rows, self.width = group, int(max_halo), int(local_rows), int(width)
        self.num_point, self.groups = num_point, groups
        rows = local_rows + 2 * self.cap
        self.dtype = dtype
        self.key_padded = torch.zeros((batch, channels_qk, rows, width), dtype=dtype, device=device)
        self.value_padded = torch.zeros((batch, channels_v, rows, width), dtype=dtype, device=device)
        self.key = self.key_padded[:, :, self.cap:self.cap + local_rows, :]
        self.value = self.value_padded[:, :, self.cap:self.cap + local_rows, :]
        self._workspace = None

    def forward(self, query, offset, halo=None, out=None):
        from . import _lib
        B, d = self.key_padded.shape[:2]
        C, Hl, W, P, G, s = self.value_padded.size(1), self.rows, self.width, self.num_point, self.groups, 2
        if halo is None:
            halo = deform_halo_rows(offset, self.group)
        if halo > self.cap:
            raise ValueError(f"the offsets reach {halo} rows beyond the slab, the buffers hold {self.cap}")
        depth = max(int(halo), 2)            # the dense similarity always reads the two window rows above and below
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            lo, hi = self.cap - depth, self.cap + Hl + depth
            _exchange_into([self.key_padded[:, :, lo:hi, :], self.value_padded[:, :, lo:hi, :]], depth, self.group)
        _lib.check_tensors(("query", query), ("key", self.key_padded), ("value", self.value_padded), ("offset", offset))
        code = _lib.dtype_code(self.key_padded)
        nbytes = int(_lib.lib().sapa_deform_fused_forward_workspace(B, Hl, W, P, s, G, code))
        if nbytes == 0:
            raise RuntimeError("DeformRowSlab needs float32 (or float16 / bfloat16 with rows of 16 bytes) and at most 16 points")
        if self._workspace is None or self._workspace.numel() < nbytes:
            self._workspace = torch.empty(nbytes, dtype=torch.uint8, device=query.device)
        if out is None:
            out = torch.empty((B, C, s * Hl, s * W), dtype=self.dtype, device=query.device)
        _lib.call("sapa_deform_fused_forward_slab", query.device, query, self.key_padded, self.value_padded, offset, out, None,
                  self._workspace, nbytes, B, d, C, Hl, W, self.cap, self.cap, P, s, G, code)
        return out
