"""Autograd functions of SAPA-B: ``qk`` (sim), ``av`` (atn) and the fused ``sapa_fused``.

``qk`` and ``av`` keep the names, positional arguments, assertions and error behaviour of the reference's
``QKFunction`` / ``AVFunction`` (sapa/sapa/sapa_func.py:9-96): AssertionError on inconsistent shapes,
NotImplementedError for CPU tensors, RuntimeError for non-contiguous tensors, ``None`` gradients for the
two integers.  They call the C ABI of ``libsapa_b200.so`` instead of the ``qk_ext`` / ``av_ext`` modules.
"""
from __future__ import annotations

import torch
from torch.autograd import Function

from . import _lib


def _check_window(kernel_size: int, scale_factor: int) -> None:
    assert scale_factor >= 1
    assert (kernel_size - 1) % 2 == 0 and kernel_size >= 1


class QKFunction(Function):
    """Local similarity: out[n, dy*K+dx, ph, pw] = <query[n,:,ph,pw], key[n,:,ph/s-r+dy, pw/s-r+dx]>."""

    @staticmethod
    def forward(ctx, query, key, kernel_size, scale_factor):
        _check_window(kernel_size, scale_factor)
        assert query.size(0) == key.size(0)
        assert query.size(-1) == key.size(-1) * scale_factor
        assert query.size(-2) == key.size(-2) * scale_factor
        if not key.is_cuda:
            raise NotImplementedError
        _lib.check_tensors(("key", key), ("query", query))
        ctx.window = (kernel_size, scale_factor)
        n, _, h, w = key.shape
        out = torch.empty((n, kernel_size ** 2, h * scale_factor, w * scale_factor), dtype=key.dtype, device=key.device)
        # channel count comes from the query, as in qk_forward_cuda (qk_cuda.cpp:50-53)
        _lib.call("sapa_qk_forward", key.device, query, key, out, n, query.size(1), h, w, kernel_size, scale_factor,
                  _lib.dtype_code(key))
        if query.requires_grad or key.requires_grad:
            ctx.save_for_backward(query, key)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        assert grad_output.is_cuda
        query, key = ctx.saved_tensors
        kernel_size, scale_factor = ctx.window
        grad_output = grad_output.contiguous()
        grad_query, grad_key = torch.empty_like(query), torch.empty_like(key)
        n, _, h, w = key.shape
        _lib.call("sapa_qk_backward", key.device, grad_output, query, key, grad_query, grad_key, n, query.size(1), h, w,
                  kernel_size, scale_factor, _lib.dtype_code(key))
        return grad_query, grad_key, None, None


qk = QKFunction.apply


class AVFunction(Function):
    """Aggregation: out[n, c, ph, pw] = sum_k attn[n, k, ph, pw] * value[n, c, window_k(ph, pw)]."""

    @staticmethod
    def forward(ctx, attn, value, kernel_size, scale_factor):
        _check_window(kernel_size, scale_factor)
        assert attn.size(1) == kernel_size * kernel_size
        assert attn.size(-1) == value.size(-1) * scale_factor
        assert attn.size(-2) == value.size(-2) * scale_factor
        if not value.is_cuda:
            raise NotImplementedError
        _lib.check_tensors(("value", value), ("attn", attn))
        ctx.window = (kernel_size, scale_factor)
        n, c, h, w = value.shape
        out = torch.empty((n, c, h * scale_factor, w * scale_factor), dtype=value.dtype, device=value.device)
        _lib.call("sapa_av_forward", value.device, attn, value, out, n, c, h, w, kernel_size, scale_factor,
                  _lib.dtype_code(value))
        if attn.requires_grad or value.requires_grad:
            ctx.save_for_backward(attn, value)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        assert grad_output.is_cuda
        attn, value = ctx.saved_tensors
        kernel_size, scale_factor = ctx.window
        grad_output = grad_output.contiguous()
        grad_attn, grad_value = torch.empty_like(attn), torch.empty_like(value)
        n, c, h, w = value.shape
        _lib.call("sapa_av_backward", value.device, grad_output, attn, value, grad_attn, grad_value, n, c, h, w,
                  kernel_size, scale_factor, _lib.dtype_code(value))
        return grad_attn, grad_value, None, None


av = AVFunction.apply


def fused_supported(kernel_size: int, scale_factor: int, dtype: torch.dtype) -> bool:
    """True when ``sapa_fused_forward`` has a single-kernel implementation for this configuration."""
    return scale_factor == 2 and kernel_size in (3, 5) and dtype in (torch.float32, torch.float16, torch.bfloat16)


def fused_forward_raw(query, key, value, kernel_size, scale_factor, want_attn, halo=(0, 0)):
    """Run the fused kernel; returns (out, attn or None).  ``halo`` = extra key/value rows (top, bottom)."""
    query, key, value = _lib.aligned(query), _lib.aligned(key), _lib.aligned(value)
    n, d, hq, wq = query.shape
    c = value.size(1)
    h, w = hq // scale_factor, wq // scale_factor
    out = torch.empty((n, c, hq, wq), dtype=value.dtype, device=value.device)
    attn = torch.empty((n, kernel_size ** 2, hq, wq), dtype=value.dtype, device=value.device) if want_attn else None
    _lib.call("sapa_fused_forward_slab", value.device, query, key, value, out, attn, n, d, c, h, w, halo[0], halo[1],
              kernel_size, scale_factor, _lib.dtype_code(value))
    return out, attn


class SapaFusedFunction(Function):
    """atn(softmax(sim(query, key)), value) as one op (the whole of ``SAPA.attention``, sapa_base.py:38-40).

    With a fused kernel available the attention map stays in registers (it is written once, for the backward
    pass, only when a gradient is required); otherwise the three separate kernels run.
    """

    @staticmethod
    def forward(ctx, query, key, value, kernel_size, scale_factor):
        _check_window(kernel_size, scale_factor)
        assert query.size(0) == key.size(0) == value.size(0)
        assert query.size(1) == key.size(1)
        assert query.size(-1) == key.size(-1) * scale_factor == value.size(-1) * scale_factor
        assert query.size(-2) == key.size(-2) * scale_factor == value.size(-2) * scale_factor
        if not value.is_cuda:
            raise NotImplementedError
        _lib.check_tensors(("value", value), ("query", query), ("key", key))
        ctx.window = (kernel_size, scale_factor)
        need_grad = any(ctx.needs_input_grad[:3])
        if fused_supported(kernel_size, scale_factor, value.dtype):
            out, attn = fused_forward_raw(query, key, value, kernel_size, scale_factor, need_grad)
        else:
            attn = torch.softmax(QKFunction.apply(query.detach(), key.detach(), kernel_size, scale_factor), dim=1)
            out = AVFunction.apply(attn, value.detach(), kernel_size, scale_factor)
        if need_grad:
            ctx.save_for_backward(query, key, value, attn)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        assert grad_output.is_cuda
        query, key, value, attn = ctx.saved_tensors
        kernel_size, scale_factor = ctx.window
        grad_output = grad_output.contiguous()
        n, d, h, w = key.shape
        c = value.size(1)
        code = _lib.dtype_code(value)
        nbytes = _lib.fused_backward_workspace(n, h, w, kernel_size, scale_factor, code)
        workspace = torch.empty(nbytes, dtype=torch.uint8, device=value.device)
        grad_query, grad_key, grad_value = torch.empty_like(query), torch.empty_like(key), torch.empty_like(value)
        _lib.call("sapa_fused_backward", value.device, grad_output, query, key, value, attn, grad_query, grad_key,
                  grad_value, workspace, nbytes, n, d, c, h, w, kernel_size, scale_factor, code)
        return grad_query, grad_key, grad_value, None, None


def sapa_fused(query, key, value, kernel_size=5, scale_factor=2):
    """Fused SAPA-B attention; differentiable with respect to query, key and value."""
    return SapaFusedFunction.apply(query, key, value, kernel_size, scale_factor)


def _nhwc_forward(query, key, value, kernel_size, scale_factor, return_attn):
    _lib.check_tensors(("value", value), ("query", query), ("key", key))
    n, hq, wq, d = query.shape
    h, w, c = value.shape[1:]
    assert key.shape == (n, h, w, d) and hq == h * scale_factor and wq == w * scale_factor
    query, key, value = _lib.aligned(query), _lib.aligned(key), _lib.aligned(value)
    out = torch.empty((n, hq, wq, c), dtype=value.dtype, device=value.device)
    attn = torch.empty((n, hq, wq, kernel_size ** 2), dtype=value.dtype, device=value.device) if return_attn else None
    _lib.call("sapa_fused_forward_nhwc", value.device, query, key, value, out, attn, n, d, c, h, w, kernel_size, scale_factor,
              _lib.dtype_code(value))
    return out, attn


class _SapaFusedNhwcFunction(Function):
    """Channels-last forward kernel; the backward goes through the channels-first kernels: the saved tensors and the
    incoming gradient are permuted to [B, C, H, W], the fused forward is run again there for its attention map, the
    fused backward follows, and the three gradients are permuted back (five layout copies and one forward more than a
    native channels-last backward would need)."""

    @staticmethod
    def forward(ctx, query, key, value, kernel_size, scale_factor):
        out, _ = _nhwc_forward(query, key, value, kernel_size, scale_factor, False)
        if any(ctx.needs_input_grad[:3]):
            ctx.cfg = (kernel_size, scale_factor)
            ctx.save_for_backward(query, key, value)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        query, key, value = ctx.saved_tensors
        kernel_size, scale_factor = ctx.cfg
        first = [t.detach().permute(0, 3, 1, 2).contiguous().requires_grad_() for t in (query, key, value)]
        with torch.enable_grad():
            out = SapaFusedFunction.apply(first[0], first[1], first[2], kernel_size, scale_factor)
        grads = torch.autograd.grad(out, first, grad_out.permute(0, 3, 1, 2).contiguous())
        gq, gk, gv = (g.permute(0, 2, 3, 1).contiguous() for g in grads)
        return gq, gk, gv, None, None


def sapa_fused_nhwc(query, key, value, kernel_size=5, scale_factor=2, return_attn=False):
    """Fused SAPA-B on channels-last tensors: ``query`` [B, sH, sW, d], ``key`` [B, H, W, d], ``value`` [B, H, W, C] ->
    [B, sH, sW, C] (plus the attention [B, sH, sW, K*K] when ``return_attn``, which is not differentiable).  The forward
    is the channels-last kernel; gradients are computed by the channels-first kernels around layout copies (see
    ``_SapaFusedNhwcFunction``).  The reference has no channels-last path."""
    if not value.is_cuda:
        raise NotImplementedError
    needs_grad = torch.is_grad_enabled() and any(t.requires_grad for t in (query, key, value))
    if return_attn:
        if needs_grad:
            raise NotImplementedError("sapa_fused_nhwc(return_attn=True) is forward only")
        return _nhwc_forward(query, key, value, kernel_size, scale_factor, True)
    if needs_grad:
        return _SapaFusedNhwcFunction.apply(query, key, value, kernel_size, scale_factor)
    return _nhwc_forward(query, key, value, kernel_size, scale_factor, False)[0]
