"""Autograd functions of SAPA-D: ``deform_qk``, ``deform_av`` and the fused ``deform_sapa_fused``.

Names, positional arguments and assertions follow ``DeformQKFunction`` / ``DeformAVFunction`` of the
reference (deformsapa/deformsapa/deform_func.py:7-114); the kernels are reached through the C ABI.
"""
from __future__ import annotations

import torch
from torch.autograd import Function

from . import _lib


def _acc_dtype(t: torch.Tensor) -> torch.dtype:
    """Scatter targets accumulate with atomics in float32 (float64 for float64 inputs)."""
    return torch.float64 if t.dtype == torch.float64 else torch.float32


def _check_offset(offset, ref_lo, num_point, scale_factor, groups):
    assert offset.size(0) == ref_lo.size(0)
    assert offset.size(1) == groups * num_point * 2
    assert offset.size(2) == ref_lo.size(2) * scale_factor
    assert offset.size(3) == ref_lo.size(3) * scale_factor
    assert num_point >= 1


def _dense_workspace_bytes(t, n, h, w, num_point, scale_factor, groups, others=()) -> int:
    """Workspace of the dense-window forward kernels for this problem, 0 when they do not apply (they need s = 2 and
    float32, or float16 / bfloat16 with rows of 16 bytes and every tensor of the call - ``t`` and ``others`` - on a
    16-byte boundary)."""
    if t.dtype not in (torch.float32, torch.float16, torch.bfloat16) or num_point > 16 or t.data_ptr() % 16 != 0:
        return 0
    if t.dtype != torch.float32 and any(o.data_ptr() % 16 != 0 for o in others):
        return 0
    return int(_lib.lib().sapa_deform_fused_forward_workspace(n, h, w, num_point, scale_factor, groups, _lib.dtype_code(t)))


def _dense_backward_bytes(t, grad_output, n, h, w, num_point, scale_factor, groups, others=(), cq=0, c=0) -> int:
    """Workspace of the dense-window backward kernels, 0 when they do not apply (they need s = 2 and float32, or
    float16 / bfloat16 with rows of 16 bytes and every tensor of the call on a 16-byte boundary; the 16-bit form adds
    float32 side buffers for the scattered gradients of ``cq`` key and ``c`` value channels)."""
    if t.dtype not in (torch.float32, torch.float16, torch.bfloat16) or num_point > 16:
        return 0
    if t.data_ptr() % 16 != 0 or grad_output.data_ptr() % 16 != 0:
        return 0
    if t.dtype == torch.float32:
        return int(_lib.lib().sapa_deform_fused_backward_workspace(n, h, w, num_point, scale_factor, groups, _lib.SAPA_F32))
    if any(o.data_ptr() % 16 != 0 for o in others):
        return 0
    code = _lib.dtype_code(t)
    base = int(_lib.lib().sapa_deform_fused_backward_workspace(n, h, w, num_point, scale_factor, groups, code))
    if not base:
        return 0
    return ((base + 15) & ~15) + int(_lib.lib().sapa_deform_fused_backward_scatter_bytes(n, cq, c, h, w, code))


class DeformQKFunction(Function):
    """out[b,g,p,qh,qw] = <query_g[b,:,qh,qw], bilinear(key_g[b], (qh/s, qw/s) + offset[b,g,p])>."""

    @staticmethod
    def forward(ctx, query, key, offset, num_point, scale_factor, groups):
        assert scale_factor >= 1
        assert query.size(0) == key.size(0)
        assert query.size(1) == key.size(1)
        assert query.size(2) == key.size(2) * scale_factor
        assert query.size(3) == key.size(3) * scale_factor
        _check_offset(offset, key, num_point, scale_factor, groups)
        assert query.size(1) % groups == 0
        if not query.is_cuda:
            raise NotImplementedError
        _lib.check_tensors(("query", query), ("key", key), ("offset", offset))
        ctx.cfg = (num_point, scale_factor, groups)
        n, c, h, w = query.shape
        out = torch.empty((n, groups, num_point, h, w), dtype=query.dtype, device=query.device)
        nbytes = _dense_workspace_bytes(query, n, key.size(2), key.size(3), num_point, scale_factor, groups, (key, offset))
        if nbytes:          # s = 2: dense 5x5 similarity of the SAPA-B kernel + bilinear combination per point
            workspace = torch.empty(nbytes, dtype=torch.uint8, device=query.device)
            _lib.call("sapa_deform_qk_forward_dense", query.device, query, key, offset, out, workspace, nbytes, n, c, key.size(2),
                      key.size(3), num_point, scale_factor, groups, _lib.dtype_code(query))
        else:
            _lib.call("sapa_deform_qk_forward", query.device, query, key, offset, out, n, c, key.size(2), key.size(3),
                      num_point, scale_factor, groups, _lib.dtype_code(query))
        if query.requires_grad or key.requires_grad or offset.requires_grad:
            ctx.save_for_backward(query, key, offset)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        assert grad_output.is_cuda
        query, key, offset = ctx.saved_tensors
        num_point, scale_factor, groups = ctx.cfg
        gq, gk, go = deform_qk_backward_raw(grad_output.contiguous(), query, key, offset, num_point, scale_factor, groups)
        return gq, gk, go, None, None, None


def deform_qk_backward_raw(grad_output, query, key, offset, num_point, scale_factor, groups):
    n, c, h, w = key.shape
    grad_offset = torch.empty_like(offset)
    nbytes = _dense_backward_bytes(query, grad_output, n, h, w, num_point, scale_factor, groups, (key, offset), cq=c)
    if nbytes:              # s = 2: SAPA-B kernels around one per-pixel kernel; the gradients have the tensors' type
        grad_query, grad_key = torch.empty_like(query), torch.empty_like(key)
        workspace = torch.empty(nbytes, dtype=torch.uint8, device=query.device)
        _lib.call("sapa_deform_qk_backward_dense", query.device, grad_output, query, key, offset, grad_query, grad_key,
                  grad_offset, workspace, nbytes, n, c, h, w, num_point, scale_factor, groups, _lib.dtype_code(query))
        return grad_query, grad_key, grad_offset
    acc = _acc_dtype(query)
    grad_query = torch.empty(query.shape, dtype=acc, device=query.device)
    grad_key = torch.empty(key.shape, dtype=acc, device=key.device)
    _lib.call("sapa_deform_qk_backward", query.device, grad_output, query, key, offset, grad_query, grad_key,
              grad_offset, n, c, h, w, num_point, scale_factor, groups, _lib.dtype_code(query))
    return grad_query.to(query.dtype), grad_key.to(key.dtype), grad_offset


deform_qk = DeformQKFunction.apply


class DeformAVFunction(Function):
    """out[b,c,qh,qw] = sum_p attn[b,g(c),p,qh,qw] * bilinear(value[b,c], (qh/s, qw/s) + offset[b,g(c),p])."""

    @staticmethod
    def forward(ctx, attn, value, offset, num_point, scale_factor, groups):
        assert scale_factor >= 1
        assert attn.size(0) == value.size(0)
        assert attn.size(1) == groups
        assert attn.size(2) == num_point
        assert attn.size(3) == value.size(2) * scale_factor
        assert attn.size(4) == value.size(3) * scale_factor
        _check_offset(offset, value, num_point, scale_factor, groups)
        if not attn.is_cuda:
            raise NotImplementedError
        _lib.check_tensors(("attn", attn), ("value", value), ("offset", offset))
        if value.size(1) % groups != 0:
            raise RuntimeError(f"value channels ({value.size(1)}) must be divisible by groups ({groups})")
        ctx.cfg = (num_point, scale_factor, groups)
        n, c, h, w = value.shape
        out = torch.empty((n, c, scale_factor * h, scale_factor * w), dtype=value.dtype, device=value.device)
        nbytes = _dense_workspace_bytes(value, n, h, w, num_point, scale_factor, groups, (attn, offset))
        if nbytes:          # s = 2: window weights per pixel + the SAPA-B aggregation kernel
            workspace = torch.empty(nbytes, dtype=torch.uint8, device=value.device)
            _lib.call("sapa_deform_av_forward_dense", value.device, attn, value, offset, out, workspace, nbytes, n, c, h, w,
                      num_point, scale_factor, groups, _lib.dtype_code(value))
        else:
            _lib.call("sapa_deform_av_forward", value.device, attn, value, offset, out, n, c, h, w, num_point, scale_factor,
                      groups, _lib.dtype_code(value))
        if attn.requires_grad or value.requires_grad or offset.requires_grad:
            ctx.save_for_backward(attn, value, offset)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        assert grad_output.is_cuda
        attn, value, offset = ctx.saved_tensors
        num_point, scale_factor, groups = ctx.cfg
        ga, gv, go = deform_av_backward_raw(grad_output.contiguous(), attn, value, offset, num_point, scale_factor, groups)
        return ga, gv, go, None, None, None


def deform_av_backward_raw(grad_output, attn, value, offset, num_point, scale_factor, groups):
    grad_attn = torch.empty_like(attn)
    grad_offset = torch.empty_like(offset)
    n, c, h, w = value.shape
    nbytes = _dense_backward_bytes(value, grad_output, n, h, w, num_point, scale_factor, groups, (attn, offset), c=c)
    if nbytes:              # the gradients have the tensors' type
        grad_value = torch.empty_like(value)
        workspace = torch.empty(nbytes, dtype=torch.uint8, device=value.device)
        _lib.call("sapa_deform_av_backward_dense", value.device, grad_output, attn, value, offset, grad_attn, grad_value,
                  grad_offset, workspace, nbytes, n, c, h, w, num_point, scale_factor, groups, _lib.dtype_code(value))
        return grad_attn, grad_value, grad_offset
    grad_value = torch.empty(value.shape, dtype=_acc_dtype(value), device=value.device)
    _lib.call("sapa_deform_av_backward", value.device, grad_output, attn, value, offset, grad_attn, grad_value,
              grad_offset, n, c, h, w, num_point, scale_factor, groups, _lib.dtype_code(value))
    return grad_attn, grad_value.to(value.dtype), grad_offset


deform_av = DeformAVFunction.apply


def deform_fused_supported(num_point: int, dtype: torch.dtype) -> bool:
    return num_point <= 16 and dtype in (torch.float32, torch.float16, torch.bfloat16)


class DeformSapaFusedFunction(Function):
    """deform_av(softmax_p(deform_qk(q, k, offset)), v, offset) as one op (``SAPADeform.attention``,
    sapa_deform.py:51-53).  The backward is one kernel too (``sapa_deform_fused_backward``): both scatter steps, the
    softmax gradient over the points between them and the sum of the two offset gradients (the offset feeds both
    ops)."""

    @staticmethod
    def forward(ctx, query, key, value, offset, num_point, scale_factor, groups):
        assert scale_factor >= 1
        assert query.size(0) == key.size(0) == value.size(0)
        assert query.size(1) == key.size(1)
        assert query.size(2) == key.size(2) * scale_factor == value.size(2) * scale_factor
        assert query.size(3) == key.size(3) * scale_factor == value.size(3) * scale_factor
        _check_offset(offset, key, num_point, scale_factor, groups)
        assert query.size(1) % groups == 0 and value.size(1) % groups == 0
        if not query.is_cuda:
            raise NotImplementedError
        _lib.check_tensors(("query", query), ("key", key), ("value", value), ("offset", offset))
        ctx.cfg = (num_point, scale_factor, groups)
        need_grad = any(ctx.needs_input_grad[:4])
        n, cq, hq, wq = query.shape
        c, h, w = value.size(1), key.size(2), key.size(3)
        if deform_fused_supported(num_point, query.dtype):
            out = torch.empty((n, c, hq, wq), dtype=value.dtype, device=value.device)
            attn = torch.empty((n, groups, num_point, hq, wq), dtype=value.dtype, device=value.device) if need_grad else None
            code = _lib.dtype_code(value)
            # s = 2: the dense-window path on the SAPA-B kernels.  float32 runs it as is; 16-bit tensors with rows of 16
            # bytes too (16-bit operands, float32 windows between the kernels); other 16-bit shapes are widened for it
            # and the results narrowed again (seven small casts against a 4x faster kernel chain).
            f32 = _lib.SAPA_F32
            aligned = all(t.data_ptr() % 16 == 0 for t in (query, key, value, offset))
            native = int(_lib.lib().sapa_deform_fused_forward_workspace(n, h, w, num_point, scale_factor, groups, code)) if aligned else 0
            nbytes = native or int(_lib.lib().sapa_deform_fused_forward_workspace(n, h, w, num_point, scale_factor, groups, f32))
            if native:
                workspace = torch.empty(nbytes, dtype=torch.uint8, device=value.device)
                _lib.call("sapa_deform_fused_forward_dense", value.device, query, key, value, offset, out, attn, workspace,
                          workspace.numel(), n, cq, c, h, w, num_point, scale_factor, groups, code)
            elif nbytes:
                workspace = torch.empty(nbytes, dtype=torch.uint8, device=value.device)
                out32 = torch.empty(out.shape, dtype=torch.float32, device=value.device)
                attn32 = torch.empty(attn.shape, dtype=torch.float32, device=value.device) if attn is not None else None
                _lib.call("sapa_deform_fused_forward_dense", value.device, query.float(), key.float(), value.float(),
                          offset.float(), out32, attn32, workspace, workspace.numel(), n, cq, c, h, w, num_point, scale_factor,
                          groups, f32)
                out.copy_(out32)
                if attn is not None:
                    attn.copy_(attn32)
            else:
                _lib.call("sapa_deform_fused_forward", value.device, query, key, value, offset, out, attn, n, cq, c, h, w,
                          num_point, scale_factor, groups, code)
        else:
            attn = torch.softmax(DeformQKFunction.apply(query.detach(), key.detach(), offset.detach(), num_point,
                                                        scale_factor, groups), dim=2)
            out = DeformAVFunction.apply(attn, value.detach(), offset.detach(), num_point, scale_factor, groups)
        if need_grad:
            ctx.save_for_backward(query, key, value, offset, attn)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        assert grad_output.is_cuda
        query, key, value, offset, attn = ctx.saved_tensors
        num_point, scale_factor, groups = ctx.cfg
        grad_output = grad_output.contiguous()
        n, cq, h, w = key.shape
        nbytes = native = 0
        if query.dtype in (torch.float32, torch.float16, torch.bfloat16) and num_point <= 16:
            tensors = (grad_output, query, key, value, offset, attn)
            if query.dtype != torch.float32 and all(t.data_ptr() % 16 == 0 for t in tensors):
                native = int(_lib.lib().sapa_deform_fused_backward_workspace(n, h, w, num_point, scale_factor, groups,
                                                                             _lib.dtype_code(query)))
            nbytes = native or int(_lib.lib().sapa_deform_fused_backward_workspace(n, h, w, num_point, scale_factor, groups,
                                                                                  _lib.SAPA_F32))
        if native:          # 16-bit tensors with rows of 16 bytes: 16-bit operands, float32 similarities, 16-bit gradients
            grad_query, grad_key, grad_value = torch.empty_like(query), torch.empty_like(key), torch.empty_like(value)
            grad_offset = torch.empty_like(offset)
            nbytes = ((native + 15) & ~15) + int(_lib.lib().sapa_deform_fused_backward_scatter_bytes(
                n, cq, value.size(1), h, w, _lib.dtype_code(query)))
            workspace = torch.empty(nbytes, dtype=torch.uint8, device=query.device)
            _lib.call("sapa_deform_fused_backward_dense", query.device, grad_output, query, key, value, offset, attn, grad_query,
                      grad_key, grad_value, grad_offset, workspace, nbytes, n, cq, value.size(1), h, w, num_point, scale_factor,
                      groups, _lib.dtype_code(query))
            return grad_query, grad_key, grad_value, grad_offset, None, None, None
        if nbytes:          # s = 2: the dense-window path on the SAPA-B kernels (float32; other 16-bit shapes are widened for it)
            dt = query.dtype
            f = (lambda t: t) if dt == torch.float32 else (lambda t: t.float())
            q32, k32, v32, o32 = f(query), f(key), f(value), f(offset)
            grad_query, grad_key, grad_value = torch.empty_like(q32), torch.empty_like(k32), torch.empty_like(v32)
            grad_offset = torch.empty_like(o32)
            workspace = torch.empty(nbytes, dtype=torch.uint8, device=query.device)
            _lib.call("sapa_deform_fused_backward_dense", query.device, f(grad_output), q32, k32, v32, o32, f(attn), grad_query,
                      grad_key, grad_value, grad_offset, workspace, nbytes, n, cq, value.size(1), h, w, num_point, scale_factor,
                      groups, _lib.SAPA_F32)
            return grad_query.to(dt), grad_key.to(dt), grad_value.to(dt), grad_offset.to(dt), None, None, None
        if deform_fused_supported(num_point, query.dtype) or (num_point <= 16 and query.dtype == torch.float64):
            acc = _acc_dtype(query)
            grad_query = torch.empty(query.shape, dtype=acc, device=query.device)
            grad_key = torch.empty(key.shape, dtype=acc, device=key.device)
            grad_value = torch.empty(value.shape, dtype=acc, device=value.device)
            grad_offset = torch.empty_like(offset)
            n, cq, h, w = key.shape
            _lib.call("sapa_deform_fused_backward", query.device, grad_output, query, key, value, offset, attn, grad_query,
                      grad_key, grad_value, grad_offset, n, cq, value.size(1), h, w, num_point, scale_factor, groups,
                      _lib.dtype_code(query))
            return (grad_query.to(query.dtype), grad_key.to(key.dtype), grad_value.to(value.dtype), grad_offset,
                    None, None, None)
        # more than 16 points: the separate backward kernels around the softmax gradient
        grad_attn, grad_value, goff_av = deform_av_backward_raw(grad_output, attn, value, offset, num_point,
                                                                scale_factor, groups)
        a32, g32 = attn.float() if attn.dtype != torch.float64 else attn, grad_attn.float() if attn.dtype != torch.float64 else grad_attn
        grad_sim = (a32 * (g32 - (a32 * g32).sum(dim=2, keepdim=True))).to(attn.dtype)
        grad_query, grad_key, goff_qk = deform_qk_backward_raw(grad_sim, query, key, offset, num_point, scale_factor, groups)
        return grad_query, grad_key, grad_value, goff_av + goff_qk, None, None, None


def deform_sapa_fused(query, key, value, offset, num_point=9, scale_factor=2, groups=4):
    """Fused SAPA-D attention; differentiable with respect to query, key, value and offset."""
    return DeformSapaFusedFunction.apply(query, key, value, offset, num_point, scale_factor, groups)
