"""``SAPA`` and ``SAPADeform``: the upsampling modules of the reference with the same constructor arguments
and parameter names, so that reference checkpoints load unchanged (``norm_y.*``, ``norm_x.*``, ``q.*``,
``k.*`` and ``offset.*``; sapa_base.py:7-49, sapa_deform.py:7-62).

One extra keyword, ``impl``: ``"fused"`` (default) runs the attention as one kernel, ``"separate"`` keeps the
reference's three steps ``qk -> F.softmax -> av`` on this library's kernels.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .deform_functions import deform_av, deform_qk, deform_sapa_fused
from .functions import av, qk, sapa_fused
from .projection import project, project_supported


def _init_projection(module: nn.Module) -> None:
    # 1x1 projections start as N(0, 0.02^2) with zero bias (sapa_base.py:42-46)
    if isinstance(module, nn.Conv2d):
        nn.init.normal_(module.weight, std=0.02)
        if module.bias is not None:
            nn.init.constant_(module.bias, 0)


def _check_impl(impl: str) -> str:
    if impl not in ("fused", "separate"):
        raise ValueError(f"impl must be 'fused' or 'separate', got {impl!r}")
    return impl


def _common_dtype(*tensors):
    """Under ``torch.autocast`` the 1x1 projections come out in the autocast type while the value (the module's
    un-normalised input) keeps the caller's type; the kernels want one element type, so everything is cast to the
    autocast type.  Outside autocast the tensors pass through untouched (mismatches are then reported by the op).
    The reference modules have no autocast handling (sapa_base.py:26-40, sapa_deform.py:34-53)."""
    if tensors[0].is_cuda and torch.is_autocast_enabled():
        dtype = torch.get_autocast_dtype("cuda")
        return tuple(t.to(dtype) for t in tensors)
    return tensors


def _projected(x, norm, conv, fuse):
    """``conv(norm(x))``.  With ``fuse`` and no gradient to record, GroupNorm and the 1x1 convolution run as one
    tensor-core GEMM (``sapa_project_forward``); training, CPU tensors and shapes that kernel does not take use the torch
    modules."""
    if fuse and x.is_cuda:
        needs_grad = torch.is_grad_enabled() and (x.requires_grad or conv.weight.requires_grad or
                                                  (norm is not None and norm.weight.requires_grad))
        if not needs_grad:
            if torch.is_autocast_enabled():
                x = x.to(torch.get_autocast_dtype("cuda"))
            if project_supported(x, norm, conv):
                return project(x, norm, conv)
    return conv(norm(x)) if norm is not None else conv(x)


class SAPA(nn.Module):
    """Similarity-aware point affiliation upsampler (SAPA-B): x (low-res) is upsampled under guidance of y."""

    def __init__(self, dim_y, dim_x=None, up_factor=2, up_kernel_size=5, embedding_dim=32, qkv_bias=True, norm=True,
                 impl="fused"):
        super().__init__()
        dim_x = dim_y if dim_x is None else dim_x
        self.up_factor, self.up_kernel_size, self.embedding_dim = up_factor, up_kernel_size, embedding_dim
        self.norm, self.impl = norm, _check_impl(impl)
        self.fuse_projection = impl == "fused"      # set to False to keep torch's GroupNorm + convolution at inference too
        if norm:
            self.norm_y = nn.GroupNorm(32, dim_y)
            self.norm_x = nn.GroupNorm(32, dim_x)
        self.q = nn.Conv2d(dim_y, embedding_dim, kernel_size=1, bias=qkv_bias)
        self.k = nn.Conv2d(dim_x, embedding_dim, kernel_size=1, bias=qkv_bias)
        self.apply(_init_projection)

    def forward(self, y, x):
        # the value is the un-normalised x; only the key is computed from the normalised one
        q = _projected(y, self.norm_y if self.norm else None, self.q, self.fuse_projection)
        k = _projected(x, self.norm_x if self.norm else None, self.k, self.fuse_projection)
        return self.attention(q, k, x)

    def attention(self, q, k, v):
        q, k, v = _common_dtype(q, k, v)
        if self.impl == "fused":
            return sapa_fused(q.contiguous(), k.contiguous(), v.contiguous(), self.up_kernel_size, self.up_factor)
        attn = F.softmax(qk(q, k, self.up_kernel_size, self.up_factor), dim=1)
        return av(attn, v, self.up_kernel_size, self.up_factor)


class SAPADeform(nn.Module):
    """Deformable variant (SAPA-D): num_point learned sampling points per group instead of a fixed window."""

    def __init__(self, dim_y, dim_x=None, up_factor=2, num_point=9, groups=4, embedding_dim=32, qkv_bias=True,
                 high_offset=True, norm=False, impl="fused"):
        super().__init__()
        dim_x = dim_y if dim_x is None else dim_x
        self.up_factor, self.num_point, self.groups = up_factor, num_point, groups
        self.embedding_dim, self.high_offset = embedding_dim, high_offset
        self.norm, self.impl = norm, _check_impl(impl)
        self.fuse_projection = impl == "fused"
        if norm:
            self.norm_y = nn.GroupNorm(32, dim_y)
            self.norm_x = nn.GroupNorm(32, dim_x)
        self.q = nn.Conv2d(dim_y, groups * embedding_dim, kernel_size=1, bias=qkv_bias)
        self.k = nn.Conv2d(dim_x, groups * embedding_dim, kernel_size=1, bias=qkv_bias)
        offset_dim = groups * num_point * 2 * (up_factor ** 2 if high_offset else 1)
        self.offset = nn.Conv2d(dim_x, offset_dim, kernel_size=1, bias=qkv_bias)
        self.apply(_init_projection)

    def forward(self, y, x):
        q = _projected(y, self.norm_y if self.norm else None, self.q, self.fuse_projection)
        k = _projected(x, self.norm_x if self.norm else None, self.k, self.fuse_projection)
        raw = self.offset(self.norm_x(x) if self.norm else x)
        if self.high_offset:   # one offset per high-res pixel, unpacked from channels
            offset = F.pixel_shuffle(raw, upscale_factor=self.up_factor)
        else:                  # every high-res pixel of a parent shares the parent's offset
            offset = F.interpolate(raw, scale_factor=self.up_factor)
        return self.attention(q, k, x, offset)

    def attention(self, q, k, x, offset):
        q, k, x, offset = _common_dtype(q, k, x, offset)
        if self.impl == "fused":
            return deform_sapa_fused(q.contiguous(), k.contiguous(), x.contiguous(), offset.contiguous(),
                                     self.num_point, self.up_factor, self.groups)
        attn = F.softmax(deform_qk(q, k, offset, self.num_point, self.up_factor, self.groups), dim=2)
        return deform_av(attn, x, offset, self.num_point, self.up_factor, self.groups)
