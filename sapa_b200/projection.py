"""GroupNorm + 1x1 projection in front of the attention (``self.q(self.norm_y(y))`` / ``self.k(self.norm_x(x))`` of the
reference modules, sapa_base.py:27-34, sapa_deform.py:35-42) as one tensor-core GEMM: ``sapa_project_forward`` of the C ABI.

Forward only.  The modules use it when no gradient is needed (inference); training keeps torch's GroupNorm and
convolution, whose backward autograd already provides.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import _lib


def project_supported(x: torch.Tensor, norm, conv: nn.Conv2d) -> bool:
    """True when :func:`project` can run this projection (CUDA, float32 / float16 / bfloat16, 1x1 convolution with
    stride 1 and one group, a shape the GEMM kernel takes)."""
    if not x.is_cuda or x.dim() != 4 or x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        return False
    if conv.kernel_size != (1, 1) or conv.stride != (1, 1) or conv.padding != (0, 0) or conv.groups != 1 or conv.dilation != (1, 1):
        return False
    if norm is not None and not isinstance(norm, nn.GroupNorm):
        return False
    if norm is not None and not norm.affine:
        return False
    b, c, h, w = x.shape
    groups = norm.num_groups if norm is not None else 0
    return int(_lib.lib().sapa_project_workspace(b, c, h * w, conv.out_channels, groups, _lib.dtype_code(x))) != 0


def project(x: torch.Tensor, norm, conv: nn.Conv2d) -> torch.Tensor:
    """``conv(norm(x))`` for a 1x1 ``conv`` and a GroupNorm (or ``None``) ``norm``; ``x`` [B, C, H, W] -> [B, d, H, W]."""
    b, c, h, w = x.shape
    d = conv.out_channels
    x = _lib.aligned(x.contiguous())
    dt = x.dtype
    weight = conv.weight.detach().reshape(d, c).to(dt).contiguous()
    bias = conv.bias.detach().to(dt).contiguous() if conv.bias is not None else None
    groups = norm.num_groups if norm is not None else 0
    gamma = norm.weight.detach().to(dt).contiguous() if norm is not None else None
    beta = norm.bias.detach().to(dt).contiguous() if norm is not None else None
    eps = float(norm.eps) if norm is not None else 0.0
    code = _lib.dtype_code(x)
    nbytes = int(_lib.lib().sapa_project_workspace(b, c, h * w, d, groups, code))
    if nbytes == 0:
        raise NotImplementedError("sapa_project_forward does not take this shape / dtype (see project_supported)")
    workspace = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    out = torch.empty((b, d, h, w), dtype=dt, device=x.device)
    _lib.call("sapa_project_forward", x.device, x, gamma, beta, weight, bias, out, workspace, workspace.numel(),
              b, c, h * w, d, groups, eps, code)
    return out
