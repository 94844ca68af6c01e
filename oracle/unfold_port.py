"""The reference's CPU path, restated in PyTorch.  TEST INFRASTRUCTURE ONLY.

The reference has no CPU kernels; the only CPU formulation of its ops is the pure-PyTorch check code that
ships next to the extensions:

* ``qk_pytorch`` / ``av_pytorch``  - sapa/sapa/forward_check.py:9-24 (zero-padded ``F.unfold`` + einsum),
* ``sample`` / ``deform_qk_pytorch`` / ``deform_av_pytorch`` - deformsapa/deformsapa/forward_check.py:6-40
  (``F.grid_sample``, bilinear, zeros padding, ``align_corners=False``).

This module restates that formulation (same tensor algebra, written independently) so that it can be timed
on host cores as the CPU baseline and differentiated with autograd as a second gradient oracle.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def _windows(x: torch.Tensor, K: int) -> torch.Tensor:
    """[B,C,H,W] -> [B,C,K*K,H,W]: the zero-padded K x K neighbourhood of every low-res pixel."""
    B, C, H, W = x.shape
    cols = F.unfold(x, kernel_size=K, padding=(K - 1) // 2)
    return cols.view(B, C, K * K, H, W)


def sim(query: torch.Tensor, key: torch.Tensor, K: int = 5, s: int = 2) -> torch.Tensor:
    """Similarity logits [B,K*K,sH,sW] (what ``qk`` computes)."""
    B, d, H, W = key.shape
    q = query.reshape(B, d, H, s, W, s)
    win = _windows(key, K)
    out = torch.einsum("bchiwj,bckhw->bkhiwj", q, win)
    return out.reshape(B, K * K, s * H, s * W)


def atn(attn: torch.Tensor, value: torch.Tensor, K: int = 5, s: int = 2) -> torch.Tensor:
    """Aggregated output [B,C,sH,sW] (what ``av`` computes)."""
    B, C, H, W = value.shape
    a = attn.reshape(B, K * K, H, s, W, s)
    win = _windows(value, K)
    out = torch.einsum("bkhiwj,bckhw->bchiwj", a, win)
    return out.reshape(B, C, s * H, s * W)


def sapa(query, key, value, K: int = 5, s: int = 2) -> torch.Tensor:
    """atn(softmax(sim(q, k), dim=1), v): the SAPA-B attention of sapa_base.py:38-40."""
    return atn(torch.softmax(sim(query, key, K, s), dim=1), value, K, s)


def _sample(x: torch.Tensor, offset: torch.Tensor, P: int, s: int, G: int) -> torch.Tensor:
    """Bilinear samples of x at (parent pixel centre + offset): [B,G,P,C/G,sH,sW].

    ``offset`` is [B, G*P*2, sH, sW] with channel 2k = x (w) offset and 2k+1 = y (h) offset in low-res
    pixels.  Pixel i of the low-res grid has centre i+0.5, so grid_sample with align_corners=False on
    ``2*(i+0.5+off)/size-1`` reads position i+off in index coordinates, as the CUDA helper does.
    """
    B, C, H, W = x.shape
    sH, sW = s * H, s * W
    off = offset.reshape(B, G * P, 2, sH, sW)
    base_x = (torch.arange(sW, device=x.device) // s).to(x.dtype) + 0.5
    base_y = (torch.arange(sH, device=x.device) // s).to(x.dtype) + 0.5
    gx = 2.0 * (base_x.view(1, 1, 1, sW) + off[:, :, 0]) / W - 1.0
    gy = 2.0 * (base_y.view(1, 1, sH, 1) + off[:, :, 1]) / H - 1.0
    grid = torch.stack((gx, gy), dim=-1).reshape(B * G * P, sH, sW, 2)
    planes = x.reshape(B, G, 1, C // G, H, W).expand(B, G, P, C // G, H, W).reshape(B * G * P, C // G, H, W)
    smp = F.grid_sample(planes, grid, mode="bilinear", padding_mode="zeros", align_corners=False)
    return smp.reshape(B, G, P, C // G, sH, sW)


def deform_sim(query, key, offset, P: int = 9, s: int = 2, G: int = 4) -> torch.Tensor:
    """Deformable logits [B,G,P,sH,sW] (what ``deform_qk`` computes)."""
    B, Cq, sH, sW = query.shape
    k = _sample(key, offset, P, s, G)
    return (query.reshape(B, G, 1, Cq // G, sH, sW) * k).sum(dim=3)


def deform_atn(attn, value, offset, P: int = 9, s: int = 2, G: int = 4) -> torch.Tensor:
    """Deformable aggregation [B,C,sH,sW] (what ``deform_av`` computes)."""
    B, _, _, sH, sW = attn.shape
    v = _sample(value, offset, P, s, G)
    return (attn.unsqueeze(3) * v).sum(dim=2).reshape(B, -1, sH, sW)


def deform_sapa(query, key, value, offset, P: int = 9, s: int = 2, G: int = 4) -> torch.Tensor:
    """deform_atn(softmax(deform_sim(...), dim=2), v, offset): SAPA-D attention of sapa_deform.py:51-53."""
    a = torch.softmax(deform_sim(query, key, offset, P, s, G), dim=2)
    return deform_atn(a, value, offset, P, s, G)
