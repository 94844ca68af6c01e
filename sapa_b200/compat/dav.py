"""Stand-in for the reference's ``dav`` pybind module (deformsapa/deformsapa/src/deform_av.cpp:32-75).
The caller-provided gradient buffers are written in place, as in the reference."""
import torch

from sapa_b200 import _lib


def forward(attn, value, offset, num_point, scale_factor, groups, output):
    _lib.check_tensors(("attn", attn), ("value", value), ("offset", offset), ("output", output))
    n, c, h, w = value.shape
    _lib.call("sapa_deform_av_forward", value.device, attn, value, offset, output, n, c, h, w, num_point, scale_factor,
              groups, _lib.dtype_code(value))
    return 1


def backward(top_grad, attn, value, offset, num_point, scale_factor, groups, grad_attn, grad_value, grad_offset):
    _lib.check_tensors(("top_grad", top_grad), ("data_attn", attn), ("data_value", value), ("data_offset", offset),
                       ("grad_attn", grad_attn), ("grad_value", grad_value), ("grad_offset", grad_offset))
    n, c, h, w = value.shape
    wide = value.dtype in (torch.float32, torch.float64)
    gv = grad_value if wide else torch.empty(value.shape, dtype=torch.float32, device=value.device)
    _lib.call("sapa_deform_av_backward", value.device, top_grad, attn, value, offset, grad_attn, gv, grad_offset, n, c,
              h, w, num_point, scale_factor, groups, _lib.dtype_code(value))
    if not wide:
        grad_value.copy_(gv)
    return 1
