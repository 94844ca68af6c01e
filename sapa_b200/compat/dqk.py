"""Stand-in for the reference's ``dqk`` pybind module (deformsapa/deformsapa/src/deform_qk.cpp:32-75).
The caller-provided gradient buffers are written in place, as in the reference."""
import torch

from sapa_b200 import _lib


def forward(query, key, offset, num_point, scale_factor, groups, output):
    _lib.check_tensors(("query", query), ("key", key), ("offset", offset), ("output", output))
    n, c, _, _ = query.shape
    _lib.call("sapa_deform_qk_forward", query.device, query, key, offset, output, n, c, key.size(2), key.size(3),
              num_point, scale_factor, groups, _lib.dtype_code(query))
    return 1


def backward(top_grad, query, key, offset, num_point, scale_factor, groups, grad_query, grad_key, grad_offset):
    _lib.check_tensors(("top_grad", top_grad), ("data_query", query), ("data_key", key), ("data_offset", offset),
                       ("grad_query", grad_query), ("grad_key", grad_key), ("grad_offset", grad_offset))
    n, c, h, w = key.shape
    wide = query.dtype in (torch.float32, torch.float64)     # scatter targets accumulate in >= float32
    gq = grad_query if wide else torch.empty(query.shape, dtype=torch.float32, device=query.device)
    gk = grad_key if wide else torch.empty(key.shape, dtype=torch.float32, device=key.device)
    _lib.call("sapa_deform_qk_backward", query.device, top_grad, query, key, offset, gq, gk, grad_offset, n, c, h, w,
              num_point, scale_factor, groups, _lib.dtype_code(query))
    if not wide:
        grad_query.copy_(gq)
        grad_key.copy_(gk)
    return 1
