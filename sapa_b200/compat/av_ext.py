"""Stand-in for the reference's ``av_ext`` pybind module (sapa/sapa/src/av_ext.cpp:18-51): value first
("features"), attention second ("masks"); sizes are taken from the output / top gradient (av_cuda.cpp:37-40)."""
from sapa_b200 import _lib


def forward(value, attn, kernel_size, scale_factor, output):
    _lib.check_tensors(("features", value), ("masks", attn), ("output", output))
    n, c, hq, wq = output.shape
    _lib.call("sapa_av_forward", value.device, attn, value, output, n, c, hq // scale_factor, wq // scale_factor,
              kernel_size, scale_factor, _lib.dtype_code(value))
    return 1


def backward(top_grad, value, attn, kernel_size, scale_factor, grad_value, grad_attn):
    _lib.check_tensors(("top_grad", top_grad), ("features", value), ("masks", attn), ("bottom_grad", grad_value),
                       ("mask_grad", grad_attn))
    n, c, hq, wq = top_grad.shape
    _lib.call("sapa_av_backward", value.device, top_grad, attn, value, grad_attn, grad_value, n, c, hq // scale_factor,
              wq // scale_factor, kernel_size, scale_factor, _lib.dtype_code(value))
    return 1
