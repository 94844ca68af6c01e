"""Stand-in for the reference's ``qk_ext`` pybind module with its positional conventions
(sapa/sapa/src/qk_ext.cpp:22-55): note that the key comes first ("features") and the query second ("masks")."""
from sapa_b200 import _lib


def forward(key, query, kernel_size, scale_factor, output):
    _lib.check_tensors(("features", key), ("masks", query), ("output", output))
    n, d, hq, wq = query.shape
    _lib.call("sapa_qk_forward", key.device, query, key, output, n, d, hq // scale_factor, wq // scale_factor,
              kernel_size, scale_factor, _lib.dtype_code(key))
    return 1


def backward(top_grad, key, query, kernel_size, scale_factor, grad_key, grad_query):
    _lib.check_tensors(("top_grad", top_grad), ("features", key), ("masks", query), ("bottom_grad", grad_key),
                       ("mask_grad", grad_query))
    n, d, hq, wq = query.shape
    _lib.call("sapa_qk_backward", key.device, top_grad, query, key, grad_query, grad_key, n, d, hq // scale_factor,
              wq // scale_factor, kernel_size, scale_factor, _lib.dtype_code(key))
    return 1
