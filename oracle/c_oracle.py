"""ctypes front end of ``libsapa_oracle.so`` (built by ``make -C oracle``).  TEST INFRASTRUCTURE ONLY.

All functions take and return numpy arrays (float32 or float64, NCHW, C-contiguous).  ``H``/``W`` of the
key / value are the low-resolution sizes; query, attention, offset and output are ``s`` times larger.
Each function names the reference kernel it restates; the C source carries the line citations.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libsapa_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the C oracle if needed and return the path of the shared library."""
    srcs = [os.path.join(_HERE, f) for f in ("sapa_oracle.c", "sapa_oracle_impl.inc")]
    stale = (not os.path.exists(_SO)) or any(
        os.path.exists(s) and os.path.getmtime(s) > os.path.getmtime(_SO) for s in srcs)
    if force or stale:
        if force and os.path.exists(_SO):
            os.remove(_SO)
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    lib().oracle_set_num_threads(ctypes.c_int(int(n)))


def _sfx(*arrays: np.ndarray) -> str:
    dt = arrays[0].dtype
    for a in arrays:
        if a.dtype != dt:
            raise TypeError("oracle inputs must share one dtype")
    if dt == np.float32:
        return "_f32"
    if dt == np.float64:
        return "_f64"
    raise TypeError(f"oracle supports float32/float64, got {dt}")


def _c(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a)


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _call(name: str, sfx: str, *args):
    fn = getattr(lib(), name + sfx)
    fn.restype = None
    conv = []
    for a in args:
        if isinstance(a, np.ndarray):
            conv.append(_p(a))
        elif isinstance(a, _Long):
            conv.append(ctypes.c_long(a.v))
        else:
            conv.append(ctypes.c_int(int(a)))
    fn(*conv)


class _Long:
    def __init__(self, v):
        self.v = int(v)


# ------------------------------------------------------------------ SAPA-B

def qk_forward(query, key, K, s):
    """Similarity logits; restates QKForward (qk_cuda_kernel.cu:29-68)."""
    query, key = _c(query), _c(key)
    B, d, H, W = key.shape
    assert query.shape == (B, query.shape[1], s * H, s * W)
    out = np.empty((B, K * K, s * H, s * W), query.dtype)
    _call("oracle_qk_forward", _sfx(query, key), query, key, out, B, query.shape[1], H, W, K, s)
    return out


def qk_backward(grad_out, query, key, K, s):
    """(dQuery, dKey); restates QKBackward (qk_cuda_kernel.cu:101-137)."""
    grad_out, query, key = _c(grad_out), _c(query), _c(key)
    B, d, H, W = key.shape
    gq, gk = np.empty_like(query), np.empty_like(key)
    _call("oracle_qk_backward", _sfx(grad_out, query, key), grad_out, query, key, gq, gk, B, d, H, W, K, s)
    return gq, gk


def av_forward(attn, value, K, s):
    """Window-weighted aggregation; restates AVForward (av_cuda_kernel.cu:29-75)."""
    attn, value = _c(attn), _c(value)
    B, C, H, W = value.shape
    out = np.empty((B, C, s * H, s * W), value.dtype)
    _call("oracle_av_forward", _sfx(attn, value), attn, value, out, B, C, H, W, K, s)
    return out


def av_backward(grad_out, attn, value, K, s):
    """(dAttn, dValue); restates AVBackward (av_cuda_kernel.cu:103-148)."""
    grad_out, attn, value = _c(grad_out), _c(attn), _c(value)
    B, C, H, W = value.shape
    ga, gv = np.empty_like(attn), np.empty_like(value)
    _call("oracle_av_backward", _sfx(grad_out, attn, value), grad_out, attn, value, ga, gv, B, C, H, W, K, s)
    return ga, gv


def softmax(x, axis):
    """Softmax over ``axis`` (SAPA-B: axis 1 of [B,K*K,sH,sW]; SAPA-D: axis 2 of [B,G,P,sH,sW])."""
    x = _c(x)
    outer = int(np.prod(x.shape[:axis], dtype=np.int64))
    inner = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
    y = np.empty_like(x)
    _call("oracle_softmax", _sfx(x), x, y, _Long(outer), x.shape[axis], _Long(inner))
    return y


def softmax_backward(y, dy, axis):
    y, dy = _c(y), _c(dy)
    outer = int(np.prod(y.shape[:axis], dtype=np.int64))
    inner = int(np.prod(y.shape[axis + 1:], dtype=np.int64))
    dx = np.empty_like(y)
    _call("oracle_softmax_backward", _sfx(y, dy), y, dy, dx, _Long(outer), y.shape[axis], _Long(inner))
    return dx


def sapa_forward(query, key, value, K, s, return_attn=False):
    """Whole SAPA-B attention: av(softmax(qk(q, k), dim=1), v)  (sapa_base.py:38-40)."""
    attn = softmax(qk_forward(query, key, K, s), 1)
    out = av_forward(attn, value, K, s)
    return (out, attn) if return_attn else out


def sapa_backward(grad_out, query, key, value, K, s):
    """(dQuery, dKey, dValue) of :func:`sapa_forward` by chaining the three backward steps."""
    attn = softmax(qk_forward(query, key, K, s), 1)
    ga, gv = av_backward(grad_out, attn, value, K, s)
    gs = softmax_backward(attn, ga, 1)
    gq, gk = qk_backward(gs, query, key, K, s)
    return gq, gk, gv


# ------------------------------------------------------------------ SAPA-D

def deform_qk_forward(query, key, offset, P, s, G):
    """Restates DeformQKForward (deform_qk_cuda_kernel.cu:139-197); output [B,G,P,sH,sW]."""
    query, key, offset = _c(query), _c(key), _c(offset)
    B, Cq, H, W = key.shape
    out = np.empty((B, G, P, s * H, s * W), query.dtype)
    _call("oracle_deform_qk_forward", _sfx(query, key, offset), query, key, offset, out, B, Cq, H, W, P, s, G)
    return out


def deform_qk_backward(grad_out, query, key, offset, P, s, G):
    """(dQuery, dKey, dOffset); restates DeformQKBackward (deform_qk_cuda_kernel.cu:233-296)."""
    grad_out, query, key, offset = _c(grad_out), _c(query), _c(key), _c(offset)
    B, Cq, H, W = key.shape
    gq, gk, go = np.empty_like(query), np.empty_like(key), np.empty_like(offset)
    _call("oracle_deform_qk_backward", _sfx(grad_out, query, key, offset), grad_out, query, key, offset,
          gq, gk, go, B, Cq, H, W, P, s, G)
    return gq, gk, go


def deform_av_forward(attn, value, offset, P, s, G):
    """Restates DeformAVForward (deform_av_cuda_kernel.cu:139-195); output [B,C,sH,sW]."""
    attn, value, offset = _c(attn), _c(value), _c(offset)
    B, C, H, W = value.shape
    out = np.empty((B, C, s * H, s * W), value.dtype)
    _call("oracle_deform_av_forward", _sfx(attn, value, offset), attn, value, offset, out, B, C, H, W, P, s, G)
    return out


def deform_av_backward(grad_out, attn, value, offset, P, s, G):
    """(dAttn, dValue, dOffset); restates DeformAVBackward (deform_av_cuda_kernel.cu:230-292)."""
    grad_out, attn, value, offset = _c(grad_out), _c(attn), _c(value), _c(offset)
    B, C, H, W = value.shape
    ga, gv, go = np.empty_like(attn), np.empty_like(value), np.empty_like(offset)
    _call("oracle_deform_av_backward", _sfx(grad_out, attn, value, offset), grad_out, attn, value, offset,
          ga, gv, go, B, C, H, W, P, s, G)
    return ga, gv, go


def deform_sapa_forward(query, key, value, offset, P, s, G, return_attn=False):
    """Whole SAPA-D attention: deform_av(softmax(deform_qk(...), dim=2), x, offset) (sapa_deform.py:51-53)."""
    attn = softmax(deform_qk_forward(query, key, offset, P, s, G), 2)
    out = deform_av_forward(attn, value, offset, P, s, G)
    return (out, attn) if return_attn else out


def deform_sapa_backward(grad_out, query, key, value, offset, P, s, G):
    """(dQuery, dKey, dValue, dOffset); the offset gradient is the sum of both ops' (it feeds both)."""
    attn = softmax(deform_qk_forward(query, key, offset, P, s, G), 2)
    ga, gv, go_av = deform_av_backward(grad_out, attn, value, offset, P, s, G)
    gs = softmax_backward(attn, ga, 2)
    gq, gk, go_qk = deform_qk_backward(gs, query, key, offset, P, s, G)
    return gq, gk, gv, go_av + go_qk
