"""ctypes binding of ``libsapa_b200.so`` (the C ABI declared in ``include/sapa_b200.h``).

There is no CPU or PyTorch fallback: if the library cannot be loaded the import of any op fails loudly.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# SAPA_B200_LIB points at another build of the same library (for example one compiled with extra flags)
LIB_PATH = os.environ.get("SAPA_B200_LIB") or os.path.join(_HERE, "libsapa_b200.so")

SAPA_F32, SAPA_F16, SAPA_BF16, SAPA_F64 = 0, 1, 2, 3
_DTYPE_CODE = {torch.float32: SAPA_F32, torch.float16: SAPA_F16, torch.bfloat16: SAPA_BF16, torch.float64: SAPA_F64}
SAPA_ERR_UNSUPPORTED = -5
ABI_VERSION = 3

_lib = None

_vp, _i, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
# name -> argument types; every function returns int except the two noted below
_SIGNATURES = {
    "sapa_qk_forward": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_qk_backward": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_av_forward": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_av_backward": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_fused_forward": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_fused_forward_nhwc": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_fused_forward_slab": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_fused_forward_slab_rows": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_fused_backward": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_fused_backward_slab": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_fused_backward_static": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_deform_qk_forward": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_deform_qk_backward": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_deform_av_forward": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_deform_av_backward": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_deform_fused_forward": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_deform_qk_forward_dense": [_vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_deform_av_forward_dense": [_vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_deform_av_backward_dense": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_deform_qk_backward_dense": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_deform_fused_forward_dense": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_deform_fused_forward_slab": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_selftest_wait_timeout": [_vp],
    "sapa_project_forward": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, ctypes.c_float, _i, _vp],
    "sapa_deform_fused_backward_dense": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "sapa_deform_fused_backward": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
}
EXPORTS = sorted(list(_SIGNATURES) + ["sapa_last_error", "sapa_last_kernels", "sapa_abi_version", "sapa_fused_backward_workspace",
                                           "sapa_deform_fused_forward_workspace", "sapa_deform_fused_backward_workspace",
                                           "sapa_deform_fused_backward_scatter_bytes", "sapa_project_workspace",
                                           "sapa_fused_backward_static_capacity", "sapa_wait_timeout_flags"])


def lib() -> ctypes.CDLL:
    """Load (building first if the toolkit is present and the library is missing) and type the library."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        try:
            from . import build as _build
            _build.build()
        except Exception as exc:  # no nvcc on this machine
            raise RuntimeError(
                f"libsapa_b200.so is missing at {LIB_PATH} and could not be built ({exc}); "
                "run `python -m sapa_b200.build` on a machine with the CUDA toolkit. "
                "There is no CPU fallback.") from exc
    handle = ctypes.CDLL(LIB_PATH)
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(handle, name)
        fn.argtypes = argtypes
        fn.restype = ctypes.c_int
    handle.sapa_last_error.argtypes = []
    handle.sapa_last_error.restype = ctypes.c_char_p
    handle.sapa_last_kernels.argtypes = []
    handle.sapa_last_kernels.restype = ctypes.c_char_p
    handle.sapa_abi_version.argtypes = []
    handle.sapa_abi_version.restype = ctypes.c_int
    handle.sapa_fused_backward_workspace.argtypes = [_i, _i, _i, _i, _i, _i]
    handle.sapa_fused_backward_workspace.restype = ctypes.c_size_t
    handle.sapa_deform_fused_backward_scatter_bytes.argtypes = [_i, _i, _i, _i, _i, _i]
    handle.sapa_deform_fused_backward_scatter_bytes.restype = ctypes.c_size_t
    handle.sapa_deform_fused_forward_workspace.argtypes = [_i, _i, _i, _i, _i, _i, _i]
    handle.sapa_deform_fused_forward_workspace.restype = ctypes.c_size_t
    handle.sapa_deform_fused_backward_workspace.argtypes = [_i, _i, _i, _i, _i, _i, _i]
    handle.sapa_deform_fused_backward_workspace.restype = ctypes.c_size_t
    handle.sapa_project_workspace.argtypes = [_i, _i, _i, _i, _i, _i]
    handle.sapa_project_workspace.restype = ctypes.c_size_t
    handle.sapa_fused_backward_static_capacity.argtypes = []
    handle.sapa_fused_backward_static_capacity.restype = ctypes.c_size_t
    handle.sapa_wait_timeout_flags.argtypes = []
    handle.sapa_wait_timeout_flags.restype = ctypes.c_int
    if handle.sapa_abi_version() != ABI_VERSION:
        raise RuntimeError("libsapa_b200.so has a different ABI version than this Python package; rebuild it")
    _lib = handle
    return _lib


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise RuntimeError(f"sapa_b200: unsupported dtype {t.dtype}") from None


def check_tensors(*named: tuple[str, torch.Tensor]) -> None:
    """The reference's CHECK_INPUT (CUDA + contiguous, qk_cuda.cpp:34-39) plus same dtype / device."""
    first = named[0][1]
    for name, t in named:
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor")
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
        if t.dtype != first.dtype:
            raise RuntimeError(f"{name} has dtype {t.dtype}, expected {first.dtype} (all tensors of a call share one dtype)")
        if t.device != first.device:
            raise RuntimeError(f"{name} is on {t.device}, expected {first.device}")


def _arg(a):
    if isinstance(a, torch.Tensor):
        return ctypes.c_void_p(a.data_ptr())
    return a


def call(name: str, device: torch.device, *args, allow_unsupported: bool = False) -> int:
    """Invoke one C entry point on ``device``'s current stream; raises RuntimeError on a failure status."""
    handle = lib()
    with torch.cuda.device(device):
        stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        status = getattr(handle, name)(*[_arg(a) for a in args], stream)
    if status != 0:
        if allow_unsupported and status == SAPA_ERR_UNSUPPORTED:
            return status
        msg = handle.sapa_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{name} failed with status {status}: {msg}")
    return 0


def last_kernels() -> list[str]:
    """Kernels launched by the most recent entry-point call of this thread, in launch order."""
    text = lib().sapa_last_kernels().decode("utf-8", "replace")
    return text.split(",") if text else []


def aligned(t: torch.Tensor) -> torch.Tensor:
    """``t`` itself when its first element sits on a 16-byte boundary, else a fresh copy (a contiguous view with an odd
    storage offset, e.g. ``x[1:]`` of an odd-sized image, is legal input for the reference; the fused kernels need
    vector alignment)."""
    return t if t.data_ptr() % 16 == 0 else t.clone()


def wait_timeout_flags(device) -> int:
    """Bit mask of the kernels whose bounded barrier waits ever gave up on ``device`` (0 = none); synchronises."""
    with torch.cuda.device(device):
        return int(lib().sapa_wait_timeout_flags())


def fused_backward_workspace(B, H, W, K, s, code) -> int:
    return int(lib().sapa_fused_backward_workspace(B, H, W, K, s, code))
