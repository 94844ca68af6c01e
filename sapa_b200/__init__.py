"""sapa_b200 — SAPA upsampling kernels (sim, softmax, atn; SAPA-B and deformable SAPA-D) for NVIDIA B200.

Drop-in for the ``sapa`` / ``deformsapa`` CUDA extensions of tiny-smart/sapa: the same function and module
names with the same arguments, backed by hand-written sm_100a kernels behind a C ABI
(``include/sapa_b200.h``).  There is no CPU path.

To keep ``from sapa import qk, av`` / ``from deformsapa import deform_qk, deform_av`` / ``import qk_ext``
working unchanged, put :func:`compat_path` on ``sys.path``.
"""
import os as _os

from .deform_functions import (DeformAVFunction, DeformQKFunction, DeformSapaFusedFunction, deform_av, deform_qk,
                               deform_sapa_fused)
from .functions import AVFunction, QKFunction, SapaFusedFunction, av, qk, sapa_fused, sapa_fused_nhwc
from .graphs import GraphedForward
from .modules import SAPA, SAPADeform
from .projection import project

__all__ = ["qk", "av", "sapa_fused", "sapa_fused_nhwc", "deform_qk", "deform_av", "deform_sapa_fused", "SAPA", "SAPADeform",
           "QKFunction", "AVFunction", "SapaFusedFunction", "DeformQKFunction", "DeformAVFunction",
           "DeformSapaFusedFunction", "GraphedForward", "project", "compat_path"]


def compat_path() -> str:
    """Directory holding import-compatible ``sapa``, ``deformsapa``, ``qk_ext``, ``av_ext``, ``dqk``, ``dav``."""
    return _os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "compat")
