"""Import the reference's Python check modules by file path (used only by make_golden.py).

Needs the reference checkout and the compiled reference extensions (``python oracle/build_ref.py``),
because the check modules import ``qk_ext`` / ``av_ext`` / ``dqk`` / ``dav`` at load time.
"""
import importlib.util
import os
import sys

REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def load(reference: str):
    """Returns (sapa forward_check module, deformsapa forward_check module)."""
    ref_so = os.path.join(REPO, "oracle", "_ref")
    for p in (ref_so, os.path.join(reference, "sapa", "sapa"),
              os.path.join(reference, "deformsapa", "deformsapa")):
        if p not in sys.path:
            sys.path.insert(0, p)
    mods = []
    for name, rel in (("ref_sapa_forward_check", "sapa/sapa/forward_check.py"),
                      ("ref_deform_forward_check", "deformsapa/deformsapa/forward_check.py")):
        spec = importlib.util.spec_from_file_location(name, os.path.join(reference, rel))
        m = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(m)
        mods.append(m)
    return tuple(mods)
