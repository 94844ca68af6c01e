"""Import-compatible stand-in for the reference's ``deformsapa`` package (deformsapa/deformsapa/__init__.py:1-2)."""
from sapa_b200.deform_functions import deform_av, deform_qk  # noqa: F401

__all__ = ["deform_qk", "deform_av"]
