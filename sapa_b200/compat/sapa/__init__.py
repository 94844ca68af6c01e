"""Import-compatible stand-in for the reference's ``sapa`` package (sapa/sapa/__init__.py:1-3)."""
from sapa_b200.functions import av, qk  # noqa: F401

__all__ = ["qk", "av"]
