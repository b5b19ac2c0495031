"""tensorwarp_b200 — the TW-Marlin W4A16 Q4 GEMM family for NVIDIA B200.

Only what this one hot path needs: ``csrc/`` holds the sm_100a kernels and the
C ABI (``include/twmarlin.h``), ``quantize`` mirrors the reference's host
interface over that ABI.  Importing the package does not load the library;
the first call does, and fails loudly if it is not built.
"""
from . import _lib  # noqa: F401
from .build import build  # noqa: F401

__all__ = ["build", "quantize"]
