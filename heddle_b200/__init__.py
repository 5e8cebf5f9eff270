"""heddle_b200 — B200-native drop-in for the attention / fused-GEMM hot path of Heddle.

Mirrors the reference's public entry points (Heddle/heddle/__init__.py:22-28):
``init()`` is kept (idempotent) and ``heddle_b200.frontend.tilelang_backend`` is the
``torch.compile`` backend.  The device code is a C-ABI library of hand-written
sm_100a kernels (``libheddle_b200.so``); there is no TileLang/TVM JIT underneath.
"""
from __future__ import annotations

__version__ = "0.1.0"

_initialised = False


def init() -> None:
    """Counterpart of ``heddle.init()`` (Heddle/heddle/__init__.py:22).

    The reference patches TileLang's pass pipeline here.  Nothing is patched in this
    implementation: the call only checks that the native library is loadable, and is
    safe to repeat.
    """
    global _initialised
    if _initialised:
        return
    from . import _lib

    _lib.load()
    _initialised = True
