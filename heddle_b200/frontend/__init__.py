"""``torch.compile`` frontend: FX capture, attention rewrites and GEMM + epilogue fusion
(counterpart of Heddle/heddle/frontend/__init__.py)."""
from .backend import tilelang_backend  # noqa: F401
from . import patterns  # noqa: F401
from . import bwd_separator  # noqa: F401
