"""ctypes binding of ``libheddle_b200.so`` (the C ABI declared in include/heddle_b200.h).

There is deliberately no fallback: if the library is missing or a call fails, a
``RuntimeError`` carrying ``hb_last_error()`` is raised.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = _PKG_DIR / "libheddle_b200.so"

HB_OK = 0
HB_ERR_BAD_ARG = 1
HB_ERR_UNSUPPORTED = 2
HB_ERR_ALIGN = 3
HB_ERR_CUDA = 4
HB_ERR_TIMEOUT = 5

HB_BF16 = 0
HB_FP16 = 1
HB_FP8_E4M3 = 2

HB_W_NK = 0
HB_W_KN = 1

HB_QUERY_SM_COUNT = 0
HB_QUERY_SMEM_OPTIN = 1
HB_QUERY_CC = 2
HB_QUERY_FA_SMEM = 3
HB_QUERY_GEMM_SMEM = 4

EPILOGUES = {
    "none": 0, "silu": 1, "relu": 2, "gelu_tanh": 3, "sigmoid": 4, "tanh": 5, "swiglu": 6, "rope": 7,
}


class FaArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p), ("lse", C.c_void_p),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("Sq", C.c_int32), ("Skv", C.c_int32),
        ("D", C.c_int32),
        ("q_stride_b", C.c_int64), ("q_stride_h", C.c_int64), ("q_stride_s", C.c_int64),
        ("k_stride_b", C.c_int64), ("k_stride_h", C.c_int64), ("k_stride_s", C.c_int64),
        ("v_stride_b", C.c_int64), ("v_stride_h", C.c_int64), ("v_stride_s", C.c_int64),
        ("o_stride_b", C.c_int64), ("o_stride_h", C.c_int64), ("o_stride_s", C.c_int64),
        ("causal", C.c_int32), ("softmax_scale", C.c_float), ("dtype", C.c_int32),
        ("q_scale", C.c_float), ("k_scale", C.c_float), ("v_scale", C.c_float), ("p_scale", C.c_float),
        ("o_scale", C.c_float),
        ("stream", C.c_void_p),
    ]


class H2oArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("lse", C.c_void_p), ("score", C.c_void_p),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("Sq", C.c_int32), ("Skv", C.c_int32),
        ("D", C.c_int32),
        ("q_stride_b", C.c_int64), ("q_stride_h", C.c_int64), ("q_stride_s", C.c_int64),
        ("k_stride_b", C.c_int64), ("k_stride_h", C.c_int64), ("k_stride_s", C.c_int64),
        ("causal", C.c_int32), ("softmax_scale", C.c_float), ("dtype", C.c_int32),
        ("stream", C.c_void_p),
    ]


class FaBwdArgs(C.Structure):
    """Mirror of hb_fa_bwd_args."""
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p), ("d_o", C.c_void_p),
        ("lse", C.c_void_p), ("delta", C.c_void_p), ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("Sq", C.c_int32), ("Skv", C.c_int32),
        ("D", C.c_int32),
        ("q_stride_b", C.c_int64), ("q_stride_h", C.c_int64), ("q_stride_s", C.c_int64),
        ("k_stride_b", C.c_int64), ("k_stride_h", C.c_int64), ("k_stride_s", C.c_int64),
        ("v_stride_b", C.c_int64), ("v_stride_h", C.c_int64), ("v_stride_s", C.c_int64),
        ("o_stride_b", C.c_int64), ("o_stride_h", C.c_int64), ("o_stride_s", C.c_int64),
        ("do_stride_b", C.c_int64), ("do_stride_h", C.c_int64), ("do_stride_s", C.c_int64),
        ("causal", C.c_int32), ("softmax_scale", C.c_float), ("dtype", C.c_int32),
        ("stream", C.c_void_p),
    ]


class GemmArgs(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("w", C.c_void_p), ("out", C.c_void_p),
        ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32),
        ("lda", C.c_int64), ("ldw", C.c_int64), ("ldo", C.c_int64),
        ("dtype", C.c_int32), ("epilogue", C.c_int32),
        ("row_scale", C.c_void_p), ("bias", C.c_void_p), ("residual", C.c_void_p), ("ldr", C.c_int64),
        ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p),
        ("rope_seq", C.c_int32), ("head_dim", C.c_int32), ("rope_cols", C.c_int32),
        ("stream", C.c_void_p),
        ("batch", C.c_int32), ("w_layout", C.c_int32),
        ("a_batch_stride", C.c_int64), ("w_batch_stride", C.c_int64), ("o_batch_stride", C.c_int64),
        ("r_batch_stride", C.c_int64), ("schedule", C.c_int32),
    ]


GEMM_SCHEDULES = {"auto": 0, "single": 1, "pair": 2}


class PrepareArgs(C.Structure):
    """Mirror of hb_prepare_args."""
    _fields_ = [
        ("src", C.c_void_p * 4), ("rows", C.c_int32 * 4), ("ld_src", C.c_int64 * 4),
        ("n_src", C.c_int32), ("K", C.c_int32), ("gamma", C.c_void_p), ("out", C.c_void_p),
        ("ld_out", C.c_int64), ("dtype", C.c_int32), ("stream", C.c_void_p),
    ]


EW_OPS = {
    "load": 0, "add": 1, "sub": 2, "rsub": 3, "mul": 4, "div": 5, "rdiv": 6, "max": 7, "min": 8, "pow": 9,
    "neg": 16, "abs": 17, "exp": 18, "log": 19, "log2": 20, "sqrt": 21, "rsqrt": 22, "recip": 23, "sigmoid": 24,
    "silu": 25, "relu": 26, "gelu_tanh": 27, "gelu_erf": 28, "tanh": 29, "round": 30, "store_tmp": 40,
    "reduce_sum": 48, "reduce_max": 49, "reduce_mean": 50, "store_out": 56,
}
EW_SRCS = {"none": 0, "input": 1, "imm": 2, "tmp": 3, "rowvec": 4, "rowscalar": 5, "reduced": 6}
EW_MAX_INST, EW_MAX_INPUTS, EW_MAX_ROWVEC, EW_MAX_ROWSCALAR, EW_MAX_OUTPUTS, EW_MAX_TMP, EW_MAX_RED = 48, 6, 4, 4, 2, 4, 4


class EwInst(C.Structure):
    """Mirror of hb_ew_inst."""
    _fields_ = [("op", C.c_int32), ("src", C.c_int32), ("index", C.c_int32), ("imm", C.c_float)]


class RowwiseArgs(C.Structure):
    """Mirror of hb_rowwise_args."""
    _fields_ = [
        ("inputs", C.c_void_p * EW_MAX_INPUTS), ("ld_in", C.c_int64 * EW_MAX_INPUTS),
        ("rowvec", C.c_void_p * EW_MAX_ROWVEC), ("rowscalar", C.c_void_p * EW_MAX_ROWSCALAR),
        ("outputs", C.c_void_p * EW_MAX_OUTPUTS), ("ld_out", C.c_int64 * EW_MAX_OUTPUTS),
        ("n_inputs", C.c_int32), ("n_rowvec", C.c_int32), ("n_rowscalar", C.c_int32), ("n_outputs", C.c_int32),
        ("rows", C.c_int64), ("cols", C.c_int32), ("dtype", C.c_int32), ("n_inst", C.c_int32),
        ("program", EwInst * EW_MAX_INST), ("stream", C.c_void_p), ("mode", C.c_int32),
    ]


ROWWISE_AUTO, ROWWISE_INTERPRET, ROWWISE_COMPILED = 0, 1, 2


# every symbol include/heddle_b200.h declares
EXPORTS = (
    "hb_fa_fwd", "hb_fa_fwd_noalloc", "hb_status_word_noalloc", "hb_fa_bwd_preprocess", "hb_fa_bwd_dkdv", "hb_fa_bwd_dq", "hb_h2o_score", "hb_gemm_epilogue", "hb_rms_rowstat", "hb_prepare_weight", "hb_row_softmax", "hb_rowwise_program", "hb_rowwise_compiler_available", "hb_debug_rowwise_compile", "hb_status_word",
    "hb_version",
    "hb_query", "hb_last_error", "hb_shutdown", "hb_debug_umma", "hb_debug_wait_timeout", "hb_debug_fa_fwd_stages",
)

_lib = None


def load() -> C.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = Path(os.environ.get("HEDDLE_B200_LIB", str(LIB_PATH)))
    if not path.exists():
        raise RuntimeError(
            f"{path} not found: build it with `python -m heddle_b200._build` "
            "(there is no CPU or PyTorch fallback for the heddle_b200 kernels)")
    lib = C.CDLL(str(path))
    lib.hb_fa_fwd.argtypes = [C.POINTER(FaArgs)]
    lib.hb_fa_fwd.restype = C.c_int
    lib.hb_fa_fwd_noalloc.argtypes = [C.POINTER(FaArgs)]
    lib.hb_fa_fwd_noalloc.restype = C.c_int
    for name in ("hb_fa_bwd_preprocess", "hb_fa_bwd_dkdv", "hb_fa_bwd_dq"):
        getattr(lib, name).argtypes = [C.POINTER(FaBwdArgs)]
        getattr(lib, name).restype = C.c_int
    lib.hb_h2o_score.argtypes = [C.POINTER(H2oArgs)]
    lib.hb_h2o_score.restype = C.c_int
    lib.hb_gemm_epilogue.argtypes = [C.POINTER(GemmArgs)]
    lib.hb_gemm_epilogue.restype = C.c_int
    lib.hb_rms_rowstat.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                   C.c_int64, C.c_float, C.c_int32, C.c_void_p]
    lib.hb_rms_rowstat.restype = C.c_int
    lib.hb_prepare_weight.argtypes = [C.POINTER(PrepareArgs)]
    lib.hb_prepare_weight.restype = C.c_int
    lib.hb_row_softmax.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int64, C.c_int64, C.c_float,
                                   C.c_int32, C.c_void_p]
    lib.hb_row_softmax.restype = C.c_int
    lib.hb_rowwise_program.argtypes = [C.POINTER(RowwiseArgs)]
    lib.hb_rowwise_program.restype = C.c_int
    lib.hb_rowwise_compiler_available.argtypes = []
    lib.hb_rowwise_compiler_available.restype = C.c_int
    lib.hb_debug_rowwise_compile.argtypes = [C.POINTER(RowwiseArgs), C.c_char_p, C.c_int64]
    lib.hb_debug_rowwise_compile.restype = C.c_int
    lib.hb_status_word.argtypes = [C.POINTER(C.c_uint32)]
    lib.hb_status_word.restype = C.c_int
    lib.hb_status_word_noalloc.argtypes = [C.POINTER(C.c_uint32), C.c_void_p]
    lib.hb_status_word_noalloc.restype = C.c_int
    lib.hb_version.argtypes = []
    lib.hb_version.restype = C.c_int
    lib.hb_query.argtypes = [C.c_int]
    lib.hb_query.restype = C.c_int
    lib.hb_last_error.argtypes = []
    lib.hb_last_error.restype = C.c_char_p
    lib.hb_shutdown.argtypes = []
    lib.hb_shutdown.restype = C.c_int
    lib.hb_debug_umma.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]
    lib.hb_debug_umma.restype = C.c_int
    lib.hb_debug_fa_fwd_stages.argtypes = [C.POINTER(FaArgs), C.c_int32]
    lib.hb_debug_fa_fwd_stages.restype = C.c_int
    lib.hb_debug_wait_timeout.argtypes = [C.c_uint32, C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)]
    lib.hb_debug_wait_timeout.restype = C.c_int
    _lib = lib
    return lib


def last_error() -> str:
    return load().hb_last_error().decode("utf-8", "replace")


class HeddleError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"heddle_b200 error {code}: {message}")
        self.code = code


def check(rc: int) -> None:
    if rc != HB_OK:
        raise HeddleError(rc, last_error())
