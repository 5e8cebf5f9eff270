"""Tensor-level wrappers over the C ABI: PyTorch supplies device memory and streams,
everything else happens in ``libheddle_b200.so``.

There is no CPU or eager fallback here: CPU tensors are rejected.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Tuple

import torch

from . import _lib

_DTYPES = {torch.bfloat16: _lib.HB_BF16, torch.float16: _lib.HB_FP16}
if hasattr(torch, "float8_e4m3fn"):
    _DTYPES[torch.float8_e4m3fn] = _lib.HB_FP8_E4M3


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "heddle_b200 kernels run on a CUDA (sm_100a) device only; got a tensor on "
                f"{t.device} — there is no CPU fallback")


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _inner_contiguous(t: torch.Tensor) -> torch.Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


def fa_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = False,
           softmax_scale: Optional[float] = None, layout: str = "bhsd", return_lse: bool = False,
           out: Optional[torch.Tensor] = None,
           scales: Optional[Tuple[float, float, float]] = None,
           ) -> "torch.Tensor | Tuple[torch.Tensor, torch.Tensor]":
    """FlashAttention forward through ``hb_fa_fwd``.

    ``layout`` is "bhsd" (q [B,H,S,D]) or "bshd" (q [B,S,H,D]); any batch/head/seq
    strides are passed through, only the head_dim axis must be contiguous.  K/V may
    have fewer heads than Q (grouped-query attention).  Returns O in the layout and
    dtype of q (bf16 for FP8 inputs) and, if requested, the natural-log LSE
    [B, Hq, Sq] in fp32.  ``scales`` = (q, k, v) per-tensor dequantisation scales for FP8.
    """
    _require_cuda(q, k, v)
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("q, k, v must be 4-D")
    if q.dtype not in _DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError(f"unsupported or mismatched dtypes: {q.dtype}, {k.dtype}, {v.dtype}")
    q, k, v = _inner_contiguous(q), _inner_contiguous(k), _inner_contiguous(v)
    if layout == "bhsd":
        b_ax, h_ax, s_ax = 0, 1, 2
    elif layout == "bshd":
        b_ax, h_ax, s_ax = 0, 2, 1
    else:
        raise ValueError(f"unknown layout {layout!r}")
    B, Hq, Sq, D = q.shape[b_ax], q.shape[h_ax], q.shape[s_ax], q.shape[3]
    Hkv, Skv = k.shape[h_ax], k.shape[s_ax]
    if k.shape[b_ax] != B or v.shape != k.shape or k.shape[3] != D:
        raise ValueError(f"shape mismatch: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}")
    out_dtype = torch.bfloat16 if q.dtype not in (torch.bfloat16, torch.float16) else q.dtype
    if out is None:
        out = torch.empty(q.shape, dtype=out_dtype, device=q.device)
    else:
        _require_cuda(out)
        if out.shape != q.shape or out.dtype != out_dtype or out.stride(-1) != 1:
            raise ValueError("out must match q's shape, have the output dtype and a contiguous last axis")
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device) if return_lse else None

    a = _lib.FaArgs()
    a.q, a.k, a.v, a.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    a.lse = lse.data_ptr() if lse is not None else None
    a.B, a.Hq, a.Hkv, a.Sq, a.Skv, a.D = B, Hq, Hkv, Sq, Skv, D
    a.q_stride_b, a.q_stride_h, a.q_stride_s = q.stride(b_ax), q.stride(h_ax), q.stride(s_ax)
    a.k_stride_b, a.k_stride_h, a.k_stride_s = k.stride(b_ax), k.stride(h_ax), k.stride(s_ax)
    a.v_stride_b, a.v_stride_h, a.v_stride_s = v.stride(b_ax), v.stride(h_ax), v.stride(s_ax)
    a.o_stride_b, a.o_stride_h, a.o_stride_s = out.stride(b_ax), out.stride(h_ax), out.stride(s_ax)
    a.causal = 1 if causal else 0
    a.softmax_scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    a.dtype = _DTYPES[q.dtype]
    if scales is not None:
        a.q_scale, a.k_scale, a.v_scale = (float(x) for x in scales)
    a.stream = _stream_ptr(q.device)
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().hb_fa_fwd(C.byref(a)))
    return (out, lse) if return_lse else out


def status_word() -> int:
    """Device status word of the current device: 0 unless a bounded device-side wait gave up."""
    w = C.c_uint32(0)
    _lib.check(_lib.load().hb_status_word(C.byref(w)))
    return int(w.value)


def debug_umma(mode: int, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """One tcgen05 tile through the library's descriptor helpers (see hb_debug_umma)."""
    _require_cuda(a, b)
    a, b = a.contiguous(), b.contiguous()
    kn = b.shape[1]
    ncols = 128 if mode == 0 else kn
    out = torch.empty((128, ncols), dtype=torch.float32, device=a.device)
    with torch.cuda.device(a.device):
        _lib.check(_lib.load().hb_debug_umma(mode, a.data_ptr(), b.data_ptr(), out.data_ptr(), kn,
                                             _DTYPES[a.dtype], _stream_ptr(a.device)))
    return out
