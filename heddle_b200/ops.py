"""Tensor-level wrappers over the C ABI: PyTorch supplies device memory and streams,
everything else happens in ``libheddle_b200.so``.

There is no CPU or eager fallback here: CPU tensors are rejected.
"""
from __future__ import annotations

import ctypes as C
import os
import math
from typing import Optional, Sequence, Tuple

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
           debug_stages: Optional[int] = None,
           ) -> "torch.Tensor | Tuple[torch.Tensor, torch.Tensor]":
    """FlashAttention forward through ``hb_fa_fwd``.

    ``layout`` is "bhsd" (q [B,H,S,D]) or "bshd" (q [B,S,H,D]); any batch/head/seq
    strides are passed through, only the head_dim axis must be contiguous.  K/V may
    have fewer heads than Q (grouped-query attention).  Returns O in the layout and
    dtype of q (bf16 for FP8 inputs) and, if requested, the natural-log LSE
    [B, Hq, Sq] in fp32.  ``scales`` = (q, k, v) per-tensor dequantisation scales for FP8.
    ``debug_stages`` (2, 3 or 5; bf16, head_dim 128) runs the kernel built with that depth of the K/V
    ring (``hb_debug_fa_fwd_stages``): results must not depend on it.
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
        if debug_stages is None:
            _lib.check(_lib.load().hb_fa_fwd(C.byref(a)))
        else:
            _lib.check(_lib.load().hb_debug_fa_fwd_stages(C.byref(a), int(debug_stages)))
    return (out, lse) if return_lse else out


def _bwd_args(q, k, v, o, d_o, lse, delta, causal, softmax_scale, layout):
    """Validated ``hb_fa_bwd_args`` for tensors in ``layout``; returns (args, kept-alive tensors, dims)."""
    _require_cuda(q, k, v, o, d_o, lse, delta)
    if q.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"attention backward supports bf16 and fp16, got {q.dtype}")
    for name, t in (("k", k), ("v", v), ("o", o), ("d_o", d_o)):
        if t is not None and t.dtype != q.dtype:
            raise TypeError(f"{name} has dtype {t.dtype}, q has {q.dtype}")
    if layout == "bhsd":
        b_ax, h_ax, s_ax = 0, 1, 2
    elif layout == "bshd":
        b_ax, h_ax, s_ax = 0, 2, 1
    else:
        raise ValueError(f"unknown layout {layout!r}")
    q, k, v, d_o = (_inner_contiguous(t) for t in (q, k, v, d_o))
    o = _inner_contiguous(o) if o is not None else None
    B, Hq, Sq, D = q.shape[b_ax], q.shape[h_ax], q.shape[s_ax], q.shape[3]
    Hkv, Skv = k.shape[h_ax], k.shape[s_ax]
    if k.shape[b_ax] != B or v.shape != k.shape or k.shape[3] != D or d_o.shape != q.shape or (
            o is not None and o.shape != q.shape):
        raise ValueError("shape mismatch between q, k, v, o and d_o")
    keep = [q, k, v, d_o, o]
    a = _lib.FaBwdArgs()
    a.q, a.k, a.v, a.d_o = q.data_ptr(), k.data_ptr(), v.data_ptr(), d_o.data_ptr()
    a.o = o.data_ptr() if o is not None else None
    for name, t in (("lse", lse), ("delta", delta)):
        if t is not None:
            if t.dtype != torch.float32 or tuple(t.shape) != (B, Hq, Sq) or not t.is_contiguous():
                raise ValueError(f"{name} must be a contiguous fp32 [B, Hq, Sq] = {(B, Hq, Sq)} tensor")
            setattr(a, name, t.data_ptr())
    a.B, a.Hq, a.Hkv, a.Sq, a.Skv, a.D = B, Hq, Hkv, Sq, Skv, D
    a.q_stride_b, a.q_stride_h, a.q_stride_s = q.stride(b_ax), q.stride(h_ax), q.stride(s_ax)
    a.k_stride_b, a.k_stride_h, a.k_stride_s = k.stride(b_ax), k.stride(h_ax), k.stride(s_ax)
    a.v_stride_b, a.v_stride_h, a.v_stride_s = v.stride(b_ax), v.stride(h_ax), v.stride(s_ax)
    a.do_stride_b, a.do_stride_h, a.do_stride_s = d_o.stride(b_ax), d_o.stride(h_ax), d_o.stride(s_ax)
    if o is not None:
        a.o_stride_b, a.o_stride_h, a.o_stride_s = o.stride(b_ax), o.stride(h_ax), o.stride(s_ax)
    a.causal = 1 if causal else 0
    a.softmax_scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    a.dtype = _DTYPES[q.dtype]
    a.stream = _stream_ptr(q.device)
    return a, keep, (B, Hq, Hkv, Sq, Skv, D)


def fa_bwd_preprocess(o: torch.Tensor, d_o: torch.Tensor, *, layout: str = "bhsd") -> torch.Tensor:
    """delta[b,h,q] = sum_d O * dO through ``hb_fa_bwd_preprocess``; fp32 [B, H, Sq]."""
    b_ax, h_ax, s_ax = (0, 1, 2) if layout == "bhsd" else (0, 2, 1)
    delta = torch.empty((o.shape[b_ax], o.shape[h_ax], o.shape[s_ax]), dtype=torch.float32, device=o.device)
    a, keep, _ = _bwd_args(o, o, o, o, d_o, None, delta, False, None, layout)
    with torch.cuda.device(o.device):
        _lib.check(_lib.load().hb_fa_bwd_preprocess(C.byref(a)))
    return delta


def fa_bwd_dkdv(q, k, v, d_o, lse, delta, *, causal: bool = False, softmax_scale: Optional[float] = None,
                layout: str = "bhsd") -> Tuple[torch.Tensor, torch.Tensor]:
    """dK, dV through ``hb_fa_bwd_dkdv``; contiguous [B, Hkv, Skv, D] (a transposed view for "bshd")."""
    a, keep, (B, Hq, Hkv, Sq, Skv, D) = _bwd_args(q, k, v, None, d_o, lse, delta, causal, softmax_scale, layout)
    dk = torch.empty((B, Hkv, Skv, D), dtype=q.dtype, device=q.device)
    dv = torch.empty_like(dk)
    a.dk, a.dv = dk.data_ptr(), dv.data_ptr()
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().hb_fa_bwd_dkdv(C.byref(a)))
    return (dk, dv) if layout == "bhsd" else (dk.transpose(1, 2), dv.transpose(1, 2))


def fa_bwd_dq(q, k, v, d_o, lse, delta, *, causal: bool = False, softmax_scale: Optional[float] = None,
              layout: str = "bhsd") -> torch.Tensor:
    """dQ through ``hb_fa_bwd_dq``; contiguous [B, Hq, Sq, D] (a transposed view for "bshd")."""
    a, keep, (B, Hq, Hkv, Sq, Skv, D) = _bwd_args(q, k, v, None, d_o, lse, delta, causal, softmax_scale, layout)
    dq = torch.empty((B, Hq, Sq, D), dtype=q.dtype, device=q.device)
    a.dq = dq.data_ptr()
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().hb_fa_bwd_dq(C.byref(a)))
    return dq if layout == "bhsd" else dq.transpose(1, 2)


def fa_bwd(q, k, v, o, d_o, lse, *, causal: bool = False, softmax_scale: Optional[float] = None,
           layout: str = "bhsd") -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Attention backward as preprocess -> dK, dV -> dQ (the split of the reference's
    ``create_separated_bwd_function``, Heddle/heddle/frontend/bwd_separator.py:366-455).

    ``lse`` is the natural-log LSE [B, Hq, Sq] of the forward pass.  Returns (dQ, dK, dV)."""
    lse = lse.to(torch.float32).contiguous()
    delta = fa_bwd_preprocess(o, d_o, layout=layout)
    dk, dv = fa_bwd_dkdv(q, k, v, d_o, lse, delta, causal=causal, softmax_scale=softmax_scale, layout=layout)
    dq = fa_bwd_dq(q, k, v, d_o, lse, delta, causal=causal, softmax_scale=softmax_scale, layout=layout)
    return dq, dk, dv


def status_word() -> int:
    """Device status word of the current device: 0 unless a bounded device-side wait gave up."""
    w = C.c_uint32(0)
    _lib.check(_lib.load().hb_status_word(C.byref(w)))
    return int(w.value)


def debug_wait_timeout(limit_us: int = 200):
    """Run the bounded-wait probe (``hb_debug_wait_timeout``): returns (status code, [ok0, ns0, ok1, ns1])."""
    if not torch.cuda.is_available():
        raise RuntimeError("heddle_b200 kernels need a CUDA device: there is no CPU fallback")
    status = C.c_uint32(0)
    res = (C.c_uint64 * 4)()
    _lib.check(_lib.load().hb_debug_wait_timeout(int(limit_us), C.byref(status), res))
    return int(status.value), [int(v) for v in res]


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


# Which GEMM kernel hb_gemm_epilogue runs: "auto" (CTA pairs when M > 128), "single" or "pair".
_gemm_schedule = os.environ.get("HEDDLE_B200_GEMM_SCHEDULE", "auto")


def set_gemm_schedule(name: str) -> str:
    """Select the GEMM kernel for later calls ("auto", "single", "pair"); returns the previous choice."""
    global _gemm_schedule
    if name not in _lib.GEMM_SCHEDULES:
        raise ValueError(f"unknown GEMM schedule {name!r}")
    prev, _gemm_schedule = _gemm_schedule, name
    return prev


def gemm_epilogue(a: torch.Tensor, w: torch.Tensor, epilogue: str = "none", *,
                  bias: Optional[torch.Tensor] = None, row_scale: Optional[torch.Tensor] = None,
                  residual: Optional[torch.Tensor] = None,
                  rope: Optional[Tuple[torch.Tensor, torch.Tensor, int, int]] = None,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``epilogue(a @ w.T)`` through ``hb_gemm_epilogue``.

    ``a`` is (..., K) and is viewed as [M, K]; ``w`` is [N, K] in nn.Linear layout
    ([2*N_out, K] = cat([Wg, Wu]) for "swiglu").  ``row_scale`` fp32 [M]; ``bias`` [N];
    ``residual`` (..., N_out); ``rope`` = (cos [S, hd/2] fp32, sin, head_dim, rope_cols)
    with position = row index mod S.  Returns (..., N_out) in a's dtype.
    """
    _require_cuda(a, w, bias, row_scale, residual)
    if a.dtype not in (torch.bfloat16, torch.float16) or w.dtype != a.dtype:
        raise TypeError(f"gemm_epilogue needs matching bf16/fp16 operands, got {a.dtype} and {w.dtype}")
    if epilogue not in _lib.EPILOGUES:
        raise ValueError(f"unknown epilogue {epilogue!r}")
    K = a.shape[-1]
    lead = a.shape[:-1]
    a2 = a.reshape(-1, K)
    if a2.stride(-1) != 1:
        a2 = a2.contiguous()
    if w.dim() != 2 or w.shape[1] != K:
        raise ValueError(f"weight shape {tuple(w.shape)} does not match K={K}")
    if w.stride(-1) != 1:
        w = w.contiguous()
    M, N = a2.shape[0], w.shape[0]
    n_out = N // 2 if epilogue == "swiglu" else N
    if out is None:
        out2 = torch.empty((M, n_out), dtype=a.dtype, device=a.device)
    else:
        out2 = out.reshape(-1, n_out)
        if out2.data_ptr() != out.data_ptr() or out2.stride(-1) != 1:
            raise ValueError("out must be viewable as a row-major [M, N_out] matrix")
    g = _lib.GemmArgs()
    g.a, g.w, g.out = a2.data_ptr(), w.data_ptr(), out2.data_ptr()
    g.M, g.N, g.K = M, N, K
    g.lda, g.ldw, g.ldo = a2.stride(0), w.stride(0), out2.stride(0)
    g.dtype = _DTYPES[a.dtype]
    g.epilogue = _lib.EPILOGUES[epilogue]
    keep = []
    if row_scale is not None:
        rs = row_scale.reshape(-1).to(torch.float32).contiguous()
        if rs.numel() != M:
            raise ValueError("row_scale must have one entry per row")
        keep.append(rs)
        g.row_scale = rs.data_ptr()
    if bias is not None:
        b = bias.to(a.dtype).contiguous()
        if b.numel() != N:
            raise ValueError("bias must have N entries")
        keep.append(b)
        g.bias = b.data_ptr()
    if residual is not None:
        r2 = residual.reshape(-1, n_out)
        if r2.dtype != a.dtype or r2.stride(-1) != 1:
            r2 = r2.to(a.dtype).contiguous()
        keep.append(r2)
        g.residual, g.ldr = r2.data_ptr(), r2.stride(0)
    if epilogue == "rope":
        if rope is None:
            raise ValueError("epilogue 'rope' needs rope=(cos, sin, head_dim, rope_cols)")
        cos, sin, hd, rope_cols = rope
        cos = cos.to(torch.float32).contiguous()
        sin = sin.to(torch.float32).contiguous()
        _require_cuda(cos, sin)
        keep += [cos, sin]
        g.rope_cos, g.rope_sin = cos.data_ptr(), sin.data_ptr()
        g.rope_seq, g.head_dim, g.rope_cols = cos.shape[0], int(hd), int(rope_cols)
    g.stream = _stream_ptr(a.device)
    with torch.cuda.device(a.device):
        g.schedule = _lib.GEMM_SCHEDULES[_gemm_schedule]
        _lib.check(_lib.load().hb_gemm_epilogue(C.byref(g)))
    return out2.reshape(*lead, n_out) if out is None else out


def _mult8(*values: int) -> bool:
    return all(int(v) % 8 == 0 for v in values)


def bmm(a: torch.Tensor, b: torch.Tensor, epilogue: str = "none", *, bias: Optional[torch.Tensor] = None,
        residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``epilogue(a @ b)`` for a [B, M, K] and b [B, K, N] (``torch.bmm``) in one launch of the tcgen05 GEMM:
    the batch index is part of the tile list.  ``b`` is read where it lies — row-major [K, N] slices through
    the MN-major operand path, ``w.transpose(-1, -2)`` views of [N, K] storage through the K-major one — so
    neither layout is copied.  Replaces the reference's batched kernel
    (Heddle/heddle/frontend/backend.py:491-536).  K, N and the strides must be multiples of 8 elements."""
    _require_cuda(a, b, bias, residual)
    if a.dim() != 3 or b.dim() != 3 or a.shape[0] != b.shape[0] or a.shape[2] != b.shape[1]:
        raise ValueError(f"bmm needs [B, M, K] x [B, K, N], got {tuple(a.shape)} and {tuple(b.shape)}")
    if a.dtype not in (torch.bfloat16, torch.float16) or b.dtype != a.dtype:
        raise TypeError(f"bmm needs matching bf16/fp16 operands, got {a.dtype} and {b.dtype}")
    if epilogue not in ("none", "silu", "relu", "gelu_tanh", "sigmoid", "tanh"):
        raise ValueError(f"bmm takes the unary epilogues only, not {epilogue!r}")
    Bn, M, K = a.shape
    N = b.shape[2]
    if not _mult8(K, N):
        raise ValueError(f"bmm needs K and N to be multiples of 8 (K={K}, N={N})")
    if a.stride(2) != 1 or not _mult8(a.stride(1), a.stride(0)) or a.data_ptr() % 16:
        a = a.contiguous()
    if b.stride(1) == 1 and b.stride(2) >= K and _mult8(b.stride(2), b.stride(0)) and b.data_ptr() % 16 == 0 and K > 1:
        layout, ldw = _lib.HB_W_NK, b.stride(2)   # a transposed view of [B, N, K] storage
    else:
        if b.stride(2) != 1 or not _mult8(b.stride(1), b.stride(0)) or b.data_ptr() % 16:
            b = b.contiguous()
        layout, ldw = _lib.HB_W_KN, b.stride(1)
    out = torch.empty((Bn, M, N), dtype=a.dtype, device=a.device)
    if Bn == 0 or M == 0:
        return out
    g = _lib.GemmArgs()
    g.a, g.w, g.out = a.data_ptr(), b.data_ptr(), out.data_ptr()
    g.M, g.N, g.K = M, N, K
    g.lda, g.ldw, g.ldo = a.stride(1), ldw, N
    g.dtype = _DTYPES[a.dtype]
    g.epilogue = _lib.EPILOGUES[epilogue]
    g.batch, g.w_layout = Bn, layout
    g.a_batch_stride, g.w_batch_stride, g.o_batch_stride = a.stride(0), b.stride(0), M * N
    keep = []
    if bias is not None:
        bb = bias.to(a.dtype).contiguous()
        if bb.numel() != N:
            raise ValueError("bias must have N entries")
        keep.append(bb)
        g.bias = bb.data_ptr()
    if residual is not None:
        r = residual.to(a.dtype).expand(Bn, M, N).contiguous()
        keep.append(r)
        g.residual, g.ldr, g.r_batch_stride = r.data_ptr(), N, M * N
    g.stream = _stream_ptr(a.device)
    with torch.cuda.device(a.device):
        g.schedule = _lib.GEMM_SCHEDULES[_gemm_schedule]
        _lib.check(_lib.load().hb_gemm_epilogue(C.byref(g)))
    return out


def gemm(a: torch.Tensor, b: torch.Tensor, epilogue: str = "none", *, bias: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``epilogue(a @ b)`` for a (..., K) and b [K, N] (``torch.mm`` / ``matmul`` with a 2-D right operand);
    the counterpart of the reference's plain GEMM (Heddle/heddle/frontend/backend.py:227-272)."""
    if b.dim() != 2 or a.shape[-1] != b.shape[0]:
        raise ValueError(f"gemm needs (..., K) x [K, N], got {tuple(a.shape)} and {tuple(b.shape)}")
    lead = a.shape[:-1]
    r = None if residual is None else residual.reshape(1, -1, b.shape[1])
    out = bmm(a.reshape(1, -1, a.shape[-1]), b.unsqueeze(0), epilogue, bias=bias, residual=r)
    return out.reshape(*lead, b.shape[1])


def rms_rowstat(x: torch.Tensor, residual: Optional[torch.Tensor] = None, eps: float = 1e-5,
                write_sum: bool = False) -> "Tuple[Optional[torch.Tensor], torch.Tensor]":
    """Row statistic of RMSNorm fused with the residual add (``hb_rms_rowstat``).

    Returns (y, rstd): y = x + residual in x's dtype (None unless ``write_sum`` or a
    residual is given), rstd fp32 of shape x.shape[:-1]."""
    _require_cuda(x, residual)
    N = x.shape[-1]
    x2 = x.reshape(-1, N)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    M = x2.shape[0]
    r2 = None
    if residual is not None:
        r2 = residual.reshape(-1, N)
        if r2.stride() != x2.stride() or r2.dtype != x.dtype:
            r2 = r2.to(x.dtype).contiguous()
            x2 = x2.contiguous()
    y = torch.empty_like(x2) if (write_sum or residual is not None) else None
    if y is not None and y.stride() != x2.stride():
        x2 = x2.contiguous()
        y = torch.empty_like(x2)
    rstd = torch.empty((M,), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().hb_rms_rowstat(x2.data_ptr(), r2.data_ptr() if r2 is not None else None,
                                              y.data_ptr() if y is not None else None, rstd.data_ptr(), M, N,
                                              x2.stride(0), float(eps), _DTYPES[x.dtype], _stream_ptr(x.device)))
    return (y.reshape(x.shape) if y is not None else None), rstd.reshape(x.shape[:-1])


def prepare_weight(weights: "Sequence[torch.Tensor]", gamma: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Stack up to four ``[rows_i, K]`` weights along the rows and fold ``gamma`` ([K]) into the
    columns in one pass (``hb_prepare_weight``): the operand ``gemm_epilogue`` takes for merged
    projections, SwiGLU (``[Wg; Wu]``) and RMSNorm-folded GEMMs."""
    ws = list(weights)
    if not 1 <= len(ws) <= 4:
        raise ValueError("prepare_weight takes 1 to 4 weights")
    _require_cuda(*ws, gamma)
    K, dt = ws[0].shape[1], ws[0].dtype
    for w in ws:
        if w.dim() != 2 or w.shape[1] != K or w.dtype != dt:
            raise ValueError("prepare_weight: weights must be 2-D with the same K and dtype")
    ws = [w if w.stride(1) == 1 else w.contiguous() for w in ws]
    if gamma is not None:
        gamma = gamma.to(dt).contiguous()
    out = torch.empty((sum(w.shape[0] for w in ws), K), dtype=dt, device=ws[0].device)
    a = _lib.PrepareArgs()
    for i, w in enumerate(ws):
        a.src[i], a.rows[i], a.ld_src[i] = w.data_ptr(), w.shape[0], w.stride(0)
    a.n_src, a.K = len(ws), K
    a.gamma = gamma.data_ptr() if gamma is not None else None
    a.out, a.ld_out, a.dtype = out.data_ptr(), out.stride(0), _DTYPES[dt]
    a.stream = _stream_ptr(out.device)
    with torch.cuda.device(out.device):
        _lib.check(_lib.load().hb_prepare_weight(C.byref(a)))
    return out


def row_softmax(x: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """softmax(scale * x) over the last dimension (``hb_row_softmax``): bf16 / fp16, last dimension a
    multiple of 8 and at most 16384."""
    _require_cuda(x)
    cols = x.shape[-1]
    x2 = x.reshape(-1, cols)
    if x2.stride(-1) != 1 or (x2.shape[0] > 1 and x2.stride(0) % 8 != 0) or x2.data_ptr() % 16 != 0:
        x2 = x2.contiguous()
    y = torch.empty((x2.shape[0], cols), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().hb_row_softmax(x2.data_ptr(), y.data_ptr(), x2.shape[0], cols, max(x2.stride(0), cols),
                                              cols, float(scale), _DTYPES[x.dtype], _stream_ptr(x.device)))
    return y.reshape(x.shape)


def rowwise_program(program, inputs=(), rowvecs=(), rowscalars=(), n_outputs: int = 1, mode: str = "auto"):
    """Run an accumulator-machine program over [rows, cols] views of ``inputs`` (``hb_rowwise_program``).

    ``program`` is a sequence of ``(op, src, index, imm)`` tuples with the names of ``_lib.EW_OPS`` /
    ``_lib.EW_SRCS`` (``src`` may be None for unary ops).  ``inputs`` are 16-bit tensors of one shape
    (..., cols); ``rowvecs`` are [cols] vectors; ``rowscalars`` are tensors with one value per row
    (shape (..., 1) or (...)), converted to fp32.  Returns ``n_outputs`` new tensors shaped like the
    inputs (a tuple when ``n_outputs`` > 1).  ``mode``: "auto" (a kernel compiled for this program at
    run time and cached; the interpreter kernel where NVRTC cannot be loaded), "interpret" or "compiled"."""
    if not inputs:
        raise ValueError("rowwise_program needs at least one full-size input")
    _require_cuda(*inputs, *rowvecs, *rowscalars)
    x0 = inputs[0]
    if x0.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"rowwise_program takes bf16/fp16 tensors, got {x0.dtype}")
    cols = x0.shape[-1]
    shape = tuple(x0.shape)
    a = _lib.RowwiseArgs()
    keep = []
    if len(inputs) > _lib.EW_MAX_INPUTS or len(rowvecs) > _lib.EW_MAX_ROWVEC or len(rowscalars) > _lib.EW_MAX_ROWSCALAR \
            or not 1 <= n_outputs <= _lib.EW_MAX_OUTPUTS or not 1 <= len(program) <= _lib.EW_MAX_INST:
        raise ValueError("rowwise_program: too many operands or instructions")
    for i, t in enumerate(inputs):
        if tuple(t.shape) != shape or t.dtype != x0.dtype:
            raise ValueError("rowwise_program: full-size inputs must share shape and dtype")
        t2 = t.reshape(-1, cols)
        if t2.stride(-1) != 1 or t2.stride(0) % 8 or t2.data_ptr() % 16:
            t2 = t2.contiguous()
        keep.append(t2)
        a.inputs[i], a.ld_in[i] = t2.data_ptr(), t2.stride(0)
    rows = keep[0].shape[0]
    for i, t in enumerate(rowvecs):
        t2 = t.reshape(-1).to(x0.dtype).contiguous()
        if t2.numel() != cols:
            raise ValueError("rowwise_program: a row vector must have cols entries")
        keep.append(t2)
        a.rowvec[i] = t2.data_ptr()
    for i, t in enumerate(rowscalars):
        t2 = t.reshape(-1).to(torch.float32).contiguous()
        if t2.numel() != rows:
            raise ValueError("rowwise_program: a per-row vector must have one entry per row")
        keep.append(t2)
        a.rowscalar[i] = t2.data_ptr()
    outs = [torch.empty(shape, dtype=x0.dtype, device=x0.device) for _ in range(n_outputs)]
    for i, o in enumerate(outs):
        a.outputs[i], a.ld_out[i] = o.data_ptr(), cols
    a.n_inputs, a.n_rowvec, a.n_rowscalar, a.n_outputs = len(inputs), len(rowvecs), len(rowscalars), n_outputs
    a.rows, a.cols, a.dtype, a.n_inst = rows, cols, _DTYPES[x0.dtype], len(program)
    for pc, (op, src, index, imm) in enumerate(program):
        a.program[pc].op = _lib.EW_OPS[op]
        a.program[pc].src = _lib.EW_SRCS[src or "none"]
        a.program[pc].index = int(index)
        a.program[pc].imm = float(imm)
    a.stream = _stream_ptr(x0.device)
    a.mode = {"auto": _lib.ROWWISE_AUTO, "interpret": _lib.ROWWISE_INTERPRET, "compiled": _lib.ROWWISE_COMPILED}[mode]
    with torch.cuda.device(x0.device):
        _lib.check(_lib.load().hb_rowwise_program(C.byref(a)))
    return outs[0] if n_outputs == 1 else tuple(outs)


def h2o_score(q: torch.Tensor, k: torch.Tensor, lse: torch.Tensor, *, causal: bool = True,
              softmax_scale: Optional[float] = None, layout: str = "bhsd") -> torch.Tensor:
    """H2O score through ``hb_h2o_score``: score[b,h,j] = sum_i exp(s_ij - lse_i), fp32 [B, Hq, Skv].

    ``lse`` is the natural-log LSE [B, Hq, Sq] that ``fa_fwd(..., return_lse=True)`` returns."""
    _require_cuda(q, k, lse)
    if q.dtype not in (torch.bfloat16, torch.float16) or k.dtype != q.dtype:
        raise TypeError(f"unsupported or mismatched dtypes: {q.dtype}, {k.dtype}")
    q, k = _inner_contiguous(q), _inner_contiguous(k)
    b_ax, h_ax, s_ax = (0, 1, 2) if layout == "bhsd" else (0, 2, 1)
    B, Hq, Sq, D = q.shape[b_ax], q.shape[h_ax], q.shape[s_ax], q.shape[3]
    Hkv, Skv = k.shape[h_ax], k.shape[s_ax]
    lse = lse.to(torch.float32).contiguous()
    if tuple(lse.shape) != (B, Hq, Sq):
        raise ValueError(f"lse must be [B, Hq, Sq] = {(B, Hq, Sq)}, got {tuple(lse.shape)}")
    score = torch.empty((B, Hq, Skv), dtype=torch.float32, device=q.device)
    a = _lib.H2oArgs()
    a.q, a.k, a.lse, a.score = q.data_ptr(), k.data_ptr(), lse.data_ptr(), score.data_ptr()
    a.B, a.Hq, a.Hkv, a.Sq, a.Skv, a.D = B, Hq, Hkv, Sq, Skv, D
    a.q_stride_b, a.q_stride_h, a.q_stride_s = q.stride(b_ax), q.stride(h_ax), q.stride(s_ax)
    a.k_stride_b, a.k_stride_h, a.k_stride_s = k.stride(b_ax), k.stride(h_ax), k.stride(s_ax)
    a.causal = 1 if causal else 0
    a.softmax_scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    a.dtype = _DTYPES[q.dtype]
    a.stream = _stream_ptr(q.device)
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().hb_h2o_score(C.byref(a)))
    return score
