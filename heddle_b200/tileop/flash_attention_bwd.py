"""Backward kernel factories with the calling protocol the reference sketches for
``heddle.tileop.flash_attention_bwd`` (named in Heddle/heddle/frontend/bwd_separator.py:388-392;
the reference ships the interface, not the kernels):

    delta  = flashattn_bwd_preprocess(B, H, T, D)(O, dO)
    dK, dV = flashattn_bwd_dkdv(B, H, Tq, Tkv, D, is_causal=..., ...)(Q, K, V, O, dO, LSE, delta)
    dQ     = flashattn_bwd_dq(B, H, Tq, Tkv, D, is_causal=..., ...)(Q, K, V, O, dO, LSE, delta)

Tensors are [B, H, S, D]; LSE is what ``flashattn_lse`` returns — fp32 ``[B, H, Sq, 1]`` in the
log2 domain — or the natural-log ``[B, H, Sq]`` of ``ops.fa_fwd(..., return_lse=True)`` when
``lse_log2=False``; delta is fp32 ``[B, H, Sq]``.  The tile / stage / thread arguments are accepted
for signature compatibility and ignored.  K/V may carry fewer heads than Q.
"""
from __future__ import annotations

import math

import torch

from .. import ops

LN2 = 0.6931471805599453


def _natural_lse(LSE: torch.Tensor, lse_log2: bool) -> torch.Tensor:
    lse = LSE.squeeze(-1) if LSE.dim() == 4 else LSE
    lse = lse.to(torch.float32)
    return (lse * LN2 if lse_log2 else lse).contiguous()


def flashattn_bwd_preprocess(batch, heads, seq_len, dim):
    """Returns ``kernel(O, dO) -> delta`` with delta = rowsum(O * dO) (bwd_separator.py:379, :430-431)."""

    def kernel(O: torch.Tensor, dO: torch.Tensor) -> torch.Tensor:
        if tuple(O.shape) != (batch, heads, seq_len, dim) or dO.shape != O.shape:
            raise ValueError(f"O / dO have shapes {tuple(O.shape)} / {tuple(dO.shape)}, "
                             f"kernel was built for {(batch, heads, seq_len, dim)}")
        return ops.fa_bwd_preprocess(O, dO)

    return kernel


def flashattn_bwd_dkdv(batch, heads, seq_q, seq_kv, dim, is_causal=False, block_M=64, block_N=128, num_stages=2,
                       threads=128, lse_log2=True):
    """Returns ``kernel(Q, K, V, O, dO, LSE, delta) -> (dK, dV)``: one CTA per key tile loops over the
    query tiles, so dK and dV are written exclusively (bwd_separator.py:433-441)."""
    if seq_kv - seq_q < 0 and is_causal:
        raise AssertionError("seq_kv must be greater than or equal to seq_q")

    def kernel(Q, K, V, O, dO, LSE, delta):
        if tuple(Q.shape) != (batch, heads, seq_q, dim) or K.shape[2] != seq_kv:
            raise ValueError(f"Q / K have shapes {tuple(Q.shape)} / {tuple(K.shape)}, kernel was built for "
                             f"{(batch, heads, seq_q, dim)} and seq_kv={seq_kv}")
        return ops.fa_bwd_dkdv(Q, K, V, dO, _natural_lse(LSE, lse_log2), delta, causal=bool(is_causal),
                               softmax_scale=1.0 / math.sqrt(dim))

    return kernel


def flashattn_bwd_dq(batch, heads, seq_q, seq_kv, dim, is_causal=False, block_M=128, block_N=64, num_stages=2,
                     threads=128, lse_log2=True):
    """Returns ``kernel(Q, K, V, O, dO, LSE, delta) -> dQ``: one CTA per query tile loops over the key
    tiles (bwd_separator.py:443-451)."""
    if seq_kv - seq_q < 0 and is_causal:
        raise AssertionError("seq_kv must be greater than or equal to seq_q")

    def kernel(Q, K, V, O, dO, LSE, delta):
        if tuple(Q.shape) != (batch, heads, seq_q, dim) or K.shape[2] != seq_kv:
            raise ValueError(f"Q / K have shapes {tuple(Q.shape)} / {tuple(K.shape)}, kernel was built for "
                             f"{(batch, heads, seq_q, dim)} and seq_kv={seq_kv}")
        return ops.fa_bwd_dq(Q, K, V, dO, _natural_lse(LSE, lse_log2), delta, causal=bool(is_causal),
                             softmax_scale=1.0 / math.sqrt(dim))

    return kernel
