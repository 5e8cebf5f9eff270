"""Factories mirroring Heddle/heddle/tileop/flash_attention.py.

``flashattn(batch, heads, seq_q, seq_kv, dim, is_causal, ...)`` returns a callable
``kernel(Q, K, V) -> O`` and ``flashattn_lse(...)`` a callable ``kernel(Q, K, V) ->
(LSE, O)`` exactly like the reference's ``tilelang.jit`` objects (outputs allocated by
the callee; LSE first, flash_attention.py:149,254-255).  The tile / stage / thread
arguments are accepted for signature compatibility and ignored: the sm_100a kernel has
one fixed schedule.

Differences from the reference, which is fp16-only and MHA-only: bf16 is accepted, and
K/V may carry fewer heads than Q.  LSE keeps the reference's convention here —
``[B, H, Sq, 1]`` fp32 in the log2 domain, log2(sum(exp2(score * scale)))
(flash_attention.py:295-298) — so ``h2o_score`` consumes it unchanged.
"""
from __future__ import annotations

import math

import torch

from .. import ops

LOG2E = 1.4426950408889634


def _check(Q, K, batch, heads, seq_q, seq_kv, dim):
    if tuple(Q.shape) != (batch, heads, seq_q, dim):
        raise ValueError(f"Q has shape {tuple(Q.shape)}, kernel was built for {(batch, heads, seq_q, dim)}")
    if K.shape[0] != batch or K.shape[2] != seq_kv or K.shape[3] != dim:
        raise ValueError(f"K has shape {tuple(K.shape)}, kernel was built for seq_kv={seq_kv}, dim={dim}")


def flashattn(batch, heads, seq_q, seq_kv, dim, is_causal, block_M=128, block_N=128, num_stages=2, threads=256):
    """Heddle/heddle/tileop/flash_attention.py:20 — returns ``kernel(Q, K, V) -> O`` on [B,H,S,D]."""
    if seq_kv - seq_q < 0 and is_causal:
        raise AssertionError("seq_kv must be greater than or equal to seq_q")

    def kernel(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor) -> torch.Tensor:
        _check(Q, K, batch, heads, seq_q, seq_kv, dim)
        return ops.fa_fwd(Q, K, V, causal=bool(is_causal), softmax_scale=1.0 / math.sqrt(dim))

    return kernel


def flashattn_lse(batch, heads, seq_q, seq_kv, dim, is_causal, block_M=128, block_N=128, num_stages=2, threads=256):
    """Heddle/heddle/tileop/flash_attention.py:158 — returns ``kernel(Q, K, V) -> (LSE, O)``."""
    if seq_kv - seq_q < 0 and is_causal:
        raise AssertionError("seq_kv must be greater than or equal to seq_q")

    def kernel(Q, K, V):
        _check(Q, K, batch, heads, seq_q, seq_kv, dim)
        out, lse = ops.fa_fwd(Q, K, V, causal=bool(is_causal), softmax_scale=1.0 / math.sqrt(dim), return_lse=True)
        return (lse * LOG2E).unsqueeze(-1), out

    return kernel
