"""Factory mirroring Heddle/heddle/tileop/h2o_attention.py:27 (``h2o_score``)."""
from __future__ import annotations

import math

import torch

from .. import ops

LN2 = 0.6931471805599453


def h2o_score(batch, heads, seq_q, seq_kv, dim, is_causal, block_M=128, block_N=128, num_stages=2, threads=256):
    """Returns ``kernel(Q, K, LSE) -> score[B, H, Skv]`` (fp32).

    LSE is ``[B, H, Sq, 1]`` fp32 in the log2 domain, as ``flashattn_lse`` produces it
    (h2o_attention.py:38-39); score[b,h,k] = sum_q exp2(score_qk * scale - LSE_q).
    """

    def kernel(Q: torch.Tensor, K: torch.Tensor, LSE: torch.Tensor) -> torch.Tensor:
        lse_nat = (LSE.reshape(batch, heads, seq_q) * LN2).contiguous()
        return ops.h2o_score(Q, K, lse_nat, causal=bool(is_causal), softmax_scale=1.0 / math.sqrt(dim))

    return kernel
