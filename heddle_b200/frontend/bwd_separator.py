"""Backward-pass separation: configuration, the shape heuristic and the three-kernel backward
function (Heddle/heddle/frontend/bwd_separator.py).

The reference decides between a "unified" backward kernel (atomic adds into dQ) and a "separated"
one (dK/dV kernel + dQ kernel, exclusive writes), and sketches the separated interface
(:366-455).  Here only the separated kernels exist — on sm_100a both accumulators of the dK/dV
kernel and the one of the dQ kernel live in TMEM and nothing is accumulated through memory — so
``should_separate_bwd`` keeps the reference's decision rule for callers that log or test it, and
``TileLangFlashAttnFunc.backward`` uses the separated kernels for every shape.  The graph-level
splitter is a placeholder in the reference (:330-359, raises NotImplementedError) and is the same
here.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from enum import Enum
from typing import Callable, Optional, Tuple

import torch


class BWDSeparationMode(Enum):
    AUTO = "auto"
    UNIFIED = "unified"
    SEPARATED = "separated"


@dataclass
class BWDSeparationConfig:
    """Same fields, defaults and environment variables as bwd_separator.py:56-91."""
    mode: BWDSeparationMode = BWDSeparationMode.AUTO
    min_seq_len_for_separation: int = 1024
    min_batch_heads: int = 4
    dkdv_block_m: int = 64
    dkdv_block_n: int = 128
    dkdv_num_stages: int = 2
    dkdv_threads: int = 128
    dq_block_m: int = 128
    dq_block_n: int = 64
    dq_num_stages: int = 2
    dq_threads: int = 128

    @classmethod
    def from_env(cls) -> "BWDSeparationConfig":
        name = os.environ.get("TILELANG_BWD_SEPARATION_MODE", "auto").strip().lower()
        mode = {m.value: m for m in BWDSeparationMode}.get(name, BWDSeparationMode.AUTO)
        return cls(mode=mode,
                   min_seq_len_for_separation=int(os.environ.get("TILELANG_BWD_MIN_SEQ_FOR_SEP", "1024")),
                   min_batch_heads=int(os.environ.get("TILELANG_BWD_MIN_BATCH_HEADS", "4")))


def should_separate_bwd(B: int, H: int, T: int, D: int, config: Optional[BWDSeparationConfig] = None) -> bool:
    """The reference's rule (bwd_separator.py:94-138): forced by the mode, else separated for
    T >= 4096, never below the sequence / batch*heads thresholds, and for B*H >= 8 in between."""
    if config is None:
        config = BWDSeparationConfig.from_env()
    if config.mode == BWDSeparationMode.UNIFIED:
        return False
    if config.mode == BWDSeparationMode.SEPARATED:
        return True
    if T < config.min_seq_len_for_separation or B * H < config.min_batch_heads:
        return False
    if T >= 4096:
        return True
    return B * H >= 8


def split_bwd_graph(gm):
    """Graph-level splitting is a placeholder in the reference as well (bwd_separator.py:330-359)."""
    raise NotImplementedError("Graph-level BWD splitting is not implemented; use the autograd.Function "
                              "route (TileLangFlashAttnFunc.backward)")


def create_separated_bwd_function(flashattn_bwd_preprocess: Callable, flashattn_bwd_dkdv: Callable,
                                  flashattn_bwd_dq: Callable) -> Callable:
    """Wraps the three kernel factories into ``separated_bwd(Q, K, V, O, grad_out, LSE, is_causal=False,
    config=None) -> (dQ, dK, dV)``: preprocess -> dK, dV -> dQ (bwd_separator.py:366-455)."""

    def separated_bwd(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, O: torch.Tensor, grad_out: torch.Tensor,
                      LSE: torch.Tensor, is_causal: bool = False,
                      config: Optional[BWDSeparationConfig] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        if config is None:
            config = BWDSeparationConfig.from_env()
        B, H, T, D = Q.shape
        Tkv = K.shape[2]
        delta = flashattn_bwd_preprocess(B, H, T, D)(O, grad_out)
        dK, dV = flashattn_bwd_dkdv(B, H, T, Tkv, D, is_causal=is_causal, block_M=config.dkdv_block_m,
                                    block_N=config.dkdv_block_n, num_stages=config.dkdv_num_stages,
                                    threads=config.dkdv_threads)(Q, K, V, O, grad_out, LSE, delta)
        dQ = flashattn_bwd_dq(B, H, T, Tkv, D, is_causal=is_causal, block_M=config.dq_block_m,
                              block_N=config.dq_block_n, num_stages=config.dq_num_stages,
                              threads=config.dq_threads)(Q, K, V, O, grad_out, LSE, delta)
        return dQ, dK, dV

    return separated_bwd
