"""Kernel factories with the reference's calling protocol (Heddle/heddle/tileop/)."""
from .flash_attention import flashattn, flashattn_lse  # noqa: F401
from .h2o_attention import h2o_score  # noqa: F401
from .flash_attention_bwd import flashattn_bwd_preprocess, flashattn_bwd_dkdv, flashattn_bwd_dq  # noqa: F401
