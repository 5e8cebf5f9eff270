"""hb_fa_fwd_noalloc — the FlashAttention-forward entry point for hosts that may not
allocate device memory (fixed memory budget, allocation forbidden after start-up, or a
call site where cudaMalloc is not permitted).  It must give the same result as
hb_fa_fwd while keeping its scratch (the kernel's status word) in a static device array
of the library, and its status must be readable without an allocation
(hb_status_word_noalloc).

The file sorts last on purpose: if it fails under ``pytest -x`` every other test has run.
It passes both alone in a fresh process (the first library call is then the no-alloc one)
and after the rest of the suite.
"""
import ctypes as C
import math

import pytest
import torch

from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu


def _args(_lib, q, k, v, out, lse, causal):
    a = _lib.FaArgs()
    a.q, a.k, a.v, a.o, a.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr()
    a.B, a.Hq, a.Sq, a.D = q.shape
    a.Hkv, a.Skv = k.shape[1], k.shape[2]
    for name, t in (("q", q), ("k", k), ("v", v), ("o", out)):
        setattr(a, f"{name}_stride_b", t.stride(0))
        setattr(a, f"{name}_stride_h", t.stride(1))
        setattr(a, f"{name}_stride_s", t.stride(2))
    a.causal = 1 if causal else 0
    a.softmax_scale = 1.0 / math.sqrt(q.shape[-1])
    a.dtype = _lib.HB_BF16 if q.dtype == torch.bfloat16 else _lib.HB_FP16
    a.stream = torch.cuda.current_stream().cuda_stream
    return a


def _status(built_lib):
    w = C.c_uint32(0xFFFFFFFF)
    rc = built_lib.hb_status_word_noalloc(C.byref(w), torch.cuda.current_stream().cuda_stream)
    return rc, int(w.value)


def test_noalloc_entry_matches_hb_fa_fwd_twice_in_a_row(built_lib):
    from heddle_b200 import _lib, ops

    gen = torch.Generator(device="cuda").manual_seed(42)
    shapes = [((2, 4, 2, 640, 640, 128), True, torch.bfloat16), ((1, 2, 2, 300, 500, 64), False, torch.float16)]
    for call, ((B, Hq, Hkv, Sq, Skv, D), causal, dt) in enumerate(shapes):
        q = torch.randn(B, Hq, Sq, D, generator=gen, device="cuda").to(dt)
        k = torch.randn(B, Hkv, Skv, D, generator=gen, device="cuda").to(dt)
        v = torch.randn(B, Hkv, Skv, D, generator=gen, device="cuda").to(dt)
        # every buffer is the caller's: the entry point itself allocates nothing
        out = torch.full_like(q, float("nan"))
        lse = torch.full((B, Hq, Sq), float("nan"), dtype=torch.float32, device="cuda")
        a = _args(_lib, q, k, v, out, lse, causal)
        rc = built_lib.hb_fa_fwd_noalloc(C.byref(a))
        assert rc == _lib.HB_OK, built_lib.hb_last_error()
        torch.cuda.synchronize()
        assert _status(built_lib) == (_lib.HB_OK, 0)
        # against the CPU oracle (the pinned restatement of the reference's eager graph) ...
        ref, ref_l = O.attention_eager(q.cpu(), k.cpu(), v.cpu(), causal=causal)
        assert not torch.isnan(out.float()).any(), f"call {call}: output not fully written"
        assert (out.float().cpu() - ref).abs().max().item() <= 2e-2
        assert (lse.cpu() - ref_l).abs().max().item() <= 1e-3
        # ... and against the existing entry point: same kernel, same inputs, in fact bit-identical
        ref_out, ref_lse = ops.fa_fwd(q, k, v, causal=causal, return_lse=True)
        torch.cuda.synchronize()
        assert torch.equal(out, ref_out) and torch.equal(lse, ref_lse)

    # immediately repeated calls on the same buffers (the shared scratch keeps its contents), and
    # the property the entry point exists for: the device's free memory does not move
    out2 = torch.empty_like(out)
    a2 = _args(_lib, q, k, v, out2, lse, causal)
    assert built_lib.hb_fa_fwd_noalloc(C.byref(a2)) == _lib.HB_OK  # set-up done before measuring
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(4):
        assert built_lib.hb_fa_fwd_noalloc(C.byref(a2)) == _lib.HB_OK
    assert _status(built_lib) == (_lib.HB_OK, 0)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "hb_fa_fwd_noalloc / hb_status_word_noalloc changed the device's free memory"
    assert torch.equal(out2, out)


def test_noalloc_entry_rejects_what_it_cannot_take(built_lib):
    from heddle_b200 import _lib

    q = torch.zeros(1, 1, 128, 128, dtype=torch.bfloat16, device="cuda")
    lse = torch.zeros(1, 1, 128, dtype=torch.float32, device="cuda")
    a = _args(_lib, q, q, q, torch.empty_like(q), lse, False)
    a.B = 70000
    a.Hq = a.Hkv = 70000  # 4.9e9 query blocks: beyond the per-call limit
    assert built_lib.hb_fa_fwd_noalloc(C.byref(a)) == _lib.HB_ERR_UNSUPPORTED
    assert b"too large" in built_lib.hb_last_error()
    a = _args(_lib, q, q, q, torch.empty_like(q), lse, False)
    a.dtype = _lib.HB_FP8_E4M3
    assert built_lib.hb_fa_fwd_noalloc(C.byref(a)) == _lib.HB_ERR_UNSUPPORTED
    # misaligned output, misaligned lse
    a = _args(_lib, q, q, q, torch.empty_like(q), lse, False)
    a.o = a.o + 2
    assert built_lib.hb_fa_fwd_noalloc(C.byref(a)) == _lib.HB_ERR_ALIGN
    a = _args(_lib, q, q, q, torch.empty_like(q), lse, False)
    a.lse = a.lse + 2
    assert built_lib.hb_fa_fwd_noalloc(C.byref(a)) == _lib.HB_ERR_ALIGN
    # causal with fewer keys than queries
    a = _args(_lib, q, q, q, torch.empty_like(q), lse, True)
    a.Skv = 64
    assert built_lib.hb_fa_fwd_noalloc(C.byref(a)) == _lib.HB_ERR_UNSUPPORTED
    assert b"Skv >= Sq" in built_lib.hb_last_error()
    # the status reader needs somewhere to write
    assert built_lib.hb_status_word_noalloc(None, None) == _lib.HB_ERR_BAD_ARG
