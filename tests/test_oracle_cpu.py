"""The CPU oracle against the reference-generated golden fixtures and against itself."""
import math

import pytest
import torch

from oracle import attention_oracle as O


def _inputs(case):
    B, Hq, Hkv, Sq, Skv, D = case["shape"]
    dt = getattr(torch, case["in_dtype"])
    q, k, v = O.make_qkv(B, Hq, Hkv, Sq, Skv, D, seed=case["seed"], dtype=dt)
    chk = float(q.double().sum() + k.double().sum() + v.double().sum())
    assert chk == pytest.approx(case["checksum"], rel=1e-12), "seeded generator drifted from the fixture"
    return q, k, v


@pytest.mark.parametrize("name", ["c1", "causal_ragged", "causal_512"])
def test_eager_oracle_matches_reference_capture(golden, name):
    case = golden[name]
    q, k, v = _inputs(case)
    out, _ = O.attention_eager(q, k, v, causal=case["causal"])
    ref = case["out"].float()
    tol = 2e-6 if case["out"].dtype == torch.float32 else 8e-3  # bf16-stored fixture
    assert (out - ref).abs().max().item() <= tol


@pytest.mark.parametrize("name", ["causal_ragged", "causal_512"])
def test_tiled_oracle_matches_reference_capture(golden, name):
    """The kernel-algorithm restatement (bf16 P, exp2 domain) stays within the bf16 tolerance."""
    case = golden[name]
    q, k, v = _inputs(case)
    out, lse2 = O.flashattn_tiled(q, k, v, case["causal"])
    assert (out.float() - case["out"].float()).abs().max().item() <= 2e-2
    _, lse = O.attention_eager(q, k, v, causal=case["causal"])
    assert (lse2 * O.LN2 - lse).abs().max().item() <= 1e-4


@pytest.mark.parametrize("block", [(64, 64), (128, 128), (128, 64)])
def test_tiled_oracle_block_size_invariance(block):
    q, k, v = O.make_qkv(1, 2, 1, 130, 300, 64, seed=7, dtype=torch.float16)
    a, la = O.flashattn_tiled(q, k, v, True, block_M=block[0], block_N=block[1])
    b, lb = O.attention_eager(q, k, v, True)
    assert (a.float() - b).abs().max().item() <= 3e-3
    assert (la * O.LN2 - lb).abs().max().item() <= 1e-4


def test_eager_matches_torch_sdpa():
    q, k, v = O.make_qkv(2, 4, 4, 96, 96, 64, seed=3)
    out, lse = O.attention_eager(q, k, v, causal=True)
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
    assert (out - ref).abs().max().item() <= 2e-6
    s = (q @ k.transpose(-2, -1)) / math.sqrt(64) + O.causal_mask(96, 96)
    assert (lse - torch.logsumexp(s, -1)).abs().max().item() <= 2e-6


def test_gqa_matches_repeated_heads():
    q, k, v = O.make_qkv(1, 8, 2, 64, 64, 64, seed=5)
    a, _ = O.attention_eager(q, k, v, causal=True)
    b, _ = O.attention_eager(q, k.repeat_interleave(4, 1), v.repeat_interleave(4, 1), causal=True)
    assert torch.equal(a, b)


def test_h2o_score_columns_sum_to_rows():
    q, k, v = O.make_qkv(1, 2, 2, 80, 80, 64, seed=9)
    _, lse = O.attention_eager(q, k, v, causal=True)
    score = O.h2o_score(q, k, lse, causal=True)
    # probabilities of every query row sum to 1, so the scores sum to Sq
    assert score.sum(-1) == pytest.approx(torch.full((1, 2), 80.0), abs=1e-3)
    # reference fallback formula (backend.py:186-201)
    s = (q @ k.transpose(-2, -1)) / math.sqrt(64) + O.causal_mask(80, 80)
    assert (score - torch.softmax(s, -1).sum(-2)).abs().max().item() <= 1e-5


def test_h2o_matches_reference_capture(golden):
    """The H2O structure run eagerly by the reference's own backend (fusion off): attention output and
    the column sums of the probabilities, keys longer than queries."""
    case = golden["h2o"]
    B, Hq, Hkv, Sq, Skv, D = case["shape"]
    q, k, v = O.make_qkv(B, Hq, Hkv, Sq, Skv, D, seed=case["seed"], dtype=torch.bfloat16)
    assert float(q.double().sum() + k.double().sum() + v.double().sum()) == pytest.approx(case["checksum"], rel=1e-12)
    out, lse = O.attention_eager(q, k, v, causal=True)
    assert (out - case["out"]).abs().max().item() <= 2e-6
    score = O.h2o_score(q, k, lse, causal=True)
    assert score.shape == case["score"].shape
    assert (score - case["score"]).abs().max().item() <= 1e-5


def test_gemm_epilogues_match_reference_capture(golden):
    gm = golden["gemm"]
    g = torch.Generator().manual_seed(gm["seed"])
    x = torch.randn(96, 128, generator=g).to(torch.bfloat16)
    w = (torch.randn(192, 128, generator=g) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(192, 128, generator=g) * 0.05).to(torch.bfloat16)
    assert float(x.double().sum() + w.double().sum() + w2.double().sum()) == pytest.approx(gm["checksum"], rel=1e-12)
    for act in ("none", "silu", "relu", "gelu_tanh", "sigmoid", "tanh"):
        out = O.gemm_epilogue(x.float(), w.float(), act)
        assert (out - gm[act]).abs().max().item() <= 2e-5, act
    out = O.gemm_epilogue(x.float(), torch.cat([w, w2]).float(), "swiglu")
    assert (out - gm["swiglu"]).abs().max().item() <= 2e-5


def test_llama_layer_matches_reference_capture(golden):
    case = golden["llama_small"]
    layer = O.LlamaLayer(hidden=256, heads=2, inter=512).init_weights(seed=case["seed"])
    for p in layer.parameters():
        p.data = p.data.to(torch.bfloat16).float()
    x = torch.randn(2, 128, 256, generator=torch.Generator().manual_seed(case["x_seed"])).to(torch.bfloat16).float()
    assert float(x.double().sum()) == pytest.approx(case["checksum"], rel=1e-12)
    with torch.no_grad():
        out = layer(x)
    assert (out - case["out"]).abs().max().item() <= 5e-5


def test_rope_epilogue_matches_rotate_half():
    g = torch.Generator().manual_seed(11)
    a = torch.randn(24, 32, generator=g)
    w = torch.randn(64, 32, generator=g)
    cos, sin = O.rope_tables(8, 32)
    out = O.gemm_epilogue(a, w, "rope", rope=(cos, sin, 32, 64))
    y = (a @ w.t()).view(3, 8, 2, 32).transpose(1, 2)  # [B=3, H=2, S=8, D=32]
    ref = O.rotate_half_rope(y, cos, sin).transpose(1, 2).reshape(24, 64)
    assert (out - ref).abs().max().item() <= 1e-5


def test_fp8_quant_roundtrip_bound():
    x = torch.randn(1000, generator=torch.Generator().manual_seed(1))
    xq, s = O.quantize_e4m3(x)
    assert s == pytest.approx(float(x.abs().max()) / 448.0)
    # e4m3 has 3 mantissa bits: relative error <= 2^-4 away from the subnormal range
    err = (O.dequantize_e4m3(xq, s) - x).abs()
    assert (err <= x.abs() * 2 ** -4 + s * 2 ** -9).all()


@pytest.mark.parametrize("causal,Hq,Hkv,Sq,Skv", [(False, 2, 2, 48, 80), (True, 4, 2, 64, 64), (True, 2, 1, 40, 100)])
def test_backward_restatement_matches_autograd(causal, Hq, Hkv, Sq, Skv):
    """The closed-form split (delta, dS, dV, dK, dQ) equals torch.autograd on the eager graph."""
    q, k, v = O.make_qkv(2, Hq, Hkv, Sq, Skv, 32, seed=11)
    d_o = torch.randn(2, Hq, Sq, 32, generator=torch.Generator().manual_seed(12))
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    out, _ = O.attention_eager(q, k, v, causal=causal)
    gq, gk, gv = torch.autograd.grad(out, (q, k, v), d_o)
    dq, dk, dv, delta = O.attention_backward(q.detach(), k.detach(), v.detach(), d_o, causal=causal)
    torch.testing.assert_close(dq, gq, atol=2e-5, rtol=1e-4)
    torch.testing.assert_close(dk, gk, atol=2e-5, rtol=1e-4)
    torch.testing.assert_close(dv, gv, atol=2e-5, rtol=1e-4)
    torch.testing.assert_close(delta, (out.detach() * d_o).sum(-1), atol=1e-5, rtol=1e-5)


def test_bwd_separation_heuristic(monkeypatch):
    """Decision rule and environment switches of the reference (bwd_separator.py:56-138)."""
    from heddle_b200.frontend import bwd_separator as bs
    for name in ("TILELANG_BWD_SEPARATION_MODE", "TILELANG_BWD_MIN_SEQ_FOR_SEP", "TILELANG_BWD_MIN_BATCH_HEADS"):
        monkeypatch.delenv(name, raising=False)
    assert bs.should_separate_bwd(4, 32, 4096, 128)
    assert not bs.should_separate_bwd(4, 32, 512, 128)      # short sequence
    assert not bs.should_separate_bwd(1, 2, 8192, 128)      # too little parallelism
    assert bs.should_separate_bwd(1, 8, 2048, 128) and not bs.should_separate_bwd(1, 4, 2048, 128)
    monkeypatch.setenv("TILELANG_BWD_SEPARATION_MODE", "unified")
    assert not bs.should_separate_bwd(4, 32, 4096, 128)
    monkeypatch.setenv("TILELANG_BWD_SEPARATION_MODE", "separated")
    assert bs.should_separate_bwd(1, 1, 128, 128)
    monkeypatch.setenv("TILELANG_BWD_SEPARATION_MODE", "auto")
    monkeypatch.setenv("TILELANG_BWD_MIN_SEQ_FOR_SEP", "256")
    assert bs.BWDSeparationConfig.from_env().min_seq_len_for_separation == 256
    with pytest.raises(NotImplementedError):
        bs.split_bwd_graph(None)


def test_separated_bwd_function_order_and_arguments():
    """create_separated_bwd_function calls preprocess -> dkdv -> dq with the reference's arguments."""
    from heddle_b200.frontend import bwd_separator as bs
    calls = []

    def pre(B, H, T, D):
        calls.append(("pre", B, H, T, D))
        return lambda o, d_o: "delta"

    def dkdv(B, H, Tq, Tkv, D, **kw):
        calls.append(("dkdv", B, H, Tq, Tkv, D, kw["is_causal"], kw["block_M"], kw["block_N"]))
        return lambda Q, K, V, O, dO, LSE, delta: ("dK", "dV") if delta == "delta" else None

    def dq(B, H, Tq, Tkv, D, **kw):
        calls.append(("dq", B, H, Tq, Tkv, D, kw["is_causal"], kw["block_M"], kw["block_N"]))
        return lambda Q, K, V, O, dO, LSE, delta: "dQ"

    f = bs.create_separated_bwd_function(pre, dkdv, dq)
    Q = torch.zeros(2, 3, 16, 8)
    K = torch.zeros(2, 3, 24, 8)
    assert f(Q, K, K, Q, Q, None, is_causal=True, config=bs.BWDSeparationConfig()) == ("dQ", "dK", "dV")
    assert calls == [("pre", 2, 3, 16, 8), ("dkdv", 2, 3, 16, 24, 8, True, 64, 128), ("dq", 2, 3, 16, 24, 8, True, 128, 64)]
