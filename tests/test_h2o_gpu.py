"""Parity of hb_h2o_score and the H2O attention leaf with the CPU oracle."""
import pytest
import torch

from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(built_lib):
    from heddle_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,D,causal,dtype", [
    (1, 2, 2, 128, 128, 128, True, torch.bfloat16),
    (2, 4, 2, 333, 333, 128, True, torch.bfloat16),
    (1, 2, 2, 200, 455, 64, True, torch.float16),
    (1, 3, 3, 300, 300, 128, False, torch.bfloat16),
    (1, 2, 1, 1024, 1024, 128, True, torch.float16),
    (1, 1, 1, 77, 900, 64, False, torch.bfloat16),
])
def test_h2o_score_matches_oracle(ops, B, Hq, Hkv, Sq, Skv, D, causal, dtype):
    q, k, v = O.make_qkv(B, Hq, Hkv, Sq, Skv, D, seed=Sq + D, dtype=dtype)
    out, lse = ops.fa_fwd(q.cuda(), k.cuda(), v.cuda(), causal=causal, return_lse=True)
    score = ops.h2o_score(q.cuda(), k.cuda(), lse, causal=causal)
    torch.cuda.synchronize()
    assert ops.status_word() == 0
    _, ref_lse = O.attention_eager(q, k, v, causal=causal)
    ref = O.h2o_score(q, k, ref_lse, causal=causal)
    assert score.shape == (B, Hq, Skv)
    # every query row distributes a total probability of 1
    assert (score.sum(-1).cpu() - Sq).abs().max().item() <= 2e-3 * Sq
    assert (score.cpu() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())


def test_h2o_matches_reference_fixture(ops, golden):
    """Against the outputs the reference's own backend produced for the H2O structure (fusion off)."""
    case = golden["h2o"]
    B, Hq, Hkv, Sq, Skv, D = case["shape"]
    q, k, v = (t.cuda() for t in O.make_qkv(B, Hq, Hkv, Sq, Skv, D, seed=case["seed"], dtype=torch.bfloat16))
    out, lse = ops.fa_fwd(q, k, v, causal=True, return_lse=True)
    score = ops.h2o_score(q, k, lse, causal=True)
    assert (out.float().cpu() - case["out"]).abs().max().item() <= 2e-2
    assert (score.cpu() - case["score"]).abs().max().item() <= 2e-2 * max(1.0, case["score"].abs().max().item())


def test_h2o_leaf_and_factories(ops):
    from heddle_b200.frontend.backend import _tilelang_h2o_attention
    from heddle_b200.tileop import flashattn_lse, h2o_score

    q, k, v = O.make_qkv(1, 2, 2, 384, 384, 128, seed=3, dtype=torch.float16)
    out, score = _tilelang_h2o_attention(q.cuda(), k.cuda(), v.cuda())
    ref_out, ref_lse = O.attention_eager(q, k, v, causal=True)
    assert (out.cpu().float() - ref_out).abs().max().item() <= 2e-2
    ref = O.h2o_score(q, k, ref_lse, causal=True)
    assert (score.cpu() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
    # the reference's factory protocol: (LSE log2-domain [B,H,S,1], O), then h2o_score(Q, K, LSE)
    lse2, o2 = flashattn_lse(1, 2, 384, 384, 128, True)(q.cuda(), k.cuda(), v.cuda())
    assert lse2.shape == (1, 2, 384, 1)
    assert (lse2[..., 0].cpu() - ref_lse * O.LOG2E).abs().max().item() <= 2e-3
    s2 = h2o_score(1, 2, 384, 384, 128, True)(q.cuda(), k.cuda(), lse2)
    assert torch.allclose(s2, score, rtol=1e-4, atol=1e-4)


def test_h2o_full_length_properties(ops):
    """Headline sequence length (S = 4096, D = 128, causal): size-independent properties over all
    heads and oracle parity on one head."""
    B, H, S, D = 2, 4, 4096, 128
    q, k, v = O.make_qkv(B, H, H, S, S, D, seed=11, dtype=torch.bfloat16)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    _, lse = ops.fa_fwd(qd, kd, vd, causal=True, return_lse=True)
    score = ops.h2o_score(qd, kd, lse, causal=True)
    again = ops.h2o_score(qd, kd, lse, causal=True)
    torch.cuda.synchronize()
    assert ops.status_word() == 0
    sc = score.cpu()
    assert (sc >= 0).all()
    # every query row hands out a total probability of 1
    assert (sc.sum(-1) - S).abs().max().item() <= 2e-3 * S
    # the last key is only seen by the last query, the first key by every query
    assert (sc[..., -1] <= 1.0 + 1e-3).all() and (sc[..., 0] >= sc[..., -1]).all()
    # two commutative atomic adds per key: the result does not depend on their order
    assert torch.equal(score, again)
    _, ref_lse = O.attention_eager(q[:1, :1], k[:1, :1], v[:1, :1], causal=True)
    ref = O.h2o_score(q[:1, :1], k[:1, :1], ref_lse, causal=True)
    assert (sc[:1, :1] - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
