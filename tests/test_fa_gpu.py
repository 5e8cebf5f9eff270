"""Parity of the sm_100a FlashAttention-forward kernel (through the C ABI) with the CPU
oracle, the reference-generated golden fixtures, and size-independent properties at the
benchmark's full sizes.

Tolerances (benchmark spec): max-abs error <= 2e-2 for 16-bit inputs against fp32,
row-wise logsumexp within 1e-3.
"""
import math

import pytest
import torch

from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu

TOL_O = 2e-2
TOL_LSE = 1e-3


@pytest.fixture(scope="module")
def ops(built_lib):
    from heddle_b200 import ops as _ops
    return _ops


def _run(ops, q, k, v, causal, **kw):
    out, lse = ops.fa_fwd(q.cuda(), k.cuda(), v.cuda(), causal=causal, return_lse=True, **kw)
    torch.cuda.synchronize()
    assert ops.status_word() == 0
    return out.cpu(), lse.cpu()


CASES = [
    # B, Hq, Hkv, Sq, Skv, D, causal, dtype
    (1, 1, 1, 128, 128, 128, False, torch.bfloat16),
    (1, 1, 1, 256, 256, 128, True, torch.bfloat16),
    (1, 4, 4, 256, 256, 64, False, torch.bfloat16),   # config 1 geometry (D=64)
    (2, 4, 2, 333, 333, 128, True, torch.bfloat16),   # ragged + GQA 2:1
    (1, 8, 1, 640, 640, 128, True, torch.bfloat16),   # GQA 8:1
    (2, 3, 3, 200, 455, 128, True, torch.float16),    # Sq != Skv, past_len rule
    (1, 2, 2, 100, 777, 64, False, torch.float16),    # ragged non-causal, D=64
    (1, 2, 2, 1, 300, 128, True, torch.bfloat16),     # single query row
    (1, 2, 2, 129, 129, 64, True, torch.float16),     # one row past a tile boundary
    (1, 1, 1, 1024, 1024, 128, True, torch.float16),  # the reference's dtype
    (3, 2, 2, 384, 384, 128, False, torch.bfloat16),  # odd number of 256-row blocks
]


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,D,causal,dtype", CASES)
def test_parity_with_cpu_oracle(ops, B, Hq, Hkv, Sq, Skv, D, causal, dtype):
    q, k, v = O.make_qkv(B, Hq, Hkv, Sq, Skv, D, seed=Sq + Skv + D, dtype=dtype)
    out, lse = _run(ops, q, k, v, causal)
    ref, ref_lse = O.attention_eager(q, k, v, causal=causal)
    assert out.dtype == dtype and not torch.isnan(out.float()).any()
    assert (out.float() - ref).abs().max().item() <= TOL_O
    assert (lse - ref_lse).abs().max().item() <= TOL_LSE


def test_parity_with_tiled_oracle_fp16(ops):
    """Against the restatement of the generated kernel's own tile algorithm (fp16, as the reference)."""
    q, k, v = O.make_qkv(1, 2, 2, 512, 512, 128, seed=21, dtype=torch.float16)
    out, lse = _run(ops, q, k, v, True)
    ref, lse2 = O.flashattn_tiled(q, k, v, True)
    assert (out.float() - ref.float()).abs().max().item() <= 4e-3
    assert (lse - lse2 * O.LN2).abs().max().item() <= 1e-4


@pytest.mark.parametrize("name", ["c1", "causal_ragged", "causal_512"])
def test_golden_fixtures(ops, golden, name):
    case = golden[name]
    B, Hq, Hkv, Sq, Skv, D = case["shape"]
    q, k, v = O.make_qkv(B, Hq, Hkv, Sq, Skv, D, seed=case["seed"], dtype=getattr(torch, case["in_dtype"]))
    # config 1 is an fp32 graph: the kernel runs on the bf16-rounded inputs, the error budget stays 2e-2
    out, _ = _run(ops, q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16), case["causal"])
    assert (out.float() - case["out"].float()).abs().max().item() <= TOL_O


def test_bshd_layout_and_strides(ops):
    """BSHD storage and non-contiguous views are addressed through strides, no copies."""
    q, k, v = O.make_qkv(2, 4, 4, 300, 300, 128, seed=4, dtype=torch.bfloat16)
    ref, _ = O.attention_eager(q, k, v, causal=True)
    qs, ks, vs = (t.transpose(1, 2).contiguous().cuda() for t in (q, k, v))  # [B,S,H,D]
    out = ops.fa_fwd(qs, ks, vs, causal=True, layout="bshd")
    assert out.shape == qs.shape
    assert (out.cpu().float().transpose(1, 2) - ref).abs().max().item() <= TOL_O
    # a BHSD *view* of the BSHD buffer
    out2 = ops.fa_fwd(qs.transpose(1, 2), ks.transpose(1, 2), vs.transpose(1, 2), causal=True)
    assert (out2.cpu().float() - ref).abs().max().item() <= TOL_O
    # packed QKV buffer [B,S,3,H,D]
    qkv = torch.stack([qs, ks, vs], dim=2)
    out3 = ops.fa_fwd(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], causal=True, layout="bshd")
    assert torch.equal(out3, out)


def test_softmax_scale_is_honoured(ops):
    q, k, v = O.make_qkv(1, 2, 2, 256, 256, 64, seed=8, dtype=torch.bfloat16)
    out, lse = ops.fa_fwd(q.cuda(), k.cuda(), v.cuda(), causal=False, softmax_scale=0.3, return_lse=True)
    ref, ref_lse = O.attention_eager(q, k, v, causal=False, scale=0.3)
    assert (out.cpu().float() - ref).abs().max().item() <= TOL_O
    assert (lse.cpu() - ref_lse).abs().max().item() <= 2e-3  # larger scores at scale 0.3


def test_large_magnitude_rows_trigger_rescale(ops):
    """Row maxima that grow along the keys force the O-rescale path of the correction warpgroup."""
    q, k, v = O.make_qkv(1, 2, 2, 256, 1024, 128, seed=13, dtype=torch.bfloat16)
    ramp = torch.linspace(0.2, 3.0, 1024)[None, None, :, None]
    k = (k.float() * ramp).to(torch.bfloat16)
    out, lse = _run(ops, q, k, v, False)
    ref, ref_lse = O.attention_eager(q, k, v, causal=False)
    assert (out.float() - ref).abs().max().item() <= TOL_O
    assert ((lse - ref_lse).abs() / ref_lse.abs().clamp_min(1.0)).max().item() <= TOL_LSE


def test_error_codes_surface_as_exceptions(ops):
    q = torch.zeros(1, 1, 128, 96, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="head_dim"):
        ops.fa_fwd(q, q, q)
    q = torch.zeros(1, 1, 128, 128, dtype=torch.bfloat16, device="cuda")
    kk = torch.zeros(1, 1, 64, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="Skv >= Sq"):
        ops.fa_fwd(q, kk, kk, causal=True)


# ----------------------------------------------------------------------------------------
# full benchmark sizes: size-independent properties + sampled oracle rows
# ----------------------------------------------------------------------------------------
def _sampled_check(out, lse, q, k, v, causal, pairs):
    g = q.shape[1] // k.shape[1]
    for b, h in pairs:
        ref, ref_lse = O.attention_eager(q[b:b + 1, h:h + 1].cpu(), k[b:b + 1, h // g:h // g + 1].cpu(),
                                         v[b:b + 1, h // g:h // g + 1].cpu(), causal=causal)
        assert (out[b, h].cpu().float() - ref[0, 0]).abs().max().item() <= TOL_O
        assert (lse[b, h].cpu() - ref_lse[0, 0]).abs().max().item() <= TOL_LSE


def test_full_size_bf16_causal_mha(ops):
    """B=4, H=32, S=4096, D=128 causal: properties of the whole output plus oracle rows for sampled heads."""
    B, H, S, D = 4, 32, 4096, 128
    gen = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randn(B, H, S, D, generator=gen, device="cuda").to(torch.bfloat16)
    k = torch.randn(B, H, S, D, generator=gen, device="cuda").to(torch.bfloat16)
    v = torch.randn(B, H, S, D, generator=gen, device="cuda").to(torch.bfloat16)
    out, lse = ops.fa_fwd(q, k, v, causal=True, return_lse=True)
    torch.cuda.synchronize()
    assert ops.status_word() == 0
    assert not torch.isnan(out.float()).any() and not torch.isinf(lse).any()
    # causal: the first query row attends to key 0 only
    assert torch.equal(out[:, :, 0], v[:, :, 0])
    assert (lse[:, :, 0] - (q[:, :, 0].float() * k[:, :, 0].float()).sum(-1) / math.sqrt(D)).abs().max() <= TOL_LSE
    # rows of P sum to one: V = 1 gives O = 1
    ones = torch.ones_like(v)
    assert (ops.fa_fwd(q, k, ones, causal=True).float() - 1.0).abs().max().item() <= 1e-2
    # linearity in V
    v2 = torch.randn(B, H, S, D, generator=gen, device="cuda").to(torch.bfloat16)
    o2 = ops.fa_fwd(q, k, v2, causal=True)
    o12 = ops.fa_fwd(q, k, ((v.float() + v2.float()) * 0.5).to(torch.bfloat16), causal=True)
    assert (o12.float() - 0.5 * (out.float() + o2.float())).abs().max().item() <= 3e-2
    # deterministic
    again = ops.fa_fwd(q, k, v, causal=True)
    assert torch.equal(again, out)
    # a batch/head permutation of the inputs permutes the output
    perm = torch.randperm(H, device="cuda")
    assert torch.equal(ops.fa_fwd(q[:, perm], k[:, perm], v[:, perm], causal=True), out[:, perm])
    _sampled_check(out, lse, q, k, v, True, [(0, 0), (1, 13), (3, 31)])


def test_full_size_gqa_slice(ops):
    """One GPU's share of the GQA configuration (one KV head with its 8 query heads, S=8192), B=2 of 8."""
    B, Hq, Hkv, S, D = 2, 8, 1, 8192, 128
    gen = torch.Generator(device="cuda").manual_seed(1)
    q = torch.randn(B, Hq, S, D, generator=gen, device="cuda").to(torch.bfloat16)
    k = torch.randn(B, Hkv, S, D, generator=gen, device="cuda").to(torch.bfloat16)
    v = torch.randn(B, Hkv, S, D, generator=gen, device="cuda").to(torch.bfloat16)
    out, lse = ops.fa_fwd(q, k, v, causal=True, return_lse=True)
    torch.cuda.synchronize()
    assert ops.status_word() == 0
    # GQA == MHA on repeated KV heads
    out_mha = ops.fa_fwd(q, k.expand(B, Hq, S, D), v.expand(B, Hq, S, D), causal=True)
    assert torch.equal(out_mha, out)
    assert (ops.fa_fwd(q, k, torch.ones_like(v), causal=True).float() - 1.0).abs().max().item() <= 1e-2
    _sampled_check(out, lse, q, k, v, True, [(0, 0), (1, 7)])


def test_long_sequence_rows(ops):
    """S = 32768 (256 key tiles per row block, the longest block a CTA walks): the first, a middle and
    the last query rows against the oracle, which sees those rows as a short query block with the
    matching causal offset; decode-shaped calls (Sq = 1 and Sq = 5 against the full keys) as well."""
    B, H, S, D = 1, 2, 32768, 128
    q, k, v = O.make_qkv(B, H, H, S, S, D, seed=77, dtype=torch.bfloat16)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    out, lse = ops.fa_fwd(qd, kd, vd, causal=True, return_lse=True)
    torch.cuda.synchronize()
    assert ops.status_word() == 0
    for lo, hi in ((0, 16), (16383, 16399), (S - 16, S)):
        # rows [lo, hi) of the causal problem = a (hi - lo)-row query block over keys [0, hi)
        ref, ref_lse = O.attention_eager(q[:, :, lo:hi], k[:, :, :hi], v[:, :, :hi], causal=True)
        assert (out[:, :, lo:hi].float().cpu() - ref).abs().max().item() <= 2e-2
        assert (lse[:, :, lo:hi].cpu() - ref_lse).abs().max().item() <= 1e-3
    for sq in (1, 5):
        o2, l2 = ops.fa_fwd(qd[:, :, S - sq:].contiguous(), kd, vd, causal=True, return_lse=True)
        ref, ref_lse = O.attention_eager(q[:, :, S - sq:], k, v, causal=True)
        assert (o2.float().cpu() - ref).abs().max().item() <= 2e-2
        assert (l2.cpu() - ref_lse).abs().max().item() <= 1e-3
        # the same rows as part of the full problem
        assert (o2.float() - out[:, :, S - sq:].float()).abs().max().item() <= 1e-2
