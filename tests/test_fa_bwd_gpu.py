"""Parity of the attention backward kernels (hb_fa_bwd_preprocess / _dkdv / _dq) with the CPU oracle.

Tolerance: gradients are sums over up to S products of 16-bit-rounded factors (P and dS are rounded to
the input type before the second matrix products, as in the forward kernel), so the error grows with
the magnitude of the gradient.  Bound used: max-abs error <= 2e-2 * max(1, max|reference|) for bf16
and 5e-3 * max(1, max|reference|) for fp16.  delta is an fp32 sum of 128 products of 16-bit values:
<= 1e-4 relative to the same sum formed in fp32 from the kernel's own (rounded) O, and <= 1e-1 (bf16) /
1e-2 (fp16) absolute against the oracle's delta, which uses the unrounded O.
"""
import pytest
import torch

from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(built_lib):
    from heddle_b200 import ops as _ops
    return _ops


def _tol(dtype, ref):
    return (2e-2 if dtype == torch.bfloat16 else 5e-3) * max(1.0, ref.abs().max().item())


def _grad_out(B, H, S, D, seed, dtype):
    return torch.randn(B, H, S, D, generator=torch.Generator().manual_seed(seed), dtype=torch.float32).to(dtype)


CASES = [
    # B, Hq, Hkv, Sq, Skv, causal, dtype
    (1, 2, 2, 128, 128, False, torch.bfloat16),
    (1, 2, 2, 256, 256, True, torch.bfloat16),
    (2, 3, 3, 384, 384, True, torch.float16),
    (1, 2, 2, 200, 333, False, torch.bfloat16),    # ragged tiles on both axes
    (1, 2, 2, 130, 300, True, torch.bfloat16),     # causal with a prefix of past keys
    (1, 4, 2, 257, 257, True, torch.bfloat16),     # grouped queries: dK, dV summed over the group
    (2, 8, 2, 192, 448, False, torch.float16),
    (1, 1, 1, 1, 77, True, torch.bfloat16),        # one query (decode-like)
    (1, 2, 1, 1024, 1024, True, torch.bfloat16),
]


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,causal,dtype", CASES)
def test_backward_matches_oracle(ops, B, Hq, Hkv, Sq, Skv, causal, dtype, D):
    q, k, v = O.make_qkv(B, Hq, Hkv, Sq, Skv, D, seed=Sq + Skv, dtype=dtype)
    d_o = _grad_out(B, Hq, Sq, D, 5 + Sq, dtype)
    qc, kc, vc, gc = q.cuda(), k.cuda(), v.cuda(), d_o.cuda()
    out, lse = ops.fa_fwd(qc, kc, vc, causal=causal, return_lse=True)
    delta = ops.fa_bwd_preprocess(out, gc)
    dk, dv = ops.fa_bwd_dkdv(qc, kc, vc, gc, lse, delta, causal=causal)
    dq = ops.fa_bwd_dq(qc, kc, vc, gc, lse, delta, causal=causal)
    torch.cuda.synchronize()
    assert ops.status_word() == 0
    rq, rk, rv, rdelta = O.attention_backward(q, k, v, d_o, causal=causal)
    assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape
    own = (out.float() * gc.float()).sum(-1)
    assert (delta - own).abs().max().item() <= 1e-4 * max(1.0, own.abs().max().item())
    assert (delta.cpu() - rdelta).abs().max().item() <= (1e-1 if dtype == torch.bfloat16 else 1e-2)
    for name, got, ref in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        err = (got.cpu().float() - ref).abs().max().item()
        assert err <= _tol(dtype, ref), f"{name}: max-abs error {err} (reference max {ref.abs().max().item()})"
    # one call for all three, same result
    dq2, dk2, dv2 = ops.fa_bwd(qc, kc, vc, out, gc, lse, causal=causal)
    assert torch.equal(dq2, dq) and torch.equal(dk2, dk) and torch.equal(dv2, dv)


def test_backward_is_linear_in_grad_out(ops):
    """dQ, dK, dV are linear in dO: g(2 dO) = 2 g(dO) exactly (a power of two commutes with every
    rounding on the path), and the gradient of a zero dO is zero."""
    B, H, S, D = 1, 2, 512, 128
    q, k, v = O.make_qkv(B, H, H, S, S, D, seed=21, dtype=torch.bfloat16)
    d_o = _grad_out(B, H, S, D, 22, torch.bfloat16)
    qc, kc, vc, gc = q.cuda(), k.cuda(), v.cuda(), d_o.cuda()
    out, lse = ops.fa_fwd(qc, kc, vc, causal=True, return_lse=True)
    a = ops.fa_bwd(qc, kc, vc, out, gc, lse, causal=True)
    b = ops.fa_bwd(qc, kc, vc, out, gc * 2, lse, causal=True)
    z = ops.fa_bwd(qc, kc, vc, out, torch.zeros_like(gc), lse, causal=True)
    for x, y, w in zip(a, b, z):
        assert torch.equal(x * 2, y)
        assert w.abs().max().item() == 0.0
    assert ops.status_word() == 0


def test_autograd_function_bshd(ops):
    """The BSHD autograd.Function of the front end: gradients against torch.autograd on the eager
    pattern the reference replaces (patterns.py:134-144), strided views in, no copies."""
    from heddle_b200.frontend.patterns import tilelang_flash_attn_wrapper, scaled_dot_product_attention_pattern
    B, S, H, D = 2, 320, 4, 128
    g = torch.Generator().manual_seed(7)
    q, k, v = (torch.randn(B, S, H, D, generator=g).to(torch.bfloat16) for _ in range(3))
    d_o = torch.randn(B, S, H, D, generator=g).to(torch.bfloat16)
    leaves = [t.cuda().requires_grad_(True) for t in (q, k, v)]
    out = tilelang_flash_attn_wrapper(*leaves, 1.0 / D ** 0.5)
    out.backward(d_o.cuda())
    torch.cuda.synchronize()
    assert ops.status_word() == 0
    ref_leaves = [t.float().requires_grad_(True) for t in (q, k, v)]
    ref_out = scaled_dot_product_attention_pattern(*ref_leaves, 1.0 / D ** 0.5)
    ref_out.backward(d_o.float())
    assert (out.detach().cpu().float() - ref_out.detach()).abs().max().item() <= 2e-2
    for got, ref in zip(leaves, ref_leaves):
        assert got.grad.shape == ref.grad.shape
        err = (got.grad.cpu().float() - ref.grad).abs().max().item()
        assert err <= _tol(torch.bfloat16, ref.grad), err
    # no gradient requested: the forward keeps nothing
    plain = tilelang_flash_attn_wrapper(q.cuda(), k.cuda(), v.cuda(), 1.0 / D ** 0.5)
    assert plain.grad_fn is None and torch.equal(plain, out.detach())


def test_factory_protocol(ops):
    """The reference's separated-backward function over the three factories, fed with the LSE of
    ``flashattn_lse`` (log2 domain, [B, H, S, 1])."""
    from heddle_b200.frontend.bwd_separator import create_separated_bwd_function
    from heddle_b200.tileop import flashattn_lse, flashattn_bwd_preprocess, flashattn_bwd_dkdv, flashattn_bwd_dq
    B, H, S, D = 1, 2, 384, 128
    q, k, v = O.make_qkv(B, H, H, S, S, D, seed=31, dtype=torch.float16)
    d_o = _grad_out(B, H, S, D, 32, torch.float16)
    qc, kc, vc, gc = q.cuda(), k.cuda(), v.cuda(), d_o.cuda()
    lse2, out = flashattn_lse(B, H, S, S, D, True)(qc, kc, vc)
    separated_bwd = create_separated_bwd_function(flashattn_bwd_preprocess, flashattn_bwd_dkdv, flashattn_bwd_dq)
    dq, dk, dv = separated_bwd(qc, kc, vc, out, gc, lse2, is_causal=True)
    torch.cuda.synchronize()
    assert ops.status_word() == 0
    rq, rk, rv, _ = O.attention_backward(q, k, v, d_o, causal=True)
    for got, ref in ((dq, rq), (dk, rk), (dv, rv)):
        assert (got.cpu().float() - ref).abs().max().item() <= _tol(torch.float16, ref)


def test_backward_empty_and_rejected_inputs(ops):
    from heddle_b200._lib import HeddleError
    q = torch.zeros(1, 2, 0, 128, dtype=torch.bfloat16, device="cuda")
    k = torch.randn(1, 2, 64, 128, device="cuda").to(torch.bfloat16)
    lse = torch.zeros(1, 2, 0, dtype=torch.float32, device="cuda")
    dq, dk, dv = ops.fa_bwd(q, k, k, q, q, lse)
    assert dq.shape == q.shape and dk.abs().max().item() == 0.0 and dv.abs().max().item() == 0.0
    q96 = torch.zeros(1, 2, 64, 96, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(HeddleError, match="head_dim"):
        ops.fa_bwd(q96, q96, q96, q96, q96, torch.zeros(1, 2, 64, device="cuda"))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.fa_bwd_preprocess(torch.zeros(1, 1, 8, 128, dtype=torch.bfloat16), torch.zeros(1, 1, 8, 128, dtype=torch.bfloat16))


def test_training_step_through_the_compiled_backend(ops):
    """torch.compile(backend=tilelang_backend) on a module that calls SDPA: the attention leaf is
    differentiable, gradients of the projections match eager PyTorch in fp32."""
    import heddle_b200 as heddle

    class Attn(torch.nn.Module):
        def __init__(self, hidden=256, heads=2):
            super().__init__()
            self.heads = heads
            self.qkv = torch.nn.Linear(hidden, 3 * hidden, bias=False)
            self.proj = torch.nn.Linear(hidden, hidden, bias=False)

        def forward(self, x):
            B, S, Hd = x.shape
            q, k, v = self.qkv(x).view(B, S, 3, self.heads, Hd // self.heads).permute(2, 0, 3, 1, 4)
            o = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
            return self.proj(o.transpose(1, 2).reshape(B, S, Hd))

    torch.manual_seed(0)
    ref = Attn().float()
    x = torch.randn(2, 256, 256)
    ref(x).square().mean().backward()
    model = Attn()
    model.load_state_dict(ref.state_dict())
    model = model.cuda().to(torch.bfloat16)
    heddle.init()
    torch._dynamo.reset()
    compiled = torch.compile(model, backend=heddle.frontend.tilelang_backend)
    loss = compiled(x.cuda().to(torch.bfloat16)).float().square().mean()
    loss.backward()
    torch.cuda.synchronize()
    assert ops.status_word() == 0
    for (name, p_ref), p_got in zip(ref.named_parameters(), model.parameters()):
        assert p_got.grad is not None, name
        err = (p_got.grad.float().cpu() - p_ref.grad).abs().max().item()
        assert err <= 3e-2 * max(p_ref.grad.abs().max().item(), 1e-3), (name, err, p_ref.grad.abs().max().item())


def test_backward_full_length_properties(ops):
    """Headline sequence length (S = 4096, D = 128, causal): a size-independent identity over all heads and
    oracle parity on one head.  With dO = 1 every column of dV[b,h,k,:] is sum_q P[q,k], which is exactly the
    H2O score that hb_h2o_score computes from the same LSE with another kernel."""
    B, H, S, D = 2, 4, 4096, 128
    q, k, v = O.make_qkv(B, H, H, S, S, D, seed=41, dtype=torch.bfloat16)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    out, lse = ops.fa_fwd(qc, kc, vc, causal=True, return_lse=True)
    ones = torch.ones_like(qc)
    _, _, dv1 = ops.fa_bwd(qc, kc, vc, out, ones, lse, causal=True)
    score = ops.h2o_score(qc, kc, lse, causal=True)
    torch.cuda.synchronize()
    assert ops.status_word() == 0
    ref = score.unsqueeze(-1).expand(-1, -1, -1, D)
    # P is rounded to bf16 before the product (relative 2^-9 per term), the sum runs over up to 4096 terms
    assert (dv1.float() - ref).abs().max().item() <= 1e-2 * max(1.0, score.max().item())
    # columns of dV are identical for dO = 1
    assert (dv1.float() - dv1.float()[..., :1]).abs().max().item() <= 2e-2 * max(1.0, score.max().item())
    # one head against the oracle
    d_o = _grad_out(B, H, S, D, 42, torch.bfloat16)
    dq, dk, dv = ops.fa_bwd(qc, kc, vc, out, d_o.cuda(), lse, causal=True)
    torch.cuda.synchronize()
    assert ops.status_word() == 0
    b, h = 1, 2
    rq, rk, rv, _ = O.attention_backward(q[b:b + 1, h:h + 1], k[b:b + 1, h:h + 1], v[b:b + 1, h:h + 1],
                                         d_o[b:b + 1, h:h + 1], causal=True)
    for name, got, ref1 in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        err = (got[b:b + 1, h:h + 1].cpu().float() - ref1).abs().max().item()
        assert err <= _tol(torch.bfloat16, ref1), f"{name}: {err} (reference max {ref1.abs().max().item()})"


def test_bshd_strided_gqa_backward(ops):
    """(B, S, H, D) views with grouped queries straight through ops.fa_bwd: strides are passed on, nothing is
    copied, dK / dV come back as (B, S, Hkv, D) views."""
    B, S, Hq, Hkv, D = 2, 300, 6, 2, 128
    g = torch.Generator().manual_seed(51)
    qkv = torch.randn(B, S, Hq + 2 * Hkv, D, generator=g).to(torch.bfloat16).cuda()   # one packed projection output
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]              # non-contiguous views
    d_o = torch.randn(B, S, Hq, D, generator=g).to(torch.bfloat16).cuda()
    out, lse = ops.fa_fwd(q, k, v, causal=True, layout="bshd", return_lse=True)
    dq, dk, dv = ops.fa_bwd(q, k, v, out, d_o, lse, causal=True, layout="bshd")
    torch.cuda.synchronize()
    assert ops.status_word() == 0
    assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape
    t = lambda x: x.transpose(1, 2).float().cpu()
    rq, rk, rv, _ = O.attention_backward(t(q), t(k), t(v), t(d_o), causal=True)
    for name, got, ref in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        err = (t(got) - ref).abs().max().item()
        assert err <= _tol(torch.bfloat16, ref), f"{name}: {err} (reference max {ref.abs().max().item()})"
