"""FP8 e4m3 attention forward (per-tensor scales, P requantised to e4m3 before the PV MMA) against
fp32 attention on the DEQUANTISED inputs.  Tolerance (benchmark spec): max-abs error <= 6e-2 on
O, row-wise logsumexp within 1e-3."""
import pytest
import torch

from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(built_lib):
    from heddle_b200 import ops as _ops
    return _ops


def _quantised(B, Hq, Hkv, Sq, Skv, D, seed):
    q, k, v = O.make_qkv(B, Hq, Hkv, Sq, Skv, D, seed=seed)
    (qq, sq), (kq, sk), (vq, sv) = O.quantize_e4m3(q), O.quantize_e4m3(k), O.quantize_e4m3(v)
    deq = (O.dequantize_e4m3(qq, sq), O.dequantize_e4m3(kq, sk), O.dequantize_e4m3(vq, sv))
    return (qq, kq, vq), (sq, sk, sv), deq


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,causal", [
    (1, 1, 1, 128, 128, False),
    (1, 2, 2, 512, 512, False),
    (2, 4, 2, 333, 333, True),
    (1, 2, 2, 200, 700, True),
    (1, 2, 2, 1024, 1024, True),
    (1, 1, 1, 2048, 2048, False),
])
def test_fp8_parity(ops, B, Hq, Hkv, Sq, Skv, causal):
    (qq, kq, vq), scales, (qd, kd, vd) = _quantised(B, Hq, Hkv, Sq, Skv, 128, seed=Sq + Skv)
    out, lse = ops.fa_fwd(qq.cuda(), kq.cuda(), vq.cuda(), causal=causal, return_lse=True, scales=scales)
    torch.cuda.synchronize()
    assert ops.status_word() == 0
    assert out.dtype == torch.bfloat16 and not torch.isnan(out.float()).any()
    ref, ref_lse = O.attention_eager(qd, kd, vd, causal=causal)
    assert (out.float().cpu() - ref).abs().max().item() <= 6e-2
    assert (lse.cpu() - ref_lse).abs().max().item() <= 1e-3


def test_fp8_full_sequence_length_slice(ops):
    """The FP8 configuration's geometry (S=8192, D=128, non-causal) on a slice of its batch x heads."""
    B, H, S, D = 1, 4, 8192, 128
    gen = torch.Generator(device="cuda").manual_seed(0)
    q, k, v = (torch.randn(B, H, S, D, generator=gen, device="cuda") for _ in range(3))
    qs, ks, vs = (float(t.abs().max()) / 448.0 for t in (q, k, v))
    qq, kq, vq = ((t / s).to(torch.float8_e4m3fn) for t, s in ((q, qs), (k, ks), (v, vs)))
    out, lse = ops.fa_fwd(qq, kq, vq, causal=False, return_lse=True, scales=(qs, ks, vs))
    torch.cuda.synchronize()
    assert ops.status_word() == 0
    ref, ref_lse = O.attention_eager((qq.float() * qs)[:, :2].cpu(), (kq.float() * ks)[:, :2].cpu(),
                                     (vq.float() * vs)[:, :2].cpu(), causal=False)
    assert (out[:, :2].float().cpu() - ref).abs().max().item() <= 6e-2
    assert (lse[:, :2].cpu() - ref_lse).abs().max().item() <= 1e-3
    # rows of P sum to one: V = 1 (exactly representable) gives O = 1 up to the e4m3 rounding of P
    ones = torch.ones_like(vq.float()).to(torch.float8_e4m3fn)
    o1 = ops.fa_fwd(qq, kq, ones, causal=False, scales=(qs, ks, 1.0))
    assert (o1.float() - 1.0).abs().max().item() <= 3e-2


def test_fp8_rejects_other_head_dims(ops):
    x = torch.zeros(1, 1, 128, 64, device="cuda").to(torch.float8_e4m3fn)
    with pytest.raises(RuntimeError, match="head_dim 128"):
        ops.fa_fwd(x, x, x)
