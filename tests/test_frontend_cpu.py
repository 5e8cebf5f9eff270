"""Graph-level tests of the torch.compile backend: run on a CPU-only host, nothing is executed
on the kernels (the rewritten graph is inspected, the original one is what runs)."""
import copy
import math

import pytest
import torch
import torch.nn.functional as F

import heddle_b200
from heddle_b200.frontend import backend as B
from heddle_b200.frontend import fusion, patterns


def capture(module, *inputs):
    """Compile `module` with a recording backend; returns the GraphModule the backend produced."""
    got = []

    def recording_backend(gm, example_inputs):
        original = copy.deepcopy(gm)
        got.append(B.tilelang_backend(gm, example_inputs))
        return original.forward

    torch._dynamo.reset()
    with torch.no_grad():
        torch.compile(module, backend=recording_backend)(*inputs)
    assert len(got) == 1, "expected a single graph"
    return got[0]


def targets(gm):
    return [n.target for n in gm.graph.nodes if n.op == "call_function"]


def qkv(B_=1, H=2, S=64, D=64, Skv=None, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(0)
    Skv = Skv or S
    return (torch.randn(B_, H, S, D, generator=g).to(dtype), torch.randn(B_, H, Skv, D, generator=g).to(dtype),
            torch.randn(B_, H, Skv, D, generator=g).to(dtype))


def test_init_is_idempotent_and_names_match_reference():
    heddle_b200.init()
    heddle_b200.init()
    from heddle_b200.frontend import tilelang_backend
    assert callable(tilelang_backend)
    for name in ("_tilelang_sdpa_direct", "_tilelang_h2o_attention", "_replace_sdpa_op",
                 "_replace_expanded_attention", "try_fuse_h2o_attention", "tilelang_backend"):
        assert hasattr(B, name)
    for name in ("scaled_dot_product_attention_pattern", "TileLangFlashAttnFunc", "tilelang_flash_attn_wrapper",
                 "tilelang_flash_attn_replacement", "TileLangH2OFunc", "tilelang_h2o_attention_wrapper",
                 "_heuristic_config"):
        assert hasattr(patterns, name)
    assert patterns._heuristic_config(4, 32, 4096, 4096, 128) == {"block_M": 128, "block_N": 128, "num_stages": 5,
                                                                  "threads": 512}


@pytest.mark.parametrize("causal", [False, True])
def test_sdpa_op_is_replaced_with_its_semantics(causal):
    class M(torch.nn.Module):
        def forward(self, q, k, v):
            return F.scaled_dot_product_attention(q, k, v, is_causal=causal, scale=0.2)

    gm = capture(M(), *qkv())
    nodes = [n for n in gm.graph.nodes if n.op == "call_function"]
    assert [n.target for n in nodes] == [B._tilelang_sdpa_direct]
    assert nodes[0].kwargs == {"is_causal": causal, "scale": 0.2}


def test_sdpa_with_mask_or_dropout_is_left_alone():
    class M(torch.nn.Module):
        def forward(self, q, k, v, m):
            return F.scaled_dot_product_attention(q, k, v, attn_mask=m)

    q, k, v = qkv()
    gm = capture(M(), q, k, v, torch.zeros(64, 64, dtype=q.dtype))
    assert B._tilelang_sdpa_direct not in targets(gm)


def test_expanded_attention_non_causal_config1_module():
    """The benchmark's first configuration: softmax(Q K^T / sqrt(D)) V, non-causal."""
    class Attn(torch.nn.Module):
        def forward(self, q, k, v):
            s = torch.matmul(q, k.transpose(-2, -1)) / math.sqrt(q.shape[-1])
            return torch.matmul(torch.softmax(s, dim=-1), v)

    gm = capture(Attn(), *qkv(1, 4, 256, 64))
    nodes = [n for n in gm.graph.nodes if n.op == "call_function"]
    assert [n.target for n in nodes] == [B._tilelang_sdpa_direct]
    assert nodes[0].kwargs["is_causal"] is False
    assert nodes[0].kwargs["scale"] == pytest.approx(1 / 8)


def test_expanded_attention_with_causal_mask_and_past():
    class Attn(torch.nn.Module):
        def forward(self, q, k, v):
            s = torch.matmul(q, k.transpose(-2, -1)) * 0.125
            Sq, Skv = q.shape[-2], k.shape[-2]
            s = s + torch.triu(torch.full((Sq, Skv), float("-inf"), dtype=q.dtype), diagonal=Skv - Sq + 1)
            return torch.matmul(torch.softmax(s, dim=-1), v)

    gm = capture(Attn(), *qkv(1, 2, 48, 64, Skv=80))
    nodes = [n for n in gm.graph.nodes if n.op == "call_function" and n.target is B._tilelang_sdpa_direct]
    assert len(nodes) == 1 and nodes[0].kwargs == {"is_causal": True, "scale": 0.125}
    assert not any("softmax" in str(t) for t in targets(gm))


def test_expanded_attention_with_other_mask_is_left_alone():
    class Attn(torch.nn.Module):
        def forward(self, q, k, v, bias):
            s = torch.matmul(q, k.transpose(-2, -1)) * 0.125 + bias
            return torch.matmul(torch.softmax(s, dim=-1), v)

    q, k, v = qkv()
    gm = capture(Attn(), q, k, v, torch.randn(64, 64).to(q.dtype))
    assert B._tilelang_sdpa_direct not in targets(gm)
    # a mask that is triangular but not the causal one for these lengths
    class Attn2(torch.nn.Module):
        def forward(self, q, k, v):
            s = torch.matmul(q, k.transpose(-2, -1)) * 0.125
            s = s + torch.triu(torch.full((64, 64), float("-inf"), dtype=q.dtype), diagonal=3)
            return torch.matmul(torch.softmax(s, dim=-1), v)

    assert B._tilelang_sdpa_direct not in targets(capture(Attn2(), q, k, v))


def test_bshd_pattern_uses_the_bshd_wrapper():
    class M(torch.nn.Module):
        def forward(self, q, k, v):
            return patterns.scaled_dot_product_attention_pattern(q, k, v, 0.125)

    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(2, 32, 4, 64, generator=g).to(torch.bfloat16) for _ in range(3))
    gm = capture(M(), q, k, v)
    assert patterns.tilelang_flash_attn_wrapper in targets(gm)
    assert not any("softmax" in str(t) for t in targets(gm))


def test_h2o_structure_is_fused_with_both_outputs():
    class H2O(torch.nn.Module):
        def forward(self, q, k, v):
            s = torch.matmul(q, k.transpose(-2, -1)) / 8.0
            s = s + torch.triu(torch.full((64, 64), float("-inf"), dtype=q.dtype), diagonal=1)
            p = torch.softmax(s, dim=-1)
            return torch.matmul(p, v), p.sum(dim=-2)

    gm = capture(H2O(), *qkv())
    t = targets(gm)
    assert B._tilelang_h2o_attention in t and B._tilelang_sdpa_direct not in t
    node = next(n for n in gm.graph.nodes if n.target is B._tilelang_h2o_attention)
    assert node.kwargs == {"is_causal": True, "scale": pytest.approx(0.125)}


def test_operands_the_kernels_cannot_take_stay_eager():
    """The rewrites are decided from the captured shapes and dtypes: what the sm_100a kernels cannot
    compute exactly as eager does stays an eager node instead of failing (or differing) at run time."""
    class Sdpa(torch.nn.Module):
        def __init__(self, causal):
            super().__init__()
            self.causal = causal

        def forward(self, q, k, v):
            return F.scaled_dot_product_attention(q, k, v, is_causal=self.causal)

    # is_causal=True with Sq != Skv: eager masks from the top-left corner, the kernel from the end of the keys
    assert B._tilelang_sdpa_direct not in targets(capture(Sdpa(True), *qkv(1, 2, 48, 64, Skv=80)))
    assert B._tilelang_sdpa_direct in targets(capture(Sdpa(False), *qkv(1, 2, 48, 64, Skv=80)))
    assert B._tilelang_sdpa_direct in targets(capture(Sdpa(True), *qkv(1, 2, 64, 64)))
    # head_dim 96, fp32 operands, 3-D operands
    assert B._tilelang_sdpa_direct not in targets(capture(Sdpa(False), *qkv(1, 2, 64, 96)))
    assert B._tilelang_sdpa_direct not in targets(capture(Sdpa(False), *qkv(1, 2, 64, 64, dtype=torch.float32)))
    q, k, v = qkv(1, 2, 64, 64)
    assert B._tilelang_sdpa_direct not in targets(capture(Sdpa(False), q[0], k[0], v[0]))

    class Expanded(torch.nn.Module):
        def forward(self, q, k, v):
            s = torch.matmul(q, k.transpose(-2, -1)) / math.sqrt(q.shape[-1])
            return torch.matmul(torch.softmax(s, dim=-1), v)

    assert B._tilelang_sdpa_direct not in targets(capture(Expanded(), *qkv(1, 2, 64, 64, dtype=torch.float32)))
    assert B._tilelang_sdpa_direct not in targets(capture(Expanded(), *qkv(1, 2, 64, 80)))
    g = torch.Generator().manual_seed(0)
    bshd = [torch.randn(2, 32, 4, 64, generator=g) for _ in range(3)]  # fp32

    class Bshd(torch.nn.Module):
        def forward(self, q, k, v):
            return patterns.scaled_dot_product_attention_pattern(q, k, v, 0.125)

    assert patterns.tilelang_flash_attn_wrapper not in targets(capture(Bshd(), *bshd))


def test_inplace_and_hand_written_softmax_spellings_still_match():
    """canonicalize_ops / recompose_softmax run in front of the matchers (the reference runs
    canonicalize_ops and decompose_ops in front of its partitioner, backend.py:1521-1530)."""
    class InplaceScale(torch.nn.Module):
        def forward(self, q, k, v):
            s = torch.matmul(q, k.transpose(-2, -1))
            s *= 0.125
            s += torch.triu(torch.full((64, 64), float("-inf"), dtype=q.dtype), diagonal=1)
            return torch.matmul(torch.softmax(s, dim=-1), v)

    gm = capture(InplaceScale(), *qkv())
    nodes = [n for n in gm.graph.nodes if n.op == "call_function" and n.target is B._tilelang_sdpa_direct]
    assert len(nodes) == 1 and nodes[0].kwargs == {"is_causal": True, "scale": 0.125}

    class SafeSoftmaxByHand(torch.nn.Module):
        def forward(self, q, k, v):
            s = torch.matmul(q, k.transpose(-2, -1)) / 8.0
            e = torch.exp(s - torch.amax(s, dim=-1, keepdim=True))
            p = e / torch.sum(e, dim=-1, keepdim=True)
            return torch.matmul(p, v)

    gm = capture(SafeSoftmaxByHand(), *qkv())
    assert targets(gm) == [B._tilelang_sdpa_direct]

    class ResidualInPlace(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = torch.nn.Linear(64, 64, bias=False)
            self.b = torch.nn.Linear(64, 64, bias=False)

        def forward(self, x):
            h = F.silu(self.a(x))
            h = h.clone()
            y = self.b(h)
            y += h            # h is produced inside the graph: the in-place add is unobservable
            return y

    gm = capture(ResidualInPlace().to(torch.bfloat16), torch.randn(4, 16, 64).to(torch.bfloat16))
    lin = [n for n in gm.graph.nodes if n.target is fusion.hb_linear]
    assert len(lin) == 2 and lin[1].kwargs.get("residual") is lin[0]
    assert not any(getattr(t, "__name__", "") in ("iadd", "clone") for t in targets(gm))

    class MutatesItsInput(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = torch.nn.Linear(64, 64, bias=False)

        def forward(self, x):
            x += self.a(x)    # the caller sees x change: must stay an in-place add on x
            return x

    gm = capture(MutatesItsInput().to(torch.bfloat16), torch.randn(4, 16, 64).to(torch.bfloat16))
    lin = [n for n in gm.graph.nodes if n.target is fusion.hb_linear]
    assert len(lin) == 1 and lin[0].kwargs.get("residual") is None
    assert any(getattr(t, "__name__", "") == "iadd" for t in targets(gm))


def test_env_switch_disables_attention_rewrite(monkeypatch):
    monkeypatch.setenv("TILELANG_FRONTEND_ENABLE_FLASHATTN_PATTERN", "0")
    monkeypatch.setenv("TILELANG_FRONTEND_ENABLE_H2O_FUSE", "0")

    class M(torch.nn.Module):
        def forward(self, q, k, v):
            return F.scaled_dot_product_attention(q, k, v, is_causal=True)

    assert B._tilelang_sdpa_direct not in targets(capture(M(), *qkv()))


def test_direct_leaf_call_keeps_reference_rule_and_rejects_cpu():
    q, k, v = qkv(dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        B._tilelang_sdpa_direct(q, k, v)


# ----------------------------------------------------------------------------------------
# GEMM + epilogue fusion
# ----------------------------------------------------------------------------------------
def test_linear_activation_groups():
    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = torch.nn.Linear(64, 128, bias=False)
            self.b = torch.nn.Linear(128, 64, bias=True)

        def forward(self, x):
            return self.b(F.gelu(self.a(x), approximate="tanh"))

    gm = capture(M().to(torch.bfloat16), torch.randn(4, 16, 64).to(torch.bfloat16))
    leaves = [n for n in gm.graph.nodes if n.target is fusion.hb_linear]
    assert [n.kwargs["act"] for n in leaves] == ["gelu_tanh", "none"]
    assert leaves[1].kwargs["bias"] is not None
    assert not any("gelu" in str(t) or "linear" == getattr(t, "__name__", "") for t in targets(gm))


def test_fp32_linear_is_not_lowered():
    gm = capture(torch.nn.Linear(64, 64), torch.randn(8, 64))
    assert fusion.hb_linear not in targets(gm)


def test_llama_layer_lowering():
    from oracle import attention_oracle as O  # the module definition doubles as the test model

    layer = O.LlamaLayer(hidden=256, heads=2, inter=512).init_weights(seed=4).to(torch.bfloat16)
    x = torch.randn(2, 128, 256).to(torch.bfloat16)
    gm = capture(layer, x)
    t = targets(gm)
    assert t.count(B._tilelang_sdpa_direct) == 1
    assert t.count(fusion.hb_swiglu) == 1
    assert t.count(fusion.hb_linear_multi) == 1    # wq, wk, wv as one GEMM
    assert t.count(fusion.hb_linear) == 2          # wo, w_down
    assert t.count(fusion.hb_rms_rowstat) == 2     # one statistic per RMSNorm
    assert fusion.hb_rmsnorm not in t              # both norms folded into their GEMMs
    assert not any(getattr(x, "__name__", "") == "cat" for x in t)            # RoPE moved into the epilogue
    lin = [n for n in gm.graph.nodes if n.target is fusion.hb_linear]
    assert sum(1 for n in lin if n.kwargs.get("residual") is not None) == 2   # wo and w_down
    qkv = next(n for n in gm.graph.nodes if n.target is fusion.hb_linear_multi)
    assert len(qkv.args[1]) == 3 and qkv.kwargs["rope_cols"] == 512 and qkv.kwargs["head_dim"] == 128
    assert qkv.kwargs.get("row_scale") is not None and qkv.kwargs.get("gamma") is not None
    sw = next(n for n in gm.graph.nodes if n.target is fusion.hb_swiglu)
    assert sw.kwargs.get("row_scale") is not None and sw.kwargs.get("gamma") is not None
    sd = next(n for n in gm.graph.nodes if n.target is B._tilelang_sdpa_direct)
    assert sd.kwargs["is_causal"] is True and sd.kwargs.get("out_bshd") is True


def test_leftover_softmax_is_lowered_with_its_scale():
    """Attention with a mask the rewrites refuse keeps its softmax; a 16-bit softmax over the last
    axis becomes hb_softmax and the scalar scale in front of it is folded in."""
    class M(torch.nn.Module):
        def forward(self, q, k, v):
            s = torch.matmul(q, k.transpose(-2, -1))
            p = torch.softmax(s * 0.125, dim=-1)
            return torch.matmul(p, v)

    q, k, v = qkv(dtype=torch.bfloat16)
    # an arbitrary additive bias in front keeps the attention rewrite away in the second module
    class M2(torch.nn.Module):
        def forward(self, q, k, v, bias):
            s = torch.matmul(q, k.transpose(-2, -1)) / 8.0 + bias
            return torch.matmul(F.softmax(s, dim=-1), v)

    gm = capture(M2(), q, k, v, torch.randn(64, 64).to(torch.bfloat16))
    leaves = [n for n in gm.graph.nodes if n.op == "call_function" and n.target is fusion.hb_softmax]
    assert len(leaves) == 1 and leaves[0].args[1] == 1.0  # the scale sits before the bias: not foldable
    assert not any(getattr(t, "__name__", "") == "softmax" for t in targets(gm))

    class M3(torch.nn.Module):
        def forward(self, x):
            return (x / 4.0).softmax(-1) + torch.softmax(x, dim=1) + F.softmax(x.float(), dim=-1).to(x.dtype)

    gm = capture(M3(), torch.randn(4, 32, 64).to(torch.float16))
    leaves = [n for n in gm.graph.nodes if n.op == "call_function" and n.target is fusion.hb_softmax]
    # only the last-axis, 16-bit one is taken (with its 1/4 folded); dim=1 and fp32 stay in PyTorch
    assert len(leaves) == 1 and leaves[0].args[1] == 0.25


def test_einsum_is_read_as_a_batched_product():
    """Two-operand einsums become hb_einsum when they are batched matrix products (the reference's
    ND-GEMM generator takes the same class, codegen.py:412-470); the plan is checked on CPU by
    replaying it with torch.bmm."""
    cases = [("bhid,bhjd->bhij", (2, 3, 16, 32), (2, 3, 24, 32)),      # QK^T: contracted last in both
             ("bhij,bhjd->bhid", (2, 3, 16, 24), (2, 3, 24, 32)),      # PV: row-major right operand
             ("bld,dn->bln", (2, 16, 32), (32, 40)),                   # no batch label: one product
             ("bnl,bdl->bnd", (2, 8, 16), (2, 24, 16)),
             ("ibk,kjb->bji", (5, 2, 16), (16, 8, 2))]                 # permuted output, batch in the middle
    for eq, sa, sb in cases:
        g = torch.Generator().manual_seed(len(eq))
        a, b = torch.randn(*sa, generator=g), torch.randn(*sb, generator=g)
        plan = fusion.einsum_plan(eq, sa, sb)
        assert plan is not None, eq
        ia, ib = plan["ia"], plan["ib"]
        batch, con, af, bf = plan["batch"], plan["contracted"], plan["a_free"], plan["b_free"]
        a3 = a.permute([ia.index(c) for c in batch + af + con]).reshape(plan["B"], plan["M"], plan["K"])
        b3 = b.permute([ib.index(c) for c in batch + con + bf]).reshape(plan["B"], plan["K"], plan["N"])
        nat = batch + af + bf
        got = torch.bmm(a3, b3).reshape([plan["size"][c] for c in nat]).permute([nat.index(c) for c in plan["out"]])
        torch.testing.assert_close(got, torch.einsum(eq, a, b), rtol=1e-5, atol=1e-5)
    for eq, sa, sb in [("ij,jk", (4, 8), (8, 8)), ("...ij,...jk->...ik", (2, 4, 8), (2, 8, 8)), ("ij,jk->k", (4, 8), (8, 8)),
                       ("ii,ij->ij", (8, 8), (8, 8)), ("ij,ij->ij", (8, 8), (8, 8)), ("bij,cjk->bik", (1, 4, 8), (3, 8, 8))]:
        assert fusion.einsum_plan(eq, sa, sb) is None, eq

    class Mixer(torch.nn.Module):
        def forward(self, x, w, y):
            h = torch.einsum("bld,dn->bln", x, w)
            return torch.einsum("bln,bmn->blm", h, y) + torch.einsum("bld,bld->bl", x, x).unsqueeze(-1)

    x, w, y = (torch.randn(*s).to(torch.bfloat16) for s in ((2, 16, 32), (32, 40), (2, 24, 40)))
    gm = capture(Mixer(), x, w, y)
    leaves = [n for n in gm.graph.nodes if n.op == "call_function" and n.target is fusion.hb_einsum]
    assert len(leaves) == 2 and [n.args[0] for n in leaves] == ["bld,dn->bln", "bln,bmn->blm"]
    assert sum(1 for t in targets(gm) if getattr(t, "__name__", "") == "einsum") == 1   # the row-wise dot stays
    gm32 = capture(Mixer(), x.float(), w.float(), y.float())
    assert not any(n.target is fusion.hb_einsum for n in gm32.graph.nodes)
