"""The torch.compile backend end to end on the GPU: rewritten graphs run on the sm_100a kernels
and match the reference-generated fixtures."""
import math

import pytest
import torch

from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def backend(built_lib):
    import heddle_b200
    heddle_b200.init()
    from heddle_b200.frontend import tilelang_backend
    return tilelang_backend


def _compile(module, backend):
    torch._dynamo.reset()
    return torch.compile(module, backend=backend)


def test_config1_module_through_the_backend(backend, golden):
    """softmax(Q K^T / sqrt(D)) V, B1 H4 S256 D64, seed 0: the reference's FX-captured eager result."""
    class Attn(torch.nn.Module):
        def forward(self, q, k, v):
            s = torch.matmul(q, k.transpose(-2, -1)) / math.sqrt(q.shape[-1])
            return torch.matmul(torch.softmax(s, dim=-1), v)

    case = golden["c1"]
    q, k, v = O.make_qkv(1, 4, 4, 256, 256, 64, seed=0, dtype=torch.bfloat16)
    with torch.no_grad():
        out = _compile(Attn(), backend)(q.cuda(), k.cuda(), v.cuda())
    assert out.dtype == torch.bfloat16
    assert (out.float().cpu() - case["out"]).abs().max().item() <= 2e-2


def test_sdpa_module_causal_gqa(backend):
    class M(torch.nn.Module):
        def forward(self, q, k, v):
            return torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)

    q, k, v = O.make_qkv(2, 8, 2, 320, 320, 128, seed=6, dtype=torch.bfloat16)
    with torch.no_grad():
        out = _compile(M(), backend)(q.cuda(), k.cuda(), v.cuda())
    ref, _ = O.attention_eager(q, k, v, causal=True)
    assert (out.float().cpu() - ref).abs().max().item() <= 2e-2


def test_small_llama_layer_through_the_backend(backend, golden):
    case = golden["llama_small"]
    layer = O.LlamaLayer(hidden=256, heads=2, inter=512).init_weights(seed=case["seed"]).to(torch.bfloat16).cuda()
    x = torch.randn(2, 128, 256, generator=torch.Generator().manual_seed(case["x_seed"])).to(torch.bfloat16)
    with torch.no_grad():
        out = _compile(layer, backend)(x.cuda())
    ref = case["out"]
    err = (out.float().cpu() - ref).abs().max().item()
    assert err <= 2e-2 * max(1.0, ref.abs().max().item()), err


def test_mlp_block_matches_oracle_epilogues(backend):
    class MLP(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.up = torch.nn.Linear(256, 768, bias=True)
            self.down = torch.nn.Linear(768, 256, bias=False)

        def forward(self, x):
            return x + self.down(torch.nn.functional.gelu(self.up(x), approximate="tanh"))

    torch.manual_seed(0)
    m = MLP().to(torch.bfloat16)
    x = torch.randn(3, 50, 256).to(torch.bfloat16)
    h = O.gemm_epilogue(x.reshape(-1, 256), m.up.weight.data, "none").float() + m.up.bias.data.float()
    h = O.epilogue_fp32(h, "gelu_tanh").to(torch.bfloat16)
    ref = O.gemm_epilogue(h, m.down.weight.data, "none", residual=x.reshape(-1, 256)).reshape(3, 50, 256)
    with torch.no_grad():
        out = _compile(m.cuda(), backend)(x.cuda())
    assert (out.float().cpu() - ref.float()).abs().max().item() <= 3e-2


def test_full_size_llama_layer(backend):
    """The fused-layer configuration at full size: hidden 4096, 32 heads of 128, SwiGLU 11008, eps 1e-5,
    theta 10000, batch 8 x seq 2048, weights N(0, 0.02), activations N(0, 1), bf16.  The whole batch runs
    through the compiled layer; batch element 0 is checked against the fp32 eager module on the CPU
    (the layer is data-parallel over batch), every element for finiteness and batch-independence."""
    layer = O.LlamaLayer().init_weights(seed=0).to(torch.bfloat16)
    x = torch.randn(8, 2048, 4096, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    with torch.no_grad():
        out = _compile(copy_to_cuda(layer), backend)(x.cuda())
        torch.cuda.synchronize()
        assert out.shape == x.shape and torch.isfinite(out.float()).all()
        ref_layer = O.LlamaLayer().init_weights(seed=0)
        for p in ref_layer.parameters():
            p.data = p.data.to(torch.bfloat16).float()
        ref = ref_layer(x[:1].float())
    err = (out[:1].float().cpu() - ref).abs().max().item()
    assert err <= 2e-2 * max(1.0, ref.abs().max().item()), err
    # the same sequence placed at another batch index gives the same rows
    with torch.no_grad():
        x2 = x.clone()
        x2[5] = x[0]
        out2 = _compile(copy_to_cuda(layer), backend)(x2.cuda())
    assert torch.equal(out2[5], out[0])


def copy_to_cuda(module):
    import copy
    return copy.deepcopy(module).cuda()


def test_biased_attention_runs_the_softmax_kernel(backend):
    """An additive bias the attention rewrites refuse: the graph keeps its matmuls and gets
    hb_softmax for the row softmax; result against the same module in fp32 on the CPU."""
    from heddle_b200.frontend import fusion

    class Biased(torch.nn.Module):
        def forward(self, q, k, v, bias):
            s = torch.matmul(q, k.transpose(-2, -1)) / 8.0 + bias
            return torch.matmul(torch.softmax(s, dim=-1), v)

    g = torch.Generator().manual_seed(4)
    q, k, v = (torch.randn(2, 4, 256, 64, generator=g).to(torch.bfloat16) for _ in range(3))
    bias = torch.randn(256, 256, generator=g).to(torch.bfloat16)
    seen = []

    def recording(gm, example_inputs):
        out = backend(gm, example_inputs)
        seen.append([n.target for n in out.graph.nodes if n.op == "call_function"] if hasattr(out, "graph") else [])
        return out

    torch._dynamo.reset()
    with torch.no_grad():
        got = torch.compile(Biased(), backend=recording)(q.cuda(), k.cuda(), v.cuda(), bias.cuda())
        ref = Biased()(q.float(), k.float(), v.float(), bias.float())
    assert any(fusion.hb_softmax in t for t in seen)
    assert (got.float().cpu() - ref).abs().max().item() <= 3e-2
