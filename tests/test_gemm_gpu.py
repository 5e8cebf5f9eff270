"""Parity of the tcgen05 GEMM + epilogue kernels (through the C ABI) with the CPU oracle
and the reference-generated fixtures.  Tolerance: the output is rounded to bf16/fp16, so
errors are measured relative to the magnitude of the result (2e-2 absolute at unit scale)."""
import pytest
import torch

from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["single", "pair"])
def ops(built_lib, request):
    """Every test of this module runs on the single-CTA kernel (128 x 256 tiles) and on CTA pairs
    (tcgen05.mma.cta_group::2, 256 x 256 tiles; forced also where M <= 128 leaves the peer CTA only
    out-of-range rows)."""
    from heddle_b200 import ops as _ops
    prev = _ops.set_gemm_schedule(request.param)
    yield _ops
    _ops.set_gemm_schedule(prev)


def _close(out, ref, tol=2e-2):
    scale = max(1.0, ref.float().abs().max().item())
    err = (out.float().cpu() - ref.float()).abs().max().item()
    assert err <= tol * scale, (err, scale)


def _mk(M, N, K, seed, dtype=torch.bfloat16, wscale=0.05):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(M, K, generator=g).to(dtype)
    w = (torch.randn(N, K, generator=g) * wscale).to(dtype)
    return a, w


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 512), (256, 512, 128), (96, 192, 128),
                                   (1000, 328, 200), (130, 264, 72), (2048, 1024, 1024), (8, 8, 8)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_plain_gemm(ops, M, N, K, dtype):
    a, w = _mk(M, N, K, seed=M + N + K, dtype=dtype)
    out = ops.gemm_epilogue(a.cuda(), w.cuda())
    torch.cuda.synchronize()
    assert ops.status_word() == 0
    _close(out, O.gemm_epilogue(a, w, "none"), tol=1e-2)


@pytest.mark.parametrize("act", ["silu", "relu", "gelu_tanh", "sigmoid", "tanh"])
def test_unary_epilogues(ops, act):
    a, w = _mk(300, 520, 256, seed=5)
    out = ops.gemm_epilogue(a.cuda(), w.cuda(), act)
    _close(out, O.gemm_epilogue(a, w, act), tol=1e-2)


def test_reference_fixture_epilogues(ops, golden):
    gm = golden["gemm"]
    g = torch.Generator().manual_seed(gm["seed"])
    x = torch.randn(96, 128, generator=g).to(torch.bfloat16)
    w = (torch.randn(192, 128, generator=g) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(192, 128, generator=g) * 0.05).to(torch.bfloat16)
    for act in ("none", "silu", "relu", "gelu_tanh", "sigmoid", "tanh"):
        _close(ops.gemm_epilogue(x.cuda(), w.cuda(), act), gm[act], tol=1e-2)
    _close(ops.gemm_epilogue(x.cuda(), torch.cat([w, w2]).cuda(), "swiglu"), gm["swiglu"], tol=1e-2)


@pytest.mark.parametrize("M,N_out,K", [(256, 128, 128), (500, 344, 264), (1024, 1408, 512)])
def test_swiglu(ops, M, N_out, K):
    a, w = _mk(M, 2 * N_out, K, seed=9)
    out = ops.gemm_epilogue(a.cuda(), w.cuda(), "swiglu")
    assert out.shape == (M, N_out)
    _close(out, O.gemm_epilogue(a, w, "swiglu"), tol=1e-2)


def test_row_scale_bias_residual(ops):
    a, w = _mk(384, 512, 320, seed=13)
    g = torch.Generator().manual_seed(14)
    rs = torch.rand(384, generator=g) + 0.5
    bias = torch.randn(512, generator=g).to(torch.bfloat16)
    res = torch.randn(384, 512, generator=g).to(torch.bfloat16)
    out = ops.gemm_epilogue(a.cuda(), w.cuda(), "silu", row_scale=rs.cuda(), bias=bias.cuda(), residual=res.cuda())
    acc = (a.float() @ w.float().t()) * rs[:, None] + bias.float()
    ref = O.epilogue_fp32(acc, "silu") + res.float()
    _close(out, ref, tol=1e-2)


@pytest.mark.parametrize("hd", [64, 128])
def test_rope_epilogue(ops, hd):
    B, S, H = 2, 96, 3
    a, w = _mk(B * S, 3 * H * hd, 256, seed=17)
    cos, sin = O.rope_tables(S, hd)
    out = ops.gemm_epilogue(a.cuda(), w.cuda(), "rope", rope=(cos.cuda(), sin.cuda(), hd, 2 * H * hd))
    ref = O.gemm_epilogue(a, w, "rope", rope=(cos, sin, hd, 2 * H * hd))
    _close(out, ref, tol=1e-2)


def test_rms_rowstat_and_folded_rmsnorm_linear(ops):
    g = torch.Generator().manual_seed(21)
    x = torch.randn(200, 512, generator=g).to(torch.bfloat16)
    r = torch.randn(200, 512, generator=g).to(torch.bfloat16)
    gamma = (torch.rand(512, generator=g) + 0.5)
    w = (torch.randn(384, 512, generator=g) * 0.05).to(torch.bfloat16)
    y, rstd = ops.rms_rowstat(x.cuda(), r.cuda(), eps=1e-5)
    y_ref, rstd_ref = O.rms_rowstat(x, r, 1e-5)
    assert torch.equal(y.cpu(), y_ref)
    assert (rstd.cpu() - rstd_ref).abs().max().item() <= 1e-5 * rstd_ref.abs().max().item() + 1e-6
    # RMSNorm(y) @ w.T  ==  rstd * (y @ (gamma * w).T)
    wf = (w.float() * gamma[None, :]).to(torch.bfloat16)
    out = ops.gemm_epilogue(y, wf.cuda(), row_scale=rstd)
    ref = (y_ref.float() * rstd_ref[:, None] * gamma[None, :]) @ w.float().t()
    _close(out, ref, tol=2e-2)
    _, rstd_only = ops.rms_rowstat(x.cuda(), None, eps=1e-5)
    assert (rstd_only.cpu() - O.rms_rowstat(x, None, 1e-5)[1]).abs().max().item() <= 1e-5


def test_full_size_projection_properties(ops):
    """Config-5 sized GEMM (M=16384, N=4096, K=4096): linearity and a sampled-row oracle check."""
    M, N, K = 16384, 4096, 4096
    gen = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn(M, K, generator=gen, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
    out = ops.gemm_epilogue(a, w)
    torch.cuda.synchronize()
    assert ops.status_word() == 0
    rows = torch.tensor([0, 1, 127, 128, 4097, 16383], device="cuda")
    ref = a[rows].float() @ w.float().t()
    assert (out[rows].float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
    # scaling A by 2 (exact in bf16) doubles the result exactly
    out2 = ops.gemm_epilogue(a * 2, w)
    assert torch.equal(out2.float(), out.float() * 2)
    # deterministic
    assert torch.equal(ops.gemm_epilogue(a, w), out)


def test_prepare_weight_stacks_and_folds(ops):
    """hb_prepare_weight against the torch expression it replaces: bit-exact (one fp32 multiply,
    one rounding), for one to four matrices, strided sources, with and without gamma."""
    g = torch.Generator().manual_seed(5)
    for dtype in (torch.bfloat16, torch.float16):
        K = 264
        ws = [(torch.randn(r, K, generator=g) * 0.05).to(dtype).cuda() for r in (40, 128, 8, 77)]
        gamma = (1.0 + 0.1 * torch.randn(K, generator=g)).to(dtype).cuda()
        for n in (1, 2, 3, 4):
            got = ops.prepare_weight(ws[:n], gamma)
            ref = (torch.cat(ws[:n], 0).float() * gamma.float()[None, :]).to(dtype)
            assert torch.equal(got, ref)
            assert torch.equal(ops.prepare_weight(ws[:n]), torch.cat(ws[:n], 0))
        wide = (torch.randn(64, 2 * K, generator=g) * 0.05).to(dtype).cuda()
        view = wide[:, K:]  # row stride 2K, 16-byte aligned start
        assert torch.equal(ops.prepare_weight([view, ws[0]]), torch.cat([view, ws[0]], 0))
    with pytest.raises(RuntimeError, match="K must be"):
        ops.prepare_weight([torch.zeros(8, 12, dtype=torch.bfloat16, device="cuda")])
    # the operand of a merged, RMSNorm-folded projection: same result as folding on the host
    x = torch.randn(256, K, generator=g).to(torch.bfloat16).cuda()
    w3 = [w.to(torch.bfloat16) for w in ws[:3]]
    gam = gamma.to(torch.bfloat16)
    y = ops.gemm_epilogue(x, ops.prepare_weight(w3, gam), "none")
    ref = x.float() @ (torch.cat(w3, 0).float() * gam.float()[None, :]).to(torch.bfloat16).float().t()
    assert (y.float() - ref).abs().max().item() <= 2e-2


@pytest.mark.parametrize("rows,cols,dtype", [
    (37, 64, torch.bfloat16), (300, 2048, torch.float16), (64, 4096, torch.bfloat16), (9, 16384, torch.bfloat16),
    (5, 200, torch.float16),
])
def test_row_softmax(ops, rows, cols, dtype):
    """hb_row_softmax against torch.softmax in fp32 on the CPU (one rounding to the 16-bit type)."""
    g = torch.Generator().manual_seed(rows + cols)
    x = (3.0 * torch.randn(rows, cols, generator=g)).to(dtype)
    masked = x.clone()
    masked[0, : cols // 2] = float("-inf")  # masked entries (meaningful for a positive scale only)
    for scale in (1.0, 0.125, -0.5):
        xin = masked if scale > 0 else x
        y = ops.row_softmax(xin.cuda(), scale)
        ref = torch.softmax(xin.float() * scale, dim=-1)
        assert y.dtype == dtype and y.shape == x.shape
        assert (y.float().cpu() - ref).abs().max().item() <= 4e-3
        assert (y.float().sum(-1).cpu() - 1.0).abs().max().item() <= 1e-2
    x3 = (torch.randn(2, 3, 40, 72, generator=g)).to(dtype)
    y3 = ops.row_softmax(x3.cuda())
    assert (y3.float().cpu() - torch.softmax(x3.float(), -1)).abs().max().item() <= 4e-3
    with pytest.raises(RuntimeError, match="multiple of 8"):
        ops.row_softmax(torch.zeros(4, 12, dtype=dtype, device="cuda"))


# ----------------------------------------------------------------------------------------
# batched products and the [K, N] operand layout
# ----------------------------------------------------------------------------------------
def _bmm_ref(a, b, act="none"):
    return O.epilogue_fp32(torch.matmul(a.float(), b.float()), act)


@pytest.mark.parametrize("Bn,M,N,K", [(1, 128, 256, 64), (3, 200, 136, 72), (8, 64, 64, 64), (5, 300, 520, 256),
                                      (16, 1024, 128, 1024), (2, 8, 8, 8)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_bmm_row_major_operands(ops, Bn, M, N, K, dtype):
    g = torch.Generator().manual_seed(Bn * 7 + M + N + K)
    a = torch.randn(Bn, M, K, generator=g).to(dtype)
    b = (torch.randn(Bn, K, N, generator=g) * 0.05).to(dtype)
    out = ops.bmm(a.cuda(), b.cuda())
    torch.cuda.synchronize()
    assert ops.status_word() == 0
    _close(out, _bmm_ref(a, b), tol=1e-2)


def test_bmm_transposed_view_and_strided_batches(ops):
    g = torch.Generator().manual_seed(11)
    a = torch.randn(4, 96, 128, generator=g).to(torch.bfloat16)
    w = (torch.randn(4, 200, 128, generator=g) * 0.05).to(torch.bfloat16)       # [B, N, K] storage
    out = ops.bmm(a.cuda(), w.cuda().transpose(1, 2))                            # read K-major, no copy
    _close(out, _bmm_ref(a, w.transpose(1, 2)), tol=1e-2)
    # batches that are slices of a larger tensor (batch stride larger than one matrix)
    big = torch.randn(4, 2, 96, 128, generator=g).to(torch.bfloat16)
    bk = (torch.randn(4, 2, 128, 72, generator=g) * 0.05).to(torch.bfloat16)
    out = ops.bmm(big.cuda()[:, 1], bk.cuda()[:, 0], "gelu_tanh")
    _close(out, _bmm_ref(big[:, 1], bk[:, 0], "gelu_tanh"), tol=1e-2)


def test_gemm_with_kn_operand_bias_and_residual(ops):
    g = torch.Generator().manual_seed(12)
    a = torch.randn(3, 50, 264, generator=g).to(torch.float16)
    b = (torch.randn(264, 328, generator=g) * 0.05).to(torch.float16)
    bias = torch.randn(328, generator=g).to(torch.float16)
    res = torch.randn(3, 50, 328, generator=g).to(torch.float16)
    out = ops.gemm(a.cuda(), b.cuda(), "silu", bias=bias.cuda(), residual=res.cuda())
    ref = O.epilogue_fp32(torch.matmul(a.float(), b.float()) + bias.float(), "silu") + res.float()
    _close(out, ref, tol=1e-2)


def test_reference_named_gemm_leaves(ops):
    """The per-op leaves of Heddle/heddle/frontend/backend.py:258-300, 523-536, 572-598 by name."""
    from heddle_b200.frontend import backend as Bk

    g = torch.Generator().manual_seed(13)
    a = torch.randn(160, 128, generator=g).to(torch.bfloat16)
    b = (torch.randn(128, 192, generator=g) * 0.05).to(torch.bfloat16)
    _close(Bk._tilelang_gemm_wrapper(a.cuda(), b.cuda()), _bmm_ref(a, b), tol=1e-2)
    x = torch.randn(2, 80, 128, generator=g).to(torch.bfloat16)
    w = (torch.randn(192, 128, generator=g) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(192, 128, generator=g) * 0.05).to(torch.bfloat16)
    x2 = x.reshape(-1, 128)
    _close(Bk._tilelang_linear_wrapper(x.cuda(), w.cuda()), O.gemm_epilogue(x2, w, "none").reshape(2, 80, 192), tol=1e-2)
    _close(Bk._tilelang_swiglu_wrapper(x.cuda(), w.cuda(), w2.cuda()),
           O.gemm_epilogue(x2, torch.cat([w, w2]), "swiglu").reshape(2, 80, 192), tol=1e-2)
    a3 = torch.randn(4, 96, 64, generator=g).to(torch.bfloat16)
    b3 = (torch.randn(4, 64, 72, generator=g) * 0.05).to(torch.bfloat16)
    _close(Bk._tilelang_bmm_wrapper(a3.cuda(), b3.cuda()), _bmm_ref(a3, b3), tol=1e-2)


def test_bmm_rejects_what_it_cannot_take(ops):
    a = torch.zeros(2, 16, 12, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros(2, 12, 16, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="multiples of 8"):
        ops.bmm(a, b)
    with pytest.raises(TypeError):
        ops.bmm(a.float(), b.float())


@pytest.mark.parametrize("eq,sa,sb", [("bhid,bhjd->bhij", (2, 3, 80, 64), (2, 3, 72, 64)),
                                      ("bhij,bhjd->bhid", (2, 3, 80, 72), (2, 3, 72, 64)),
                                      ("bld,dn->bln", (3, 50, 128), (128, 200)),
                                      ("ibk,kjb->bji", (40, 2, 64), (64, 24, 2))])
def test_einsum_leaf_on_the_batched_gemm(ops, eq, sa, sb):
    """hb_einsum (one launch of the batched GEMM) against fp32 einsum of the same 16-bit operands."""
    from heddle_b200.frontend import fusion

    g = torch.Generator().manual_seed(len(eq) + sum(sa))
    a = torch.randn(*sa, generator=g).to(torch.bfloat16)
    b = (torch.randn(*sb, generator=g) * 0.1).to(torch.bfloat16)
    out = fusion.hb_einsum(eq, a.cuda(), b.cuda())
    ref = torch.einsum(eq, a.float(), b.float())
    assert tuple(out.shape) == tuple(ref.shape)
    _close(out, ref, tol=1e-2)
    assert ops.status_word() == 0


def test_compiled_module_with_einsums(ops):
    class Mixer(torch.nn.Module):
        def forward(self, x, w, y):
            h = torch.einsum("bld,dn->bln", x, w)
            return torch.einsum("bln,bmn->blm", h, y)

    g = torch.Generator().manual_seed(21)
    x = torch.randn(2, 96, 128, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(128, 160, generator=g) * 0.1).to(torch.bfloat16).cuda()
    y = (torch.randn(2, 72, 160, generator=g) * 0.1).to(torch.bfloat16).cuda()
    m = Mixer()
    ref = torch.einsum("bln,bmn->blm", torch.einsum("bld,dn->bln", x.float(), w.float()).to(torch.bfloat16).float(), y.float())
    from heddle_b200.frontend import fusion, tilelang_backend
    seen = []

    def backend(gm, example_inputs):
        out = tilelang_backend(gm, example_inputs)
        seen.extend(n.target for n in out.graph.nodes if n.op == "call_function")
        return out

    torch._dynamo.reset()
    with torch.no_grad():
        out = torch.compile(m, backend=backend)(x, w, y)
    assert seen.count(fusion.hb_einsum) == 2
    _close(out, ref.cpu(), tol=1e-2)


def test_cta_pairs_and_single_cta_kernels_agree_bitwise(ops):
    """Both kernels accumulate every output element over K in the same order: equal bits."""
    g = torch.Generator().manual_seed(31)
    cases = [(300, 264, 200, "none"), (2048, 1024, 1024, "gelu_tanh"), (640, 512, 320, "swiglu"), (100, 512, 72, "none")]
    prev = ops.set_gemm_schedule("single")
    try:
        for M, N, K, epi in cases:
            a = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
            w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
            ops.set_gemm_schedule("single")
            one = ops.gemm_epilogue(a, w, epi)
            ops.set_gemm_schedule("pair")
            two = ops.gemm_epilogue(a, w, epi)
            assert torch.equal(one, two), (M, N, K, epi)
        b3 = (torch.randn(3, 136, 200, generator=g) * 0.05).to(torch.bfloat16).cuda()   # [B, K, N] row-major
        a3 = torch.randn(3, 260, 136, generator=g).to(torch.bfloat16).cuda()
        ops.set_gemm_schedule("single")
        one = ops.bmm(a3, b3)
        ops.set_gemm_schedule("pair")
        two = ops.bmm(a3, b3)
        assert torch.equal(one, two)
        assert ops.status_word() == 0
    finally:
        ops.set_gemm_schedule(prev)


def test_full_size_projection_by_size_independent_properties(ops):
    """16384 x 4096 x 4096 (the layer's O projection): sampled rows against fp32, the row sums against
    a @ (w^T 1) (a checksum of checksums), and exact linearity in the activation (x2 is exact in bf16)."""
    g = torch.Generator(device="cuda").manual_seed(41)
    M, N, K = 16384, 4096, 4096
    a = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    out = ops.gemm_epilogue(a, w)
    assert ops.status_word() == 0
    rows = torch.tensor([0, 1, 127, 128, 255, 256, 8191, 8192, 16383], device="cuda")
    ref = a[rows].float() @ w.float().t()
    assert float((out[rows].float() - ref).abs().max()) <= 1e-2 * max(1.0, float(ref.abs().max()))
    # sum over the 4096 outputs of a row: rounding errors of the bf16 results add up like a random walk
    checksum = a.float() @ w.float().sum(dim=0)
    got = out.float().sum(dim=1)
    bound = 64.0 * 2.0 ** -9 * out.float().abs().max() + 1e-3 * checksum.abs().max()
    assert float((got - checksum).abs().max()) <= float(bound)
    twice = ops.gemm_epilogue(a * 2, w)
    assert torch.equal(twice, out * 2)
