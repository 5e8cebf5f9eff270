"""hb_rowwise_program on the GPU (through the C ABI) against the CPU oracle interpreter of the same
program, and compiled modules whose pointwise / reduction partitions run on it against eager fp32.
Tolerance: outputs are rounded to bf16 / fp16; the kernel's fp32 functions may differ from the
CPU's in the last fp32 bits, so up to 2 ulps of the 16-bit type (plus 1e-6 absolute) are allowed."""
import pytest
import torch
import torch.nn.functional as F

from oracle.program_oracle import run_program

pytestmark = pytest.mark.gpu


class _OpsInMode:
    """The package's ops with ``rowwise_program`` pinned to one execution mode."""

    def __init__(self, ops, mode):
        self._ops, self.mode = ops, mode

    def rowwise_program(self, *args, **kw):
        return self._ops.rowwise_program(*args, mode=self.mode, **kw)

    def __getattr__(self, name):
        return getattr(self._ops, name)


@pytest.fixture(scope="module", params=["compiled", "interpret"])
def ops(built_lib, request):
    """Every test runs on the kernel compiled for its program and on the interpreter kernel."""
    from heddle_b200 import ops as _ops
    if request.param == "compiled" and not built_lib.hb_rowwise_compiler_available():
        pytest.fail("libnvrtc cannot be loaded on this machine: the specialised rowwise kernels cannot run")
    return _OpsInMode(_ops, request.param)


def _t(*shape, seed=0, dtype=torch.bfloat16, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def _close(got, want, ulps=2.0):
    eps = 2.0 ** -8 if want.dtype == torch.bfloat16 else 2.0 ** -11
    err = (got.float().cpu() - want.float()).abs()
    bound = ulps * eps * want.float().abs().clamp_min(1e-3) + 1e-6
    assert bool((err <= bound).all()), float((err - bound).max())


UNARY = ["neg", "abs", "exp", "log", "log2", "sqrt", "rsqrt", "recip", "sigmoid", "silu", "relu", "gelu_tanh",
         "gelu_erf", "tanh", "round"]
BINARY = ["add", "sub", "rsub", "mul", "div", "rdiv", "max", "min"]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_every_op_against_the_oracle(ops, dtype):
    x = _t(37, 264, seed=1, dtype=dtype)
    y = _t(37, 264, seed=2, dtype=dtype)
    for op in UNARY:
        src = x.abs() + 0.25 if op in ("log", "log2", "sqrt", "rsqrt", "recip") else x
        prog = (("load", "input", 0, 0.0), (op, None, 0, 0.0), ("store_out", None, 0, 0.0))
        _close(ops.rowwise_program(prog, [src.cuda()]), run_program(prog, [src]))
    for op in BINARY:
        b = y.abs() + 0.5 if op in ("div",) else y
        a = x.abs() + 0.5 if op in ("rdiv",) else x
        prog = (("load", "input", 0, 0.0), (op, "input", 1, 0.0), ("store_out", None, 0, 0.0))
        _close(ops.rowwise_program(prog, [a.cuda(), b.cuda()]), run_program(prog, [a, b]))
        prog = (("load", "input", 0, 0.0), (op, "imm", 0, 1.75), ("store_out", None, 0, 0.0))
        _close(ops.rowwise_program(prog, [a.cuda()]), run_program(prog, [a]))
    prog = (("load", "input", 0, 0.0), ("abs", None, 0, 0.0), ("pow", "imm", 0, 1.5), ("store_out", None, 0, 0.0))
    _close(ops.rowwise_program(prog, [x.cuda()]), run_program(prog, [x]), ulps=3.0)
    assert ops.status_word() == 0


def test_broadcast_operands_temporaries_and_two_outputs(ops):
    x, y = _t(4, 50, 128, seed=3), _t(4, 50, 128, seed=4)
    g, s = _t(128, seed=5), _t(4, 50, 1, seed=6).float()
    prog = (("load", "input", 0, 0.0), ("silu", None, 0, 0.0), ("round", None, 0, 0.0), ("mul", "input", 1, 0.0),
            ("store_out", None, 0, 0.0), ("store_tmp", None, 2, 0.0), ("sigmoid", None, 0, 0.0), ("mul", "tmp", 2, 0.0),
            ("mul", "rowvec", 0, 0.0), ("sub", "rowscalar", 0, 0.0), ("store_out", None, 1, 0.0))
    got = ops.rowwise_program(prog, [x.cuda(), y.cuda()], [g.cuda()], [s.cuda()], n_outputs=2)
    want = run_program(prog, [x, y], [g], [s], n_outputs=2)
    for a, b in zip(got, want):
        assert a.shape == x.shape
        _close(a, b)


@pytest.mark.parametrize("rows,cols", [(33, 64), (130, 1024), (17, 1032), (64, 4096), (5, 16384)])
def test_row_reductions_against_the_oracle(ops, rows, cols):
    x = _t(rows, cols, seed=rows + cols)
    softmax = (("load", "input", 0, 0.0), ("reduce_max", None, 0, 0.0), ("sub", "reduced", 0, 0.0), ("exp", None, 0, 0.0),
               ("reduce_sum", None, 1, 0.0), ("div", "reduced", 1, 0.0), ("store_out", None, 0, 0.0))
    got = ops.rowwise_program(softmax, [x.cuda()])
    _close(got, run_program(softmax, [x]))
    _close(got, torch.softmax(x.float(), -1).to(x.dtype))          # and the function it spells
    g = _t(cols, seed=7)
    norm = (("load", "input", 0, 0.0), ("reduce_mean", None, 0, 0.0), ("sub", "reduced", 0, 0.0), ("store_tmp", None, 0, 0.0),
            ("mul", "tmp", 0, 0.0), ("reduce_mean", None, 1, 0.0), ("load", "reduced", 1, 0.0), ("add", "imm", 0, 1e-5),
            ("rsqrt", None, 0, 0.0), ("mul", "tmp", 0, 0.0), ("mul", "rowvec", 0, 0.0), ("store_out", None, 0, 0.0))
    got = ops.rowwise_program(norm, [x.cuda()], [g.cuda()])
    _close(got, run_program(norm, [x], [g]), ulps=3.0)
    ln = F.layer_norm(x.float(), (cols,), g.float(), None, 1e-5).to(x.dtype)
    _close(got, ln, ulps=3.0)
    assert ops.status_word() == 0


def test_strided_rows_and_rejections(ops):
    big = _t(64, 512, seed=9).cuda()
    view = big[:, 128:384]                       # row stride 512, 16-byte aligned start
    prog = (("load", "input", 0, 0.0), ("relu", None, 0, 0.0), ("add", "imm", 0, 1.0), ("store_out", None, 0, 0.0))
    _close(ops.rowwise_program(prog, [view]), run_program(prog, [view.cpu()]))
    with pytest.raises(TypeError):
        ops.rowwise_program(prog, [big.float()])
    with pytest.raises(RuntimeError, match="multiple of 8"):
        ops.rowwise_program(prog, [big[:, :60].contiguous()])
    with pytest.raises(RuntimeError, match="before a LOAD"):
        ops.rowwise_program((("exp", None, 0, 0.0), ("store_out", None, 0, 0.0)), [big])
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.rowwise_program(prog, [big.cpu()])


def test_compiled_modules_run_their_partitions_on_the_kernel(ops):
    import heddle_b200
    from heddle_b200.frontend import fusion

    class Mlp(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = torch.nn.Linear(256, 512, bias=False)
            self.b = torch.nn.Linear(512, 256, bias=False)

        def forward(self, x, g):
            h = self.a(x)
            h = h * torch.sigmoid(1.702 * h) + 0.1 * torch.tanh(h)   # not one of the GEMM epilogues
            y = self.b(h)
            mu = y.mean(-1, keepdim=True)
            d = y - mu
            return d * torch.rsqrt((d * d).mean(-1, keepdim=True) + 1e-5) * g

    torch.manual_seed(0)
    m = Mlp().to(torch.bfloat16).cuda().eval()
    x, g = _t(8, 64, 256, seed=11).cuda(), _t(256, seed=12).cuda()
    seen = []

    def backend(gm, example_inputs):
        out = heddle_b200.frontend.tilelang_backend(gm, example_inputs)
        seen.append([n.target for n in out.graph.nodes if n.op == "call_function"])
        return out

    torch._dynamo.reset()
    with torch.no_grad():
        got = torch.compile(m, backend=backend)(x, g)
        want = m.float()(x.float(), g.float())
    assert seen and seen[0].count(fusion.hb_rowwise) == 2 and seen[0].count(fusion.hb_linear) == 2
    err = (got.float() - want).abs().max().item()
    assert err <= 2e-2 * max(1.0, want.abs().max().item()), err


def test_full_size_programs_by_size_independent_properties(ops):
    """32768 x 4096 bf16 (the bench configuration): exact doubling, a softmax program whose rows sum to one,
    and a sampled block against the CPU oracle."""
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(32768, 4096, generator=g, device="cuda").to(torch.bfloat16)
    y = torch.randn(32768, 4096, generator=g, device="cuda").to(torch.bfloat16)
    double = (("load", "input", 0, 0.0), ("mul", "imm", 0, 2.0), ("store_out", None, 0, 0.0))
    assert torch.equal(ops.rowwise_program(double, [x]), x * 2)
    chain = (("load", "input", 0, 0.0), ("silu", None, 0, 0.0), ("mul", "input", 1, 0.0), ("add", "imm", 0, 1.5),
             ("store_out", None, 0, 0.0))
    out = ops.rowwise_program(chain, [x, y])
    rows = slice(20000, 20064)
    _close(out[rows], run_program(chain, [x[rows].cpu(), y[rows].cpu()]))
    softmax = (("load", "input", 0, 0.0), ("reduce_max", None, 0, 0.0), ("sub", "reduced", 0, 0.0), ("exp", None, 0, 0.0),
               ("store_tmp", None, 0, 0.0), ("reduce_sum", None, 1, 0.0), ("load", "tmp", 0, 0.0), ("div", "reduced", 1, 0.0),
               ("store_out", None, 0, 0.0))
    p = ops.rowwise_program(softmax, [x])
    sums = p.float().sum(dim=1)
    assert float((sums - 1.0).abs().max()) <= 4e-3      # 4096 bf16 roundings of values that sum to one
    assert float(p.float().min()) >= 0.0
    _close(p[rows], run_program(softmax, [x[rows].cpu()]), ulps=3.0)
    assert ops.status_word() == 0
