"""Pointwise / row-reduction partitions: grouping (GraphPartitioner), pruning switches, lowering to
the rowwise op-code program, and the program's arithmetic — checked on CPU by running every lowered
program through the oracle interpreter (oracle/program_oracle.py) and comparing with the values the
captured FX graph itself produces for the same nodes."""
import copy

import pytest
import torch
import torch.fx as fx
import torch.nn.functional as F

from heddle_b200.frontend.partitioner import GraphPartitioner, lower_partition
from heddle_b200.frontend.support import Capability, SupportPolicy
from oracle.program_oracle import run_program


def capture_raw(module, *inputs):
    got = []

    def backend(gm, example_inputs):
        got.append(copy.deepcopy(gm))
        return gm.forward

    torch._dynamo.reset()
    with torch.no_grad():
        torch.compile(module, backend=backend)(*inputs)
    assert len(got) == 1
    return got[0]


class Recorder(fx.Interpreter):
    def __init__(self, gm):
        super().__init__(gm)
        self.values = {}

    def run_node(self, n):
        out = super().run_node(n)
        self.values[n] = out
        return out


def eval_partition_fp32(p, values):
    """The partition's nodes evaluated in fp32 from the graph's own (16-bit valued) partition inputs."""
    env = {}

    def val(a):
        if isinstance(a, fx.Node):
            if a in env:
                return env[a]
            v = values[a]
            return v.float() if isinstance(v, torch.Tensor) and v.is_floating_point() else v
        return a

    for n in p.nodes:
        args = fx.node.map_arg(n.args, val)
        kwargs = fx.node.map_arg(n.kwargs, val)
        env[n] = n.target(*args, **kwargs) if n.op == "call_function" else getattr(args[0], n.target)(*args[1:], **kwargs)
    return env


def check_partitions(module, *inputs, expect_parts=None, tol_ulps=2.0, **env):
    """Partition + lower the captured graph; every program must reproduce the graph's own values: the
    fp32 evaluation of the graph for the default lowering (fp32 chain, one rounding at the store), and
    the 16-bit eager evaluation for ``exact_intermediates=True`` on pure pointwise groups."""
    gm = capture_raw(module, *inputs)
    gp = GraphPartitioner(gm)
    parts = gp.partition()
    if expect_parts is not None:
        assert len(parts) == expect_parts, (gp.prune_stats, [[n.name for n in p.nodes] for p in parts])
    rec = Recorder(gm)
    with torch.no_grad():
        rec.run(*inputs)
    lowered = []
    for p in parts:
        has_reduction = any(n.target in (torch.sum, torch.mean, torch.amax) or str(n.target) in ("sum", "mean", "amax")
                            for n in p.nodes)
        modes = (False,) if has_reduction else (False, True)
        with torch.no_grad():
            fp32 = eval_partition_fp32(p, rec.values)
        for exact in modes:
            lp = lower_partition(p, exact_intermediates=exact)
            assert lp is not None, [n.name for n in p.nodes]
            assert any(i[0] == "round" for i in lp.program) == exact
            outs = run_program(lp.program, [rec.values[n] for n in lp.inputs], [rec.values[n] for n in lp.rowvecs],
                               [rec.values[n] for n in lp.rowscalars], len(lp.outputs))
            outs = outs if isinstance(outs, tuple) else (outs,)
            for node, got in zip(lp.outputs, outs):
                # default: the fp32 graph rounded once; exact: eager's own 16-bit values.  What is left is the
                # difference between two fp32 evaluations of the same formula: a few 16-bit ulps
                want = rec.values[node] if exact else fp32[node].to(rec.values[node].dtype)
                assert got.shape == want.shape and got.dtype == want.dtype
                eps = 2.0 ** -8 if want.dtype == torch.bfloat16 else 2.0 ** -11
                err = (got.float() - want.float()).abs()
                bound = tol_ulps * eps * want.float().abs().clamp_min(1e-3) + 1e-6
                assert bool((err <= bound).all()), (node.name, exact, float(err.max()), lp.program)
        lowered.append(lower_partition(p))
    return gm, parts, lowered


def bf(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)


def test_policy_classification_and_reasons():
    class M(torch.nn.Module):
        def forward(self, x, w):
            y = F.linear(x, w)
            z = torch.exp(y) * 2.0
            return z.clone().expand(2, *z.shape), torch.sort(z)[0], z.view(-1)

    gm = capture_raw(M(), bf(16, 64), bf(64, 64, seed=1))
    pol = SupportPolicy.default()
    by_name = {getattr(n.target, "__name__", str(n.target)): n for n in gm.graph.nodes if n.op != "placeholder"}
    assert pol.classify(by_name["linear"]) == Capability.SUPPORTED and pol.family(by_name["linear"]) == "gemm"
    assert pol.family(by_name["exp"]) == "pointwise" and pol.op_name(by_name["exp"]) == "exp"
    assert pol.classify(by_name["clone"]) == Capability.HARD_BOUNDARY
    assert pol.classify(by_name["expand"]) == Capability.HARD_BOUNDARY
    assert pol.classify(by_name["view"]) == Capability.SOFT_BOUNDARY
    assert pol.classify(by_name["sort"]) == Capability.UNSUPPORTED
    assert "stays in PyTorch" in pol.explain(by_name["sort"])
    assert not pol.is_supported_inside_partition(by_name["linear"])  # GEMMs are lowered by the pattern passes


def test_chain_with_broadcast_operands_and_two_outputs():
    class M(torch.nn.Module):
        def forward(self, x, y, g, s):
            h = F.silu(x) * y + 1.5
            z = (h * torch.sigmoid(h) * g - s) / 3.0
            return z, h

    x, y = bf(4, 64, 128), bf(4, 64, 128, seed=1)
    g, s = bf(128, seed=2), bf(4, 64, 1, seed=3)
    gm, parts, lowered = check_partitions(M(), x, y, g, s, expect_parts=1)
    lp = lowered[0]
    assert len(lp.inputs) == 2 and len(lp.rowvecs) == 1 and len(lp.rowscalars) == 1 and len(lp.outputs) == 2
    ops = [i[0] for i in lp.program]
    assert ops.count("store_out") == 2 and "store_tmp" in ops  # h is needed again after sigmoid(h)


def test_softmax_written_by_hand_and_layernorm_like_reductions():
    class Softmax(torch.nn.Module):
        def forward(self, x):
            e = torch.exp(x - torch.amax(x, dim=-1, keepdim=True))
            return e / torch.sum(e, dim=-1, keepdim=True)

    _, _, lowered = check_partitions(Softmax(), bf(8, 32, 256), expect_parts=1)
    ops = [i[0] for i in lowered[0].program]
    assert ops.count("reduce_max") == 1 and ops.count("reduce_sum") == 1
    assert ops.index("reduce_max") < ops.index("exp") < ops.index("reduce_sum")

    class Norm(torch.nn.Module):
        def forward(self, x, g):
            mu = x.mean(-1, keepdim=True)
            d = x - mu
            var = (d * d).mean(-1, keepdim=True)
            return d * torch.rsqrt(var + 1e-5) * g

    check_partitions(Norm(), bf(4, 16, 512), bf(512, seed=5), expect_parts=1, tol_ulps=4.0)


def test_unsupported_node_splits_the_groups_and_stays_eager():
    class M(torch.nn.Module):
        def forward(self, x):
            a = torch.tanh(x) * 0.5 + x
            b = torch.cumsum(a, dim=-1)          # no native kernel: boundary
            return torch.relu(b) * torch.sigmoid(b) - 1.0

    gm, parts, _ = check_partitions(M(), bf(64, 128), expect_parts=2)
    assert all("cumsum" not in [getattr(n.target, "__name__", "") for n in p.nodes] for p in parts)


def test_groups_stay_convex():
    """y depends on the group through an unsupported node; joining it would create a cycle."""
    class M(torch.nn.Module):
        def forward(self, x):
            a = torch.exp(x) * 2.0
            y = torch.cumsum(a, dim=-1)
            return (a + 1.0) * y + a

    gm, parts, _ = check_partitions(M(), bf(64, 128))
    for p in parts:
        inside = set(p.nodes)
        for n in p.nodes:
            for a in n.all_input_nodes:
                if a not in inside:
                    # no external input may depend on a member of the group
                    stack, seen = [a], set()
                    while stack:
                        m = stack.pop()
                        assert m not in inside
                        for b in m.all_input_nodes:
                            if b not in seen:
                                seen.add(b)
                                stack.append(b)


def test_prune_switches_keep_their_names_and_defaults(monkeypatch):
    class M(torch.nn.Module):
        def forward(self, x, y):
            return torch.relu(x + y), torch.exp(x) * y * 0.5 + y

    x, y = bf(64, 128), bf(64, 128, seed=1)
    gm = capture_raw(M(), x, y)
    gp = GraphPartitioner(gm)
    parts = gp.partition()
    # relu(x + y): 2 nodes, 2 inputs, 1 output -> 2/6 flop per byte < 0.5: pruned as memory-bound
    assert gp.prune_stats["low_ai"] == 1 and gp.prune_stats["kept"] == 1 and len(parts) == 1
    monkeypatch.setenv("TILELANG_FRONTEND_MIN_AI", "0.0")
    assert len(GraphPartitioner(gm).partition()) == 2
    monkeypatch.setenv("TILELANG_FRONTEND_MIN_NODES", "3")
    assert len(GraphPartitioner(gm).partition()) == 1
    monkeypatch.setenv("TILELANG_FRONTEND_MIN_NODES", "2")
    monkeypatch.setenv("TILELANG_FRONTEND_MIN_ELEMS", str(64 * 128 + 1))
    assert GraphPartitioner(gm).partition() == []


def test_operands_the_machine_cannot_address_are_left_out():
    class M(torch.nn.Module):
        def forward(self, x, col, f32):
            a = torch.exp(x) * 2.0
            b = a * col          # [rows-like broadcast of a different rank]: not addressable
            return b + f32       # fp32 operand promotes the result: not a 16-bit node

    x = bf(8, 16, 128)
    gm = capture_raw(M(), x, bf(16, 1, seed=2), torch.randn(8, 16, 128))
    parts = GraphPartitioner(gm).partition()
    names = [[getattr(n.target, "__name__", "") for n in p.nodes] for p in parts]
    assert names == [["exp", "mul"]]


def test_independent_sibling_chains_merge_into_one_group():
    class M(torch.nn.Module):
        def forward(self, h):
            return h * torch.sigmoid(1.702 * h) + 0.1 * torch.tanh(h)

    _, parts, lowered = check_partitions(M(), bf(32, 256), expect_parts=1)
    assert len(parts[0].nodes) == 6 and len(lowered[0].inputs) == 1
