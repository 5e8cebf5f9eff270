"""GEMM + epilogue fusion on a captured FX graph.

The reference reaches its fused GEMM kernels through decomposition, canonicalisation,
shape propagation, a DFS partitioner and a source-text code generator
(Heddle/heddle/frontend/backend.py:1521-1812, partitioner.py:343-400,
codegen.py:980-1244).  The kernels here are fixed, so that machinery collapses into a
direct lowering: each group the reference's partitioner would keep around a GEMM
(``linear`` + unary epilogue, the dual-GEMM SwiGLU, codegen.py:1181-1202) is replaced by
one ``@torch.fx.wrap`` leaf that calls ``hb_gemm_epilogue``.  Two further groups the
reference only analyses (elementwise_fusion.py:59-143) are lowered as well: the
residual add behind a projection, and RMSNorm in front of projections — folded as
``RMSNorm(x) W^T = diag(rstd) (x (gamma * W)^T)`` with one ``hb_rms_rowstat`` pass.

Passes, in order:  RMSNorm recognition -> linear(+activation) -> SwiGLU -> residual add
-> RMSNorm folding into its consumer GEMMs -> rotate-half RoPE into the projection epilogue ->
sibling projections (Q, K, V) merged into one GEMM on stacked weights.
"""
from __future__ import annotations

import collections
import operator
import weakref
from typing import Dict, List, Optional, Tuple

import torch
import torch.fx as fx

from .. import ops

_ACT_NAMES = {"silu": "silu", "relu": "relu", "sigmoid": "sigmoid", "tanh": "tanh"}


# ----------------------------------------------------------------------------------------
# leaves
# ----------------------------------------------------------------------------------------
class _PreparedWeights:
    """Cache of stacked / gamma-folded weight operands, one entry per group of source tensors.

    An entry is keyed by the identity of its source tensors and remembers their storage addresses
    and versions: a hit requires the very same tensor objects, unchanged.  An in-place update
    (optimizer step), a ``.data`` swap or a reload replaces the entry instead of adding one, and a
    finalizer drops the entry when a source tensor dies, so the cache holds at most one operand per
    live weight group (and never more than ``capacity``)."""

    def __init__(self, capacity: int = 256):
        self.capacity = capacity
        self._entries: "collections.OrderedDict[Tuple[int, ...], Tuple]" = collections.OrderedDict()

    @staticmethod
    def _state(t: torch.Tensor) -> Tuple:
        try:
            version = t._version
        except RuntimeError:  # inference-mode tensors do not track versions
            version = -1
        return (t.data_ptr(), version, tuple(t.shape), tuple(t.stride()), t.dtype, str(t.device))

    def get(self, sources, build):
        key = tuple(id(t) for t in sources)
        state = tuple(self._state(t) for t in sources)
        entry = self._entries.get(key)
        if entry is not None:
            refs, old_state, value = entry
            if old_state == state and all(r() is t for r, t in zip(refs, sources)):
                self._entries.move_to_end(key)
                return value
        value = build()

        def drop(_ref, key=key, entries=self._entries):
            entries.pop(key, None)

        self._entries[key] = (tuple(weakref.ref(t, drop) for t in sources), state, value)
        self._entries.move_to_end(key)
        while len(self._entries) > self.capacity:
            self._entries.popitem(last=False)
        return value

    def __len__(self) -> int:
        return len(self._entries)

    def clear(self) -> None:
        self._entries.clear()


_prepared = _PreparedWeights()


def _prepare(ws, gamma: Optional[torch.Tensor]) -> torch.Tensor:
    """The GEMM's weight operand: the given nn.Linear weights stacked along the rows ([Wg; Wu],
    [Wq; Wk; Wv]; the reference concatenates likewise, codegen.py:1146-1152) with the RMSNorm
    weight folded into the columns, built once per state of (weights, gamma) by hb_prepare_weight
    (the reference caches its transposed weight by ``data_ptr()`` alone, codegen.py:1128-1129)."""
    ws = tuple(ws)
    if len(ws) == 1 and gamma is None:
        return ws[0]

    def build():
        if len(ws) <= 4 and all(w.shape[1] % 8 == 0 and w.dtype in (torch.bfloat16, torch.float16) for w in ws):
            return ops.prepare_weight(ws, gamma)
        # more than four matrices or an odd K: compose on the device with torch
        hit = torch.cat(list(ws), dim=0)
        if gamma is not None:
            hit = (hit.float() * gamma.float()[None, :]).to(hit.dtype)
        return hit.contiguous()

    sources = ws if gamma is None else ws + (gamma,)
    return _prepared.get(sources, build)


@torch.fx.wrap
def hb_linear(x, w, bias=None, act="none", residual=None, row_scale=None, gamma=None,
              rope_cos=None, rope_sin=None, head_dim=0):
    """act(row_scale * (x @ (gamma*w).T) + bias) + residual in one kernel; with ``rope_cos`` /
    ``rope_sin`` ([S, head_dim/2]) the rotate-half rotary embedding is applied per head instead
    of an activation (position = row index modulo S)."""
    w = _prepare((w,), gamma)
    if rope_cos is not None:
        return ops.gemm_epilogue(x, w, "rope", bias=bias, residual=residual, row_scale=row_scale,
                                 rope=(rope_cos, rope_sin, head_dim, w.shape[0]))
    return ops.gemm_epilogue(x, w, act, bias=bias, residual=residual, row_scale=row_scale)


@torch.fx.wrap
def hb_linear_multi(x, ws, row_scale=None, gamma=None, rope_cos=None, rope_sin=None, head_dim=0, rope_cols=0):
    """Several projections of one input as a single GEMM on the stacked weights (e.g. Q, K, V):
    returns the (..., sum N_i) result; columns [0, rope_cols) carry the rotary embedding."""
    w = _prepare(ws, gamma)
    if rope_cos is not None and rope_cols > 0:
        return ops.gemm_epilogue(x, w, "rope", row_scale=row_scale, rope=(rope_cos, rope_sin, head_dim, rope_cols))
    return ops.gemm_epilogue(x, w, "none", row_scale=row_scale)


@torch.fx.wrap
def hb_swiglu(x, wg, wu, residual=None, row_scale=None, gamma=None):
    """silu(x @ wg.T) * (x @ wu.T) in one kernel."""
    w = _prepare((wg, wu), gamma)
    return ops.gemm_epilogue(x, w, "swiglu", residual=residual, row_scale=row_scale)


@torch.fx.wrap
def hb_rmsnorm(x, gamma, eps):
    """Unfused RMSNorm (kept only when a consumer cannot absorb it)."""
    _, rstd = ops.rms_rowstat(x, None, eps)
    return (x.float() * rstd[..., None] * gamma.float()).to(x.dtype)


@torch.fx.wrap
def hb_rms_rowstat(x, eps):
    """rsqrt(mean(x^2) + eps) per row, fp32."""
    return ops.rms_rowstat(x, None, eps)[1]


@torch.fx.wrap
def hb_softmax(x, scale=1.0):
    """softmax(scale * x) over the last dimension in one kernel (``hb_row_softmax``)."""
    return ops.row_softmax(x, scale)


@torch.fx.wrap
def hb_matmul(a, b):
    """``torch.matmul(a, b)`` for 16-bit operands on the tcgen05 GEMM: a 2-D ``b`` is one product
    (``_tilelang_gemm_wrapper``), equal leading dimensions are a batch (``_tilelang_bmm_wrapper``, one
    launch with the batch in the tile list).  The right operand is read where it lies, row-major
    [K, N] or a transposed view of [N, K] storage."""
    if b.dim() == 2:
        return ops.gemm(a, b)
    lead = a.shape[:-2]
    out = ops.bmm(a.reshape(-1, a.shape[-2], a.shape[-1]), b.reshape(-1, b.shape[-2], b.shape[-1]))
    return out.reshape(*lead, a.shape[-2], b.shape[-1])


def einsum_plan(equation: str, shape_a, shape_b):
    """Reads a two-operand einsum as a batched GEMM: labels in both operands and the output are the
    batch, labels in both operands only are contracted, the rest are the free (M / N) labels of the
    operand they occur in — the classification of the reference's ND-GEMM generator
    (Heddle/heddle/frontend/codegen.py:455-470).  Returns None for what is not such a product
    (ellipsis, implicit output, repeated labels, a label summed out of one operand, nothing contracted)."""
    eq = equation.replace(" ", "")
    if "->" not in eq or "." in eq:
        return None
    lhs, out = eq.split("->")
    if lhs.count(",") != 1:
        return None
    ia, ib = lhs.split(",")
    if len(set(ia)) != len(ia) or len(set(ib)) != len(ib) or len(set(out)) != len(out):
        return None
    if len(ia) != len(shape_a) or len(ib) != len(shape_b) or not set(out) <= set(ia) | set(ib):
        return None
    size = {}
    for labels, shape in ((ia, shape_a), (ib, shape_b)):
        for c, n in zip(labels, shape):
            if size.setdefault(c, int(n)) != int(n):
                return None  # broadcasting of size-1 dimensions stays in PyTorch
    batch = [c for c in out if c in ia and c in ib]
    contracted = [c for c in ia if c in ib and c not in out]
    a_free = [c for c in ia if c not in ib]
    b_free = [c for c in ib if c not in ia]
    if not contracted or any(c not in out for c in a_free + b_free):
        return None

    def prod(labels):
        r = 1
        for c in labels:
            r *= size[c]
        return r

    return {"ia": ia, "ib": ib, "out": out, "batch": batch, "contracted": contracted, "a_free": a_free, "b_free": b_free,
            "size": size, "B": prod(batch), "M": prod(a_free), "N": prod(b_free), "K": prod(contracted)}


@torch.fx.wrap
def hb_einsum(equation, a, b):
    """Two-operand ``torch.einsum`` as ONE launch of the batched tcgen05 GEMM: the operands are viewed
    as [batch, M, K] and [batch, K, N] (permutations are views; a copy is made only where the merged
    dimensions are not contiguous in storage), the right operand keeps whichever of its two layouts
    it already has, and the result is viewed back in the output's label order.  The reference
    generates an ND-indexed GEMM for the same node (Heddle/heddle/frontend/codegen.py:412-978)."""
    plan = einsum_plan(equation, a.shape, b.shape)
    if plan is None:
        raise ValueError(f"hb_einsum cannot read {equation!r} as a batched matrix product")
    ia, ib, size = plan["ia"], plan["ib"], plan["size"]
    batch, con, af, bf = plan["batch"], plan["contracted"], plan["a_free"], plan["b_free"]
    a3 = a.permute([ia.index(c) for c in batch + af + con]).reshape(plan["B"], plan["M"], plan["K"])
    # contracted labels last in b's own order: [batch, N, K] storage, read through the K-major path
    if [c for c in ib if c not in batch][-len(con):] == con:
        b3 = b.permute([ib.index(c) for c in batch + bf + con]).reshape(plan["B"], plan["N"], plan["K"]).transpose(1, 2)
    else:
        b3 = b.permute([ib.index(c) for c in batch + con + bf]).reshape(plan["B"], plan["K"], plan["N"])
    o3 = ops.bmm(a3, b3)
    natural = batch + af + bf
    o = o3.reshape([size[c] for c in natural])
    return o.permute([natural.index(c) for c in plan["out"]])


@torch.fx.wrap
def hb_rowwise(inputs, rowvecs, rowscalars, program, n_outputs=1):
    """A fused group of pointwise / row-reduction nodes as one ``hb_rowwise_program`` launch.
    ``program`` is the accumulator-machine program ``partitioner.lower_partition`` produced."""
    return ops.rowwise_program(program, inputs, rowvecs, rowscalars, n_outputs)


GEMM_LEAVES = (hb_linear, hb_swiglu, hb_linear_multi)


# ----------------------------------------------------------------------------------------
# matching helpers
# ----------------------------------------------------------------------------------------
def _fname(n) -> str:
    if not isinstance(n, fx.Node):
        return ""
    if n.op == "call_function":
        return getattr(n.target, "__name__", None) or str(n.target)
    if n.op == "call_method":
        return str(n.target)
    return ""


def _is_linear(n) -> bool:
    return isinstance(n, fx.Node) and n.op == "call_function" and _fname(n) == "linear"


def _meta_dtype(n) -> Optional[torch.dtype]:
    if not isinstance(n, fx.Node):
        return None
    v = n.meta.get("example_value", n.meta.get("val", None))
    return getattr(v, "dtype", None)


def _meta_shape(n) -> Optional[Tuple[int, ...]]:
    v = n.meta.get("example_value", n.meta.get("val", None)) if isinstance(n, fx.Node) else None
    return tuple(int(s) for s in v.shape) if v is not None and hasattr(v, "shape") else None


def _gemm_supported(x: fx.Node, w: fx.Node) -> bool:
    """The kernels take bf16/fp16 operands with K and N multiples of 8."""
    dt = _meta_dtype(x)
    ws = _meta_shape(w)
    if dt is not None and dt not in (torch.bfloat16, torch.float16):
        return False
    if dt is not None and _meta_dtype(w) not in (None, dt):
        return False
    if ws is not None and (len(ws) != 2 or ws[0] % 8 or ws[1] % 8):
        return False
    return True


def _act_of(n: fx.Node) -> Optional[str]:
    nm = _fname(n)
    if nm in _ACT_NAMES:
        return _ACT_NAMES[nm]
    if nm == "gelu" and (n.kwargs.get("approximate") == "tanh" or (len(n.args) > 1 and n.args[1] == "tanh")):
        return "gelu_tanh"
    return None


def _single_user(n: fx.Node) -> Optional[fx.Node]:
    users = list(n.users)
    return users[0] if len(users) == 1 else None


def _match_rmsnorm(mul_g: fx.Node) -> Optional[Tuple[fx.Node, fx.Node, float]]:
    """x * rsqrt(mean(x^2, -1, keepdim) + eps) * gamma  ->  (x, gamma, eps)."""
    if _fname(mul_g) != "mul" or len(mul_g.args) != 2:
        return None
    for inner, gamma in (mul_g.args, mul_g.args[::-1]):
        if not (isinstance(inner, fx.Node) and isinstance(gamma, fx.Node)) or _fname(inner) != "mul":
            continue
        for x, rs in (inner.args, inner.args[::-1]):
            if not (isinstance(x, fx.Node) and isinstance(rs, fx.Node)) or _fname(rs) != "rsqrt":
                continue
            add = rs.args[0]
            if not isinstance(add, fx.Node) or _fname(add) != "add":
                continue
            mean, eps = add.args[0], add.args[1]
            if not isinstance(eps, (int, float)) or not isinstance(mean, fx.Node) or _fname(mean) != "mean":
                continue
            dim = mean.args[1] if len(mean.args) > 1 else mean.kwargs.get("dim")
            keep = mean.args[2] if len(mean.args) > 2 else mean.kwargs.get("keepdim", False)
            pw = mean.args[0]
            if dim not in (-1, (-1,), [-1]) or not keep or not isinstance(pw, fx.Node) or _fname(pw) != "pow":
                continue
            if pw.args[0] is not x or pw.args[1] != 2:
                continue
            gs, xs = _meta_shape(gamma), _meta_shape(x)
            if gs is not None and xs is not None and (len(gs) != 1 or gs[0] != xs[-1]):
                continue
            return x, gamma, float(eps)
    return None


# ----------------------------------------------------------------------------------------
# passes
# ----------------------------------------------------------------------------------------
def _pass_rmsnorm(gm: fx.GraphModule) -> int:
    n = 0
    for node in list(gm.graph.nodes):
        m = _match_rmsnorm(node) if node.op == "call_function" else None
        if m is None:
            continue
        x, gamma, eps = m
        if _meta_dtype(x) not in (None, torch.bfloat16, torch.float16):
            continue
        with gm.graph.inserting_before(node):
            new = gm.graph.call_function(hb_rmsnorm, (x, gamma, eps))
        new.meta = dict(node.meta)
        node.replace_all_uses_with(new)
        n += 1
    if n:
        gm.graph.eliminate_dead_code()
    return n


def _pass_linear(gm: fx.GraphModule) -> int:
    n = 0
    for node in list(gm.graph.nodes):
        if not _is_linear(node):
            continue
        x = node.args[0]
        w = node.args[1]
        bias = node.args[2] if len(node.args) > 2 else node.kwargs.get("bias", None)
        if not isinstance(x, fx.Node) or not isinstance(w, fx.Node) or not _gemm_supported(x, w):
            continue
        act, tail = "none", node
        user = _single_user(node)
        if user is not None and _act_of(user) is not None and user.args[0] is node:
            act, tail = _act_of(user), user
        with gm.graph.inserting_before(tail):
            new = gm.graph.call_function(hb_linear, (x, w), {"bias": bias, "act": act})
        new.meta = dict(tail.meta)
        tail.replace_all_uses_with(new)
        n += 1
    if n:
        gm.graph.eliminate_dead_code()
    return n


def _pass_swiglu(gm: fx.GraphModule) -> int:
    """mul(hb_linear(x, wg, act=silu), hb_linear(x, wu)) -> hb_swiglu(x, wg, wu)."""
    n = 0
    for node in list(gm.graph.nodes):
        if _fname(node) != "mul" or len(node.args) != 2:
            continue
        for g, u in (node.args, node.args[::-1]):
            if not (isinstance(g, fx.Node) and isinstance(u, fx.Node)):
                continue
            if g.target is not hb_linear or u.target is not hb_linear or g is u:
                continue
            if g.kwargs.get("act") != "silu" or u.kwargs.get("act") != "none":
                continue
            if g.kwargs.get("bias") is not None or u.kwargs.get("bias") is not None:
                continue
            if g.args[0] is not u.args[0] or len(g.users) != 1 or len(u.users) != 1:
                continue
            if _meta_shape(g.args[1]) != _meta_shape(u.args[1]):
                continue
            with gm.graph.inserting_before(node):
                new = gm.graph.call_function(hb_swiglu, (g.args[0], g.args[1], u.args[1]))
            new.meta = dict(node.meta)
            node.replace_all_uses_with(new)
            n += 1
            break
    if n:
        gm.graph.eliminate_dead_code()
    return n


def _pass_residual(gm: fx.GraphModule) -> int:
    """add(r, gemm_leaf(...)) with the leaf used once -> residual=r inside the epilogue."""
    n = 0
    for node in list(gm.graph.nodes):
        # functional adds only: an in-place add that survived canonicalisation mutates storage the
        # caller can see, which a fresh output tensor would not reproduce
        if _fname(node) != "add" or len(node.args) != 2 or node.kwargs:
            continue
        for r, g in (node.args, node.args[::-1]):
            if not (isinstance(r, fx.Node) and isinstance(g, fx.Node)):
                continue
            if g.target not in GEMM_LEAVES or len(g.users) != 1 or g.kwargs.get("residual") is not None:
                continue
            if _meta_shape(r) is not None and _meta_shape(r) != _meta_shape(node):
                continue  # broadcasting add
            if _meta_dtype(r) is not None and _meta_dtype(g) is not None and _meta_dtype(r) != _meta_dtype(g):
                continue  # eager would promote (e.g. an fp32 residual stream): keep its add
            kwargs = dict(g.kwargs)
            kwargs["residual"] = r
            # the leaf must come after r in the graph: re-create it at the add's position
            with gm.graph.inserting_before(node):
                new = gm.graph.call_function(g.target, g.args, kwargs)
            new.meta = dict(node.meta)
            node.replace_all_uses_with(new)
            n += 1
            break
    if n:
        gm.graph.eliminate_dead_code()
    return n


def _pass_fold_rmsnorm(gm: fx.GraphModule) -> int:
    """hb_rmsnorm(x, gamma, eps) consumed only by GEMM leaves (as their activation input):
    one row statistic, gamma folded into each weight, rstd applied in the epilogue."""
    n = 0
    for node in list(gm.graph.nodes):
        if node.op != "call_function" or node.target is not hb_rmsnorm:
            continue
        users = list(node.users)
        if not users or not all(u.target in GEMM_LEAVES and u.args[0] is node and node not in u.args[1:]
                                and node not in u.kwargs.values() for u in users):
            continue
        x, gamma, eps = node.args
        with gm.graph.inserting_before(node):
            rstd = gm.graph.call_function(hb_rms_rowstat, (x, eps))
        for u in users:
            kwargs = dict(u.kwargs)
            kwargs["row_scale"] = rstd
            kwargs["gamma"] = gamma
            u.args = (x,) + tuple(u.args[1:])
            u.kwargs = kwargs
        n += 1
    if n:
        gm.graph.eliminate_dead_code()
    return n


def _uncast(n):
    """Look through ``.to(...)`` casts of a table (the kernel keeps cos / sin in fp32)."""
    while isinstance(n, fx.Node) and n.op == "call_method":
        dtype_only = _fname(n) == "float" or (_fname(n) == "to" and len(n.args) == 2 and not n.kwargs
                                              and isinstance(n.args[1], torch.dtype))
        if not dtype_only:  # a cast that also moves the table between devices stays in the graph
            break
        n = n.args[0]
    return n


def _match_rotate_half(cat: fx.Node):
    """cat([x1*cos - x2*sin, x2*cos + x1*sin], -1) with x1, x2 the halves of x's last axis.
    Returns (x, cos, sin, half) or None."""
    if _fname(cat) != "cat" or not cat.args or not isinstance(cat.args[0], (list, tuple)) or len(cat.args[0]) != 2:
        return None
    dim = cat.args[1] if len(cat.args) > 1 else cat.kwargs.get("dim", 0)
    lo, hi = cat.args[0]
    if dim != -1 or _fname(lo) != "sub" or _fname(hi) != "add":
        return None

    def prod(n):
        if _fname(n) != "mul" or len(n.args) != 2:
            return None
        return n.args

    a, b = prod(lo.args[0]), prod(lo.args[1])       # x1*cos, x2*sin
    c, d = prod(hi.args[0]), prod(hi.args[1])       # x2*cos, x1*sin
    if None in (a, b, c, d):
        return None
    x1, cos = a
    x2, sin = b
    if not (c[0] is x2 and c[1] is cos and d[0] is x1 and d[1] is sin):
        return None

    def half_of(n):
        if _fname(n) != "getitem" or len(n.args) != 2 or not isinstance(n.args[1], tuple) or len(n.args[1]) != 2:
            return None
        e, sl = n.args[1]
        if e is not Ellipsis or not isinstance(sl, slice) or sl.step not in (None, 1):
            return None
        return n.args[0], sl.start, sl.stop

    h1, h2 = half_of(x1), half_of(x2)
    if h1 is None or h2 is None or h1[0] is not h2[0]:
        return None
    x = h1[0]
    half = h1[2]
    if h1[1] not in (None, 0) or not isinstance(half, int) or h2[1] != half or h2[2] is not None:
        return None
    if len(x.users) != 2 or len(x1.users) != 2 or len(x2.users) != 2:
        return None
    return x, cos, sin, half


def _pass_rope(gm: fx.GraphModule) -> int:
    """rotate-half RoPE applied to transpose(view(hb_linear(...), B, S, H, D), 1, 2) moves into the
    projection's epilogue."""
    n = 0
    for cat in list(gm.graph.nodes):
        m = _match_rotate_half(cat) if cat.op == "call_function" else None
        if m is None:
            continue
        x, cos, sin, half = m
        if _fname(x) != "transpose" or tuple(x.args[1:]) not in ((1, 2), (2, 1)):
            continue
        view = x.args[0]
        if _fname(view) not in ("view", "reshape") or len(view.users) != 1:
            continue
        lin = view.args[0]
        if not isinstance(lin, fx.Node) or lin.target is not hb_linear or len(lin.users) != 1:
            continue
        if lin.kwargs.get("act", "none") != "none" or lin.kwargs.get("residual") is not None \
                or lin.kwargs.get("rope_cos") is not None:
            continue
        shp = view.args[1:] if len(view.args) > 2 else tuple(view.args[1])
        cs = _meta_shape(cos)
        if len(shp) != 4 or shp[3] != 2 * half or 2 * half not in (64, 128, 256) or cs is None \
                or tuple(cs) != (shp[1], half):
            continue
        kwargs = dict(lin.kwargs)
        kwargs.update(rope_cos=_uncast(cos), rope_sin=_uncast(sin), head_dim=2 * half)
        lin.kwargs = kwargs
        cat.replace_all_uses_with(x)
        n += 1
    if n:
        # the tables may be computed after the projection in program order: re-sort topologically
        from torch.fx.passes.tools_common import legalize_graph

        legalize_graph(gm)
        gm.graph.eliminate_dead_code()
    return n


def _pass_merge_siblings(gm: fx.GraphModule) -> int:
    """Projections of the same input (same RMSNorm fold, no bias / activation / residual) become
    one GEMM on stacked weights; rotary ones first so that they form the rotated column prefix."""
    groups: Dict[Tuple, List[fx.Node]] = {}
    for node in gm.graph.nodes:
        if node.op != "call_function" or node.target is not hb_linear:
            continue
        kw = node.kwargs
        if kw.get("bias") is not None or kw.get("residual") is not None or kw.get("act", "none") != "none":
            continue
        key = (node.args[0], kw.get("row_scale"), kw.get("gamma"))
        groups.setdefault(key, []).append(node)
    merged = 0
    for (x, row_scale, gamma), nodes in groups.items():
        if len(nodes) < 2:
            continue
        rot = [n for n in nodes if n.kwargs.get("rope_cos") is not None]
        if rot and any((n.kwargs["rope_cos"], n.kwargs["rope_sin"], n.kwargs["head_dim"]) !=
                       (rot[0].kwargs["rope_cos"], rot[0].kwargs["rope_sin"], rot[0].kwargs["head_dim"]) for n in rot):
            continue
        order = rot + [n for n in nodes if n not in rot]
        widths = []
        for n in order:
            ws = _meta_shape(n.args[1])
            widths.append(None if ws is None else ws[0])
        if any(w is None for w in widths):
            continue
        if len({_meta_dtype(n.args[1]) for n in order}) != 1:
            continue  # mixed weight dtypes cannot share one stacked operand
        if rot and any(w % rot[0].kwargs["head_dim"] for w in widths):
            continue  # the rotary epilogue works on whole head_dim-wide column groups
        order_in_graph = {n: i for i, n in enumerate(gm.graph.nodes)}
        last = max(nodes, key=lambda n: order_in_graph[n])
        kwargs = {"row_scale": row_scale, "gamma": gamma}
        if rot:
            kwargs.update(rope_cos=rot[0].kwargs["rope_cos"], rope_sin=rot[0].kwargs["rope_sin"],
                          head_dim=rot[0].kwargs["head_dim"], rope_cols=sum(widths[:len(rot)]))
        # created where the last sibling stood (all operands are defined there); users of earlier
        # siblings are moved behind it by the topological re-sort below
        with gm.graph.inserting_before(last):
            big = gm.graph.call_function(hb_linear_multi, (x, [n.args[1] for n in order]), kwargs)
            col = 0
            for n, w in zip(order, widths):
                part = gm.graph.call_function(operator.getitem, (big, (Ellipsis, slice(col, col + w))))
                part.meta = dict(n.meta)
                n.replace_all_uses_with(part)
                col += w
        merged += 1
    if merged:
        from torch.fx.passes.tools_common import legalize_graph

        legalize_graph(gm)
        gm.graph.eliminate_dead_code()
    return merged


def _pass_matmul(gm: fx.GraphModule) -> int:
    """matmul / bmm / mm / ``@`` of 16-bit tensors that is not an nn.Linear call (attention the
    rewrites refused, hand-written projections) -> ``hb_matmul``.  The reference has per-op leaves
    for these (backend.py:258-272, 523-536) whose rewriters are disabled (:1487-1491)."""
    done = 0
    for n in list(gm.graph.nodes):
        if n.op == "call_function" and (_fname(n) in ("matmul", "bmm", "mm") or n.target is operator.matmul):
            pass
        elif n.op == "call_method" and _fname(n) in ("matmul", "bmm", "mm"):
            pass
        else:
            continue
        if len(n.args) != 2 or n.kwargs:
            continue
        a, b = n.args
        sa, sb = _meta_shape(a), _meta_shape(b)
        if sa is None or sb is None or _meta_dtype(a) not in (torch.bfloat16, torch.float16) \
                or _meta_dtype(b) != _meta_dtype(a):
            continue
        if len(sa) < 2 or len(sb) < 2 or sa[-1] != sb[-2] or sa[-1] % 8 or sb[-1] % 8:
            continue
        if len(sb) > 2 and tuple(sa[:-2]) != tuple(sb[:-2]):
            continue  # broadcast batch dimensions stay in PyTorch
        with gm.graph.inserting_before(n):
            new = gm.graph.call_function(hb_matmul, (a, b))
        new.meta = dict(n.meta)
        n.replace_all_uses_with(new)
        gm.graph.erase_node(n)
        done += 1
    if done:
        gm.graph.eliminate_dead_code()
    return done


def _pass_einsum(gm: fx.GraphModule) -> int:
    """Two-operand ``torch.einsum`` of 16-bit tensors that reads as a batched product -> ``hb_einsum``."""
    done = 0
    for n in list(gm.graph.nodes):
        if n.op != "call_function" or _fname(n) != "einsum" or n.kwargs:
            continue
        args = list(n.args)
        if len(args) == 2 and isinstance(args[1], (list, tuple)):
            args = [args[0], *args[1]]
        if len(args) != 3 or not isinstance(args[0], str) or not all(isinstance(t, fx.Node) for t in args[1:]):
            continue
        a, b = args[1], args[2]
        sa, sb = _meta_shape(a), _meta_shape(b)
        if sa is None or sb is None or _meta_dtype(a) not in (torch.bfloat16, torch.float16) or _meta_dtype(b) != _meta_dtype(a):
            continue
        plan = einsum_plan(args[0], sa, sb)
        if plan is None or plan["K"] % 8 or plan["N"] % 8 or 0 in (plan["B"], plan["M"]):
            continue
        with gm.graph.inserting_before(n):
            new = gm.graph.call_function(hb_einsum, (args[0], a, b))
        new.meta = dict(n.meta)
        n.replace_all_uses_with(new)
        gm.graph.erase_node(n)
        done += 1
    return done


def _softmax_dim(n: fx.Node):
    """(input, dim, has_dtype) of a softmax node, or None."""
    name = _fname(n)
    if name != "softmax" or n.op not in ("call_function", "call_method"):
        return None
    args = list(n.args)
    x = args[0] if args else n.kwargs.get("input")
    dim = args[1] if len(args) > 1 else n.kwargs.get("dim")
    has_dtype = (len(args) > 2 and args[-1] is not None) or n.kwargs.get("dtype") is not None
    if n.op == "call_function" and len(args) > 3:  # F.softmax(input, dim, _stacklevel, dtype)
        has_dtype = args[3] is not None
    return x, dim, has_dtype


def _pass_softmax(gm: fx.GraphModule) -> int:
    """softmax over the last axis of a 16-bit tensor (what remains of attention the rewrites could
    not take, e.g. with an arbitrary mask) -> hb_softmax; a scalar multiply or divide that only
    feeds the softmax is folded into its scale.  The reference compiles such reductions with its
    generated softmax-like kernel (codegen.py:1246-1400)."""
    done = 0
    for n in list(gm.graph.nodes):
        m = _softmax_dim(n)
        if m is None:
            continue
        x, dim, has_dtype = m
        shp = _meta_shape(x)
        if has_dtype or not isinstance(x, fx.Node) or shp is None or not isinstance(dim, int):
            continue
        if dim not in (-1, len(shp) - 1) or _meta_dtype(x) not in (torch.bfloat16, torch.float16):
            continue
        if shp[-1] % 8 != 0 or shp[-1] > 16384:
            continue
        scale, src = 1.0, x
        if _fname(x) in ("mul", "truediv", "div") and len(x.users) == 1 and len(x.args) == 2:
            a, b = x.args
            if isinstance(a, fx.Node) and isinstance(b, (int, float)) and b != 0:
                scale, src = (float(b) if _fname(x) == "mul" else 1.0 / float(b)), a
            elif _fname(x) == "mul" and isinstance(b, fx.Node) and isinstance(a, (int, float)):
                scale, src = float(a), b
        if src is not x and (_meta_dtype(src) != _meta_dtype(x) or _meta_shape(src) != shp):
            scale, src = 1.0, x
        with gm.graph.inserting_before(n):
            new = gm.graph.call_function(hb_softmax, (src, scale))
        new.meta = dict(n.meta)
        n.replace_all_uses_with(new)
        gm.graph.erase_node(n)
        done += 1
    if done:
        gm.graph.eliminate_dead_code()
    return done


def _pass_rowwise(gm: fx.GraphModule) -> int:
    """What is left of the graph's pointwise chains and last-axis reductions -> ``hb_rowwise`` leaves:
    SupportPolicy decides membership, GraphPartitioner groups and prunes
    (TILELANG_FRONTEND_MIN_NODES / MIN_ELEMS / MIN_AI), lower_partition writes the program.  The
    reference sends the same partitions through its elementwise / reduction code generators
    (backend.py:1603-1700, codegen.py:1246-1498)."""
    from .partitioner import GraphPartitioner, lower_partition

    gp = GraphPartitioner(gm)
    done = 0
    for part in gp.partition():
        lp = lower_partition(part, gp.support)
        if lp is None:
            continue
        last = part.nodes[-1]
        with gm.graph.inserting_after(last):
            leaf = gm.graph.call_function(hb_rowwise, (list(lp.inputs), list(lp.rowvecs), list(lp.rowscalars),
                                                        lp.program, len(lp.outputs)))
        if len(lp.outputs) == 1:
            leaf.meta = dict(lp.outputs[0].meta)
            lp.outputs[0].replace_all_uses_with(leaf)
        else:
            prev = leaf
            for i, o in enumerate(lp.outputs):
                with gm.graph.inserting_after(prev):
                    item = gm.graph.call_function(operator.getitem, (leaf, i))
                item.meta = dict(o.meta)
                o.replace_all_uses_with(item)
                prev = item
        done += 1
    if done:
        from torch.fx.passes.tools_common import legalize_graph

        legalize_graph(gm)
        gm.graph.eliminate_dead_code()
    return done


def fuse_gemm_epilogues(gm: fx.GraphModule) -> int:
    """Run all passes; returns the number of GEMM leaves in the rewritten graph."""
    _pass_rmsnorm(gm)
    _pass_linear(gm)
    _pass_swiglu(gm)
    _pass_residual(gm)
    _pass_fold_rmsnorm(gm)
    _pass_rope(gm)
    _pass_merge_siblings(gm)
    _pass_matmul(gm)
    _pass_einsum(gm)
    _pass_softmax(gm)
    _pass_rowwise(gm)
    gm.graph.lint()
    gm.recompile()
    return sum(1 for n in gm.graph.nodes if n.op == "call_function" and n.target in GEMM_LEAVES)
