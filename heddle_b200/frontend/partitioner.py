"""Fused groups of pointwise / row-reduction nodes — counterpart of
Heddle/heddle/frontend/partitioner.py:317-400 (``GraphPartitioner.partition``), :605-690
(``_prune_candidates``) and of the code generators those partitions feed
(Heddle/heddle/frontend/codegen.py:1246-1498).

The reference enumerates connected subgraphs (DFS, at most 10 nodes, 2000 candidates), prunes them
and greedily selects by a score, then generates TileLang source per partition.  With one fixed
kernel per family that search is unnecessary: a maximal convex group of nodes the rowwise kernel
can compute *is* the best partition, so groups are grown in one topological sweep.  What is kept:
the capability policy decides membership (``SupportPolicy``), groups are pruned by the
reference's ``TILELANG_FRONTEND_MIN_NODES`` / ``MIN_ELEMS`` / ``MIN_AI`` switches with the
reference's defaults (partitioner.py:606-610), and a group is rejected when a hard boundary
consumes its output (:652-664).  GEMM and attention nodes are not grouped here: they are lowered
by the pattern passes of ``fusion.py`` / ``backend.py`` (the reference likewise keeps every GEMM
partition, :629-636, :675-679).

``lower_partition`` turns a group into the accumulator-machine program of ``hb_rowwise_program``.
"""
from __future__ import annotations

import logging
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Set, Tuple

import torch
import torch.fx as fx

from .support import SupportPolicy

log = logging.getLogger("heddle_b200")

_COMMUTATIVE = {"add", "mul", "max", "min"}
_REVERSED = {"sub": "rsub", "div": "rdiv"}
_MAX_TMP, _MAX_RED, _MAX_INPUTS, _MAX_ROWVEC, _MAX_ROWSCALAR, _MAX_OUTPUTS, _MAX_INST = 4, 4, 6, 4, 4, 2, 48


def _env_int(name: str, default: int) -> int:
    try:
        return int(os.environ.get(name, str(default)).strip())
    except ValueError:
        return default


def _env_float(name: str, default: float) -> float:
    try:
        return float(os.environ.get(name, str(default)).strip())
    except ValueError:
        return default


def _meta(n):
    if not isinstance(n, fx.Node):
        return None
    v = n.meta.get("example_value", n.meta.get("val", None))
    if v is not None and hasattr(v, "shape"):
        return v
    return n.meta.get("tensor_meta", None)


def _shape(n) -> Optional[Tuple[int, ...]]:
    m = _meta(n)
    return None if m is None else tuple(int(s) for s in m.shape)


def _dtype(n) -> Optional[torch.dtype]:
    m = _meta(n)
    return None if m is None else m.dtype


@dataclass
class Partition:
    """A convex group of nodes computed by one ``hb_rowwise_program`` launch."""

    nodes: List[fx.Node] = field(default_factory=list)  # topological order
    shape: Tuple[int, ...] = ()
    dtype: Optional[torch.dtype] = None
    inputs: List[fx.Node] = field(default_factory=list)
    outputs: List[fx.Node] = field(default_factory=list)

    def estimate_work_items(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def calculate_arithmetic_intensity(self) -> float:
        """Operations per byte moved to and from HBM (partitioner.py:243 in the reference)."""
        elems = self.estimate_work_items()
        bytes_moved = 0
        for t in self.inputs:
            shp, dt = _shape(t), _dtype(t)
            if shp is None or dt is None:
                continue
            cnt = 1
            for s in shp:
                cnt *= s
            bytes_moved += cnt * torch.empty((), dtype=dt).element_size()
        esize = 2 if self.dtype in (torch.bfloat16, torch.float16) else 4
        bytes_moved += len(self.outputs) * elems * esize
        return (len(self.nodes) * elems) / max(1, bytes_moved)


class GraphPartitioner:
    """Finds the pointwise / row-reduction groups of a graph (same constructor and ``partition``
    entry point as the reference's class, partitioner.py:317-343)."""

    def __init__(self, gm: fx.GraphModule, example_inputs: Optional[Sequence[torch.Tensor]] = None,
                 support_policy: Optional[SupportPolicy] = None):
        self.gm = gm
        self.example_inputs = list(example_inputs or [])
        self.support = support_policy or SupportPolicy.default()
        self.candidates: List[Partition] = []
        self.prune_stats: Dict[str, int] = {}

    # ---- membership ------------------------------------------------------------------------
    def _full_shape_of(self, n: fx.Node) -> Optional[Tuple[int, ...]]:
        """Shape of the [.., cols] tensor a node works on: its own for pointwise nodes, its input's
        for a reduction."""
        if self.support.family(n) == "reduction":
            src = n.args[0] if n.args else None
            return _shape(src)
        return _shape(n)

    def _eligible(self, n: fx.Node) -> bool:
        if not self.support.is_supported_inside_partition(n):
            return False
        shp, dt = self._full_shape_of(n), _dtype(n)
        if shp is None or len(shp) < 1 or shp[-1] == 0:
            return False
        if self.support.family(n) == "pointwise" and shp[-1] == 1 and len(shp) >= 2:
            # arithmetic on per-row values (e.g. rsqrt(var + eps)): lives in a group only next to the
            # reductions that feed it; the sweep checks that
            if dt not in (torch.bfloat16, torch.float16, torch.float32):
                return False
            for a in n.args:
                if isinstance(a, fx.Node):
                    if _shape(a) != shp:
                        return False
                elif not isinstance(a, (int, float)):
                    return False
            return not {k: v for k, v in n.kwargs.items() if v is not None and k != "approximate"}
        if shp[-1] % 8 != 0:
            return False
        if self.support.family(n) == "reduction":
            dim = n.args[1] if len(n.args) > 1 else n.kwargs.get("dim")
            keep = n.args[2] if len(n.args) > 2 else n.kwargs.get("keepdim", False)
            if isinstance(dim, (list, tuple)) and len(dim) == 1:
                dim = dim[0]
            if not isinstance(dim, int) or dim not in (-1, len(shp) - 1) or not keep:
                return False
            if n.kwargs.get("dtype") is not None:
                return False
            return _dtype(n.args[0]) in (torch.bfloat16, torch.float16)
        if dt not in (torch.bfloat16, torch.float16):
            return False
        if self.support.op_name(n) == "pow":
            exp = n.args[1] if len(n.args) > 1 else None
            if not isinstance(exp, (int, float)):
                return False  # tensor exponents stay in PyTorch
        for a in n.args:
            if isinstance(a, fx.Node):
                if _classify_operand(a, shp, dt) is None:
                    return False
            elif not isinstance(a, (int, float)):
                return False
        extra = {k: v for k, v in n.kwargs.items() if not (k == "approximate" or v is None)}
        if extra and not (list(extra) == ["alpha"] and extra["alpha"] == 1):
            return False
        return True

    def _is_row_value(self, n: fx.Node) -> bool:
        """A pointwise node on [..., 1] tensors."""
        shp = _shape(n)
        return self.support.family(n) == "pointwise" and shp is not None and len(shp) >= 2 and shp[-1] == 1

    def _eligible_compute_nodes(self) -> List[fx.Node]:
        return [n for n in self.gm.graph.nodes if n.op in ("call_function", "call_method") and self._eligible(n)]

    # ---- grouping --------------------------------------------------------------------------
    def partition(self, cost_model: str = "heuristic") -> List[Partition]:
        """Grow maximal convex groups in one topological sweep, then prune.  ``cost_model`` is accepted
        for signature parity (the reference ranks overlapping candidates with it; groups here do not
        overlap)."""
        self.support.debug_dump(self.gm)
        order = {n: i for i, n in enumerate(self.gm.graph.nodes)}
        group_of: Dict[fx.Node, int] = {}
        members: Dict[int, List[fx.Node]] = {}
        # dep[n]: ids of the groups n depends on (through any path, group members included).  A node
        # may join group g only if none of its other inputs depends on g: the group stays convex,
        # so it can be replaced by one node without creating a cycle.
        dep: Dict[fx.Node, Set[int]] = {}
        full_shape: Dict[int, Tuple[int, ...]] = {}
        for n in self.gm.graph.nodes:
            d: Set[int] = set()
            for a in n.all_input_nodes:
                d |= dep.get(a, set())
                if a in group_of:
                    d.add(group_of[a])
            dep[n] = d
            if n.op not in ("call_function", "call_method") or not self._eligible(n):
                continue
            shp = self._full_shape_of(n)
            row_value = self._is_row_value(n)
            target = None
            for a in n.all_input_nodes:
                g = group_of.get(a)
                if g is None:
                    continue
                gshape = full_shape[g]
                if row_value:
                    # joins the group whose reductions (or other per-row values) feed it
                    if not (self.support.family(a) == "reduction" or self._is_row_value(a)) or gshape[:-1] != shp[:-1]:
                        continue
                elif gshape != shp:
                    continue
                others = [b for b in n.all_input_nodes if group_of.get(b) != g]
                if any(g in dep.get(b, set()) for b in others):
                    continue
                target = g
                break
            if target is None:
                if row_value:
                    continue  # per-row arithmetic without a producing reduction in a group stays eager
                target = len(members)
                members[target] = []
                full_shape[target] = shp
            group_of[n] = target
            members[target].append(n)
            # sibling groups feeding n that are independent of the target group become part of it
            for b in n.all_input_nodes:
                g2 = group_of.get(b)
                if g2 is None or g2 == target or full_shape[g2] != full_shape[target]:
                    continue
                if any(g2 in dep[m] for m in members[target] if m is not n) or any(target in dep[m] for m in members[g2]):
                    continue
                if any(g2 in dep.get(c, set()) for c in n.all_input_nodes if group_of.get(c) != g2):
                    continue  # n also reaches g2 through a node outside of it
                for m in members[g2]:
                    group_of[m] = target
                members[target].extend(members.pop(g2))
                full_shape.pop(g2)
                for dset in dep.values():
                    if g2 in dset:
                        dset.discard(g2)
                        dset.add(target)

        self.candidates = []
        for g, nodes in members.items():
            nodes.sort(key=lambda m: order[m])
            first_full = next((m for m in nodes if not self._is_row_value(m) and self.support.family(m) != "reduction"), None)
            dt = _dtype(first_full) if first_full is not None else _dtype(nodes[0].args[0])
            p = Partition(nodes=nodes, shape=full_shape[g], dtype=dt)
            node_set = set(nodes)
            seen_in: List[fx.Node] = []
            for m in nodes:
                for a in m.all_input_nodes:
                    if a not in node_set and a not in seen_in:
                        seen_in.append(a)
            p.inputs = seen_in
            p.outputs = [m for m in nodes if any(u not in node_set for u in m.users)]
            self.candidates.append(p)
        self._prune_candidates()
        return list(self.candidates)

    def _prune_candidates(self) -> None:
        """Same switches and defaults as the reference (partitioner.py:605-690)."""
        min_nodes = _env_int("TILELANG_FRONTEND_MIN_NODES", 2)
        min_elems = _env_int("TILELANG_FRONTEND_MIN_ELEMS", 4096)
        min_ai = _env_float("TILELANG_FRONTEND_MIN_AI", 0.5)
        reason = {"too_small": 0, "bad_io": 0, "reduction_escapes": 0, "too_few_elems": 0, "low_ai": 0, "kept": 0}
        kept = []
        for p in self.candidates:
            if len(p.nodes) < min_nodes:
                reason["too_small"] += 1
                continue
            node_set = set(p.nodes)
            if any(self.support.is_hard_boundary(u) for o in p.outputs for u in o.users if u not in node_set):
                reason["bad_io"] += 1
                continue
            # a reduction result (or arithmetic on it) is only available inside the kernel
            if any(_shape(o) != p.shape for o in p.outputs):
                reason["reduction_escapes"] += 1
                continue
            if p.estimate_work_items() < min_elems:
                reason["too_few_elems"] += 1
                continue
            if p.calculate_arithmetic_intensity() < min_ai:
                reason["low_ai"] += 1
                continue
            reason["kept"] += 1
            kept.append(p)
        self.prune_stats = reason
        if os.environ.get("TILELANG_FRONTEND_DUMP_PRUNE_STATS", "0").strip() == "1":
            print(f"[Partitioner] prune stats: {reason}")
        log.info("rowwise partitions: %s", reason)
        self.candidates = kept


def _classify_operand(a: fx.Node, full: Tuple[int, ...], dtype) -> Optional[str]:
    """How a tensor operand of a group node is addressed: 'full', 'rowvec', 'rowscalar' or None."""
    shp, dt = _shape(a), _dtype(a)
    if shp is None or dt is None:
        return None
    if shp == full:
        return "full" if dt == dtype or dtype is None else None
    cols = full[-1]
    numel = 1
    for s in shp:
        numel *= s
    if len(shp) >= 1 and shp[-1] == cols and numel == cols and dt in (torch.bfloat16, torch.float16, torch.float32):
        return "rowvec" if dt == dtype else None
    if len(shp) == len(full) and shp[:-1] == full[:-1] and shp[-1] == 1:
        return "rowscalar"
    return None


# ------------------------------------------------------------------------------------------------
# partition -> program
# ------------------------------------------------------------------------------------------------
@dataclass
class LoweredPartition:
    program: Tuple[Tuple[str, Optional[str], int, float], ...]
    inputs: List[fx.Node]
    rowvecs: List[fx.Node]
    rowscalars: List[fx.Node]
    outputs: List[fx.Node]


def lower_partition(p: Partition, support: Optional[SupportPolicy] = None,
                    exact_intermediates: bool = False) -> Optional[LoweredPartition]:
    """Linearise a group into an accumulator-machine program, or None when it does not fit the
    machine (too many live values, operands or instructions).

    Every node becomes ``acc = op(acc, operand)``; a value that is still needed when acc is about to
    be overwritten is saved to a temporary first.  The chain runs in fp32 and is rounded once, when it
    is stored: that is the arithmetic of the path's oracle (the FX graph executed eagerly in fp32) and of
    the reference's reduction kernel, which keeps its intermediate and reduction results in fp32
    (codegen.py:1438-1440).  With ``exact_intermediates`` acc is instead rounded to the 16-bit type after
    every node whose eager result is a 16-bit tensor, which reproduces eager 16-bit PyTorch (and the
    reference's pointwise kernels, which compute in the buffers' own type, codegen.py:1466-1490) up to
    the last bits of the fp32 formulas."""
    support = support or SupportPolicy.default()
    node_set = set(p.nodes)
    full, dtype = p.shape, p.dtype
    inputs: List[fx.Node] = []
    rowvecs: List[fx.Node] = []
    rowscalars: List[fx.Node] = []
    prog: List[Tuple[str, Optional[str], int, float]] = []
    loc: Dict[fx.Node, Tuple[str, int]] = {}   # value -> addressable location (src kind, index)
    remaining: Dict[fx.Node, int] = {n: sum(1 for u in n.users if u in node_set) for n in p.nodes}
    tmp_owner: List[Optional[fx.Node]] = [None] * _MAX_TMP
    in_acc: Optional[fx.Node] = None
    red_slots = 0
    outputs: List[fx.Node] = []

    def external(a: fx.Node) -> Optional[Tuple[str, int]]:
        kind = _classify_operand(a, full, dtype)
        table, limit = {"full": (inputs, _MAX_INPUTS), "rowvec": (rowvecs, _MAX_ROWVEC),
                        "rowscalar": (rowscalars, _MAX_ROWSCALAR)}.get(kind, (None, 0))
        if table is None:
            return None
        if a not in table:
            if len(table) >= limit:
                return None
            table.append(a)
        return {"full": "input", "rowvec": "rowvec", "rowscalar": "rowscalar"}[kind], table.index(a)

    def address(a) -> Optional[Tuple[str, int, float]]:
        if isinstance(a, (int, float)):
            return "imm", 0, float(a)
        if a in node_set:
            l = loc.get(a)
            return None if l is None else (l[0], l[1], 0.0)
        e = external(a)
        return None if e is None else (e[0], e[1], 0.0)

    def spill_acc() -> bool:
        """Save the value in acc if something still needs it."""
        nonlocal in_acc
        if in_acc is None or remaining.get(in_acc, 0) <= 0 or in_acc in loc:
            return True
        for k in range(_MAX_TMP):
            if tmp_owner[k] is None or remaining.get(tmp_owner[k], 0) <= 0:
                if tmp_owner[k] is not None:
                    loc.pop(tmp_owner[k], None)
                tmp_owner[k] = in_acc
                loc[in_acc] = ("tmp", k)
                prog.append(("store_tmp", None, k, 0.0))
                return True
        return False

    def load(a) -> bool:
        nonlocal in_acc
        if isinstance(a, fx.Node) and a is in_acc:
            return True
        if not spill_acc():
            return False
        ad = address(a)
        if ad is None:
            return False
        prog.append(("load", ad[0], ad[1], ad[2]))
        in_acc = a if isinstance(a, fx.Node) else None
        return True

    def consume(a) -> None:
        if isinstance(a, fx.Node) and a in remaining:
            remaining[a] -= 1

    for n in p.nodes:
        fam, op = support.family(n), support.op_name(n)
        if op is None:
            return None
        if fam == "reduction":
            src = n.args[0]
            if red_slots >= _MAX_RED or not load(src):
                return None
            consume(src)
            prog.append((op, None, red_slots, 0.0))
            loc[n] = ("reduced", red_slots)
            red_slots += 1
            continue  # acc still holds src
        args = [a for a in n.args if isinstance(a, (fx.Node, int, float))]
        if op in ("add", "sub", "mul", "div", "max", "min", "pow"):
            if len(args) != 2:
                return None
            a, b = args
            if isinstance(a, (int, float)) and isinstance(b, (int, float)):
                return None
            # which operand goes through the accumulator?
            if isinstance(b, fx.Node) and b is in_acc and not (isinstance(a, fx.Node) and a is in_acc):
                if op in _COMMUTATIVE:
                    a, b = b, a
                elif op in _REVERSED and (isinstance(a, (int, float)) or address(a) is not None):
                    op, a, b = _REVERSED[op], b, a
            if isinstance(a, (int, float)):
                # scalar on the left: load the tensor operand instead where the op allows it
                if op in _COMMUTATIVE:
                    a, b = b, a
                elif op in _REVERSED:
                    op, a, b = _REVERSED[op], b, a
                else:
                    return None
            if isinstance(b, fx.Node) and b is a:
                # x op x: the operand must be addressable, so park the value first
                if not load(a):
                    return None
                if a in node_set and a not in loc:
                    remaining[a] = max(remaining.get(a, 0), 1)
                    if not spill_acc():
                        return None
            if not load(a):
                return None
            consume(a)
            if isinstance(b, fx.Node) and b is in_acc and b not in loc and not isinstance(b, (int, float)):
                return None
            ad = address(b)
            if ad is None:
                return None
            consume(b)
            # the value in acc is replaced: keep it if someone else still needs it
            if in_acc is not None and remaining.get(in_acc, 0) > 0 and in_acc not in loc:
                if not spill_acc():
                    return None
            prog.append((op, ad[0], ad[1], ad[2]))
        else:
            if len(args) < 1 or not isinstance(args[0], fx.Node):
                return None
            a = args[0]
            if not load(a):
                return None
            consume(a)
            if in_acc is not None and remaining.get(in_acc, 0) > 0 and in_acc not in loc:
                if not spill_acc():
                    return None
            prog.append((op, None, 0, 0.0))
        in_acc = n
        if exact_intermediates and _dtype(n) in (torch.bfloat16, torch.float16):
            prog.append(("round", None, 0, 0.0))
        if n in p.outputs:
            if len(outputs) >= _MAX_OUTPUTS:
                return None
            prog.append(("store_out", None, len(outputs), 0.0))
            outputs.append(n)
        if len(prog) > _MAX_INST:
            return None
    if not outputs or not inputs:
        return None
    return LoweredPartition(tuple(prog), inputs, rowvecs, rowscalars, outputs)
