"""What the native kernels can take — counterpart of Heddle/heddle/frontend/support.py:72-254
(``SupportPolicy.default`` / ``classify``).

The reference's policy answers "can TileLang code-generate this node"; here the kernels are
fixed, so the policy answers "which kernel family takes this node":

  gemm        linear / matmul / mm / bmm            -> hb_gemm_epilogue (fusion.py)
  attention   softmax-centred attention, SDPA op    -> hb_fa_fwd (backend.py)
  pointwise   the op table of the rowwise program   -> hb_rowwise_program
  reduction   sum / mean / amax over the last axis  -> hb_rowwise_program
  view        layout-only nodes                     -> boundary, stays in PyTorch

``classify`` keeps the reference's four-way answer (SUPPORTED / SOFT_BOUNDARY / HARD_BOUNDARY /
UNSUPPORTED) so that the partitioner reads the same way, and ``explain`` says why — the log the
fusion pass prints for nodes it leaves in eager PyTorch.  Like the reference it is conservative:
what is not listed is UNSUPPORTED.
"""
from __future__ import annotations

import logging
import operator
import os
from dataclasses import dataclass, field
from enum import Enum, auto
from typing import Any, Dict, Optional, Set, Tuple

import torch
import torch.fx as fx
import torch.nn.functional as F

log = logging.getLogger("heddle_b200")


class Capability(Enum):
    SUPPORTED = auto()
    SOFT_BOUNDARY = auto()
    HARD_BOUNDARY = auto()
    UNSUPPORTED = auto()


def _target_key(target: Any) -> str:
    name = getattr(target, "__name__", None)
    return str(name) if name else str(target)


# op name of the rowwise program for binary / unary pointwise targets
_BINARY: Dict[Any, str] = {
    operator.add: "add", torch.add: "add", "add": "add",
    operator.sub: "sub", torch.sub: "sub", "sub": "sub",
    operator.mul: "mul", torch.mul: "mul", "mul": "mul",
    operator.truediv: "div", torch.div: "div", torch.true_divide: "div", "div": "div", "true_divide": "div",
    torch.maximum: "max", "maximum": "max", torch.minimum: "min", "minimum": "min",
    torch.pow: "pow", operator.pow: "pow", "pow": "pow",
}
_UNARY: Dict[Any, str] = {
    operator.neg: "neg", torch.neg: "neg", "neg": "neg", torch.abs: "abs", "abs": "abs",
    torch.exp: "exp", "exp": "exp", torch.log: "log", "log": "log", torch.log2: "log2", "log2": "log2",
    torch.sqrt: "sqrt", "sqrt": "sqrt", torch.rsqrt: "rsqrt", "rsqrt": "rsqrt",
    torch.reciprocal: "recip", "reciprocal": "recip",
    torch.sigmoid: "sigmoid", F.sigmoid: "sigmoid", "sigmoid": "sigmoid",
    F.silu: "silu", "silu": "silu", torch.relu: "relu", F.relu: "relu", "relu": "relu",
    torch.tanh: "tanh", F.tanh: "tanh", "tanh": "tanh",
    F.gelu: "gelu",  # tanh or erf form, decided from the node's `approximate` argument
}
_REDUCTIONS: Dict[Any, str] = {
    torch.sum: "reduce_sum", "sum": "reduce_sum", torch.mean: "reduce_mean", "mean": "reduce_mean",
    torch.amax: "reduce_max", "amax": "reduce_max",
}
_GEMM_NAMES = ("linear", "matmul", "mm", "bmm")
_VIEW_METHODS = {"view", "reshape", "permute", "transpose", "contiguous", "flatten", "unsqueeze", "squeeze", "t"}
_CAST_METHODS = {"to", "type", "float", "half", "bfloat16"}


@dataclass
class SupportPolicy:
    """Capability policy used by GraphPartitioner (support.py:55-70 in the reference)."""

    binary: Dict[Any, str] = field(default_factory=dict)
    unary: Dict[Any, str] = field(default_factory=dict)
    reductions: Dict[Any, str] = field(default_factory=dict)
    hard_boundary_call_method_targets: Set[str] = field(default_factory=set)
    soft_boundary_call_method_targets: Set[str] = field(default_factory=set)
    view_call_method_targets: Set[str] = field(default_factory=set)

    @staticmethod
    def default() -> "SupportPolicy":
        return SupportPolicy(
            binary=dict(_BINARY), unary=dict(_UNARY), reductions=dict(_REDUCTIONS),
            # as in the reference (support.py:189-203): aliasing / materialising nodes end a partition,
            # chunk / split and dtype casts may sit at its edge but not inside
            hard_boundary_call_method_targets={"expand", "repeat", "detach", "clone"},
            soft_boundary_call_method_targets={"chunk", "split"} | _CAST_METHODS,
            view_call_method_targets=set(_VIEW_METHODS),
        )

    # ---- lookups --------------------------------------------------------------------------
    def _key(self, n: fx.Node):
        return n.target if n.op == "call_function" else str(n.target)

    def family(self, n: fx.Node) -> Optional[str]:
        """Kernel family of a node, or None."""
        if n.op not in ("call_function", "call_method"):
            return None
        key = self._key(n)
        if key in self.binary or key in self.unary:
            return "pointwise"
        if key in self.reductions:
            return "reduction"
        name = _target_key(n.target)
        if name in _GEMM_NAMES or (n.op == "call_function" and n.target is operator.matmul):
            return "gemm"
        if "scaled_dot_product_attention" in name or name == "softmax":
            return "attention"
        if n.op == "call_method" and name in self.view_call_method_targets:
            return "view"
        return None

    def op_name(self, n: fx.Node) -> Optional[str]:
        """Name of the rowwise-program op that computes a pointwise / reduction node."""
        key = self._key(n)
        if key in self.binary:
            return self.binary[key]
        if key in self.unary:
            name = self.unary[key]
            if name == "gelu":
                approx = n.kwargs.get("approximate", n.args[1] if len(n.args) > 1 else "none")
                return "gelu_tanh" if approx == "tanh" else "gelu_erf"
            return name
        return self.reductions.get(key)

    def classify(self, n: fx.Node) -> Capability:
        if n.op in ("get_attr", "call_module"):
            return Capability.HARD_BOUNDARY
        if n.op == "call_method":
            tgt = str(n.target)
            if tgt in self.hard_boundary_call_method_targets:
                return Capability.HARD_BOUNDARY
            if tgt in self.soft_boundary_call_method_targets:
                return Capability.SOFT_BOUNDARY
        if n.op in ("call_function", "call_method"):
            fam = self.family(n)
            if fam in ("pointwise", "reduction", "gemm", "attention"):
                return Capability.SUPPORTED
            if fam == "view":
                return Capability.SOFT_BOUNDARY
            name = _target_key(n.target)
            if any(s in name for s in ("clone", "detach", "expand", "repeat")):
                return Capability.HARD_BOUNDARY
        return Capability.UNSUPPORTED

    def explain(self, n: fx.Node) -> str:
        c = self.classify(n)
        fam = self.family(n)
        if c == Capability.SUPPORTED:
            return f"{fam}: native kernel family"
        if c == Capability.SOFT_BOUNDARY:
            return "layout / dtype node: allowed at the edge of a fused group, not inside"
        if c == Capability.HARD_BOUNDARY:
            return "aliasing, materialising or module-attribute node: ends a fused group"
        return f"{_target_key(n.target) if n.op != 'placeholder' else n.op}: no native kernel takes it, stays in PyTorch"

    def is_supported_inside_partition(self, n: fx.Node) -> bool:
        return self.classify(n) == Capability.SUPPORTED and self.family(n) in ("pointwise", "reduction")

    def is_any_boundary(self, n: fx.Node) -> bool:
        return self.classify(n) in (Capability.SOFT_BOUNDARY, Capability.HARD_BOUNDARY)

    def is_hard_boundary(self, n: fx.Node) -> bool:
        return self.classify(n) == Capability.HARD_BOUNDARY

    def debug_dump(self, gm: fx.GraphModule, head: int = 50) -> None:
        """TILELANG_FRONTEND_DUMP_CAPABILITY=1 prints the classification of the first nodes
        (support.py:242-254)."""
        if os.environ.get("TILELANG_FRONTEND_DUMP_CAPABILITY", "0").strip() != "1":
            return
        shown = 0
        for n in gm.graph.nodes:
            if n.op in ("call_function", "call_method", "call_module", "get_attr"):
                print(f"[SupportPolicy] {n.name}: {n.op} {_target_key(n.target)} => {self.classify(n).name} ({self.explain(n)})")
                shown += 1
                if shown >= head:
                    break
