"""Canonical form of a captured FX graph — counterpart of
Heddle/heddle/frontend/normalization.py:9-50 (``canonicalize_ops``).

The rewrites of this package match functional nodes (``add``, ``mul``, ``softmax`` ...).  User
code reaches the same arithmetic through in-place operators (``x += y``, ``x.mul_(s)``) and
through ``detach`` / ``clone`` copies; this pass brings those spellings to the functional one so
that the matchers see one form, as the reference does before partitioning.

An in-place node is only made functional when that cannot change what the caller observes:
the mutated value must be produced inside the graph (not a placeholder, a parameter/buffer, or
a view of either), so nobody outside the graph holds the storage.  Later uses of the mutated
value are redirected to the functional result (``x.add_(y); f(x)`` becomes
``t = add(x, y); f(t)``); the reference only swaps the target of ``operator.iadd`` nodes and
leaves method-style in-place ops alone (normalization.py:19-33).
"""
from __future__ import annotations

import operator
from typing import Dict, Optional

import torch
import torch.fx as fx

# in-place operator.* targets -> functional twin
_INPLACE_FUNCTIONS = {
    operator.iadd: operator.add,
    operator.imul: operator.mul,
    operator.isub: operator.sub,
    operator.itruediv: operator.truediv,
}
# in-place tensor methods -> functional method
_INPLACE_METHODS = {
    "add_": "add", "mul_": "mul", "sub_": "sub", "div_": "div", "relu_": "relu", "sigmoid_": "sigmoid",
    "tanh_": "tanh", "exp_": "exp", "neg_": "neg", "clamp_": "clamp",
}
# nodes whose result aliases their first argument
_VIEW_METHODS = {"view", "reshape", "transpose", "permute", "squeeze", "unsqueeze", "expand", "flatten", "t",
                 "contiguous", "detach", "narrow", "select", "chunk", "split", "unbind", "__getitem__"}
_IDENTITY_METHODS = ("detach", "clone")


def _aliases_external_storage(node, memo: Dict[fx.Node, bool]) -> bool:
    """True if ``node``'s storage may be visible outside the graph (an input, a module attribute, or a
    view of one)."""
    if not isinstance(node, fx.Node):
        return False
    if node in memo:
        return memo[node]
    memo[node] = True  # cycles cannot occur in a DAG; conservative default while recursing
    if node.op in ("placeholder", "get_attr"):
        res = True
    elif node.op == "call_method" and str(node.target) in _VIEW_METHODS:
        res = _aliases_external_storage(node.args[0], memo) if node.args else True
    elif node.op == "call_function" and node.target is operator.getitem:
        res = _aliases_external_storage(node.args[0], memo)
    else:
        res = False
    memo[node] = res
    return res


def _redirect_later_uses(graph: fx.Graph, old: fx.Node, new: fx.Node) -> None:
    """Uses of ``old`` that come after ``new`` in program order read ``new`` instead."""
    seen_new = False
    for n in graph.nodes:
        if n is new:
            seen_new = True
            continue
        if seen_new and old in n.all_input_nodes:
            n.replace_input_with(old, new)


def canonicalize_ops(gm: fx.GraphModule) -> fx.GraphModule:
    """In-place arithmetic -> functional nodes where that is unobservable; ``detach`` / ``clone`` of
    graph-internal values removed.  Returns ``gm`` (rewritten in place), like the reference."""
    graph = gm.graph
    memo: Dict[fx.Node, bool] = {}
    inplace_left = False
    for node in list(graph.nodes):
        target: Optional[object] = None
        if node.op == "call_function" and node.target in _INPLACE_FUNCTIONS:
            target = _INPLACE_FUNCTIONS[node.target]
        elif node.op == "call_method" and str(node.target) in _INPLACE_METHODS:
            target = _INPLACE_METHODS[str(node.target)]
        if target is None:
            continue
        dst = node.args[0] if node.args else None
        if not isinstance(dst, fx.Node) or _aliases_external_storage(dst, memo):
            inplace_left = True  # the caller can see this mutation: keep it
            continue
        node.target = target
        _redirect_later_uses(graph, dst, node)

    if not inplace_left:
        # a clone only protects its source from later in-place writes; with none left it is an identity
        for node in list(graph.nodes):
            is_identity = (node.op == "call_method" and str(node.target) in _IDENTITY_METHODS) or (
                node.op == "call_function" and node.target in (torch.clone, torch.detach)) or (
                node.op == "call_function" and node.target in (torch.ops.aten.detach.default, torch.ops.aten.clone.default))
            if not is_identity or not node.args or not isinstance(node.args[0], fx.Node):
                continue
            if node.kwargs.get("memory_format") not in (None, torch.preserve_format):
                continue
            if any(u.op == "output" for u in node.users) and _aliases_external_storage(node.args[0], memo):
                continue  # returning a copy of an input must stay a copy
            node.replace_all_uses_with(node.args[0])
            graph.erase_node(node)

    graph.lint()
    gm.recompile()
    return gm
