"""Softmax decomposition and its inverse — counterpart of
Heddle/heddle/frontend/decomposition.py:8-198 (``decompose_ops`` / ``_decompose_softmax``).

The reference decomposes ``softmax(x, dim)`` into ``amax / sub / exp / sum / div`` before
partitioning so that its code generator sees elementary nodes (:167-198).  The kernels of this
package are fixed, so the attention and softmax matchers want the *composite* node instead:
``recompose_softmax`` folds a safe-softmax chain that user code (or an earlier decomposition)
wrote out by hand back into one ``softmax`` node; ``decompose_ops`` is kept with the reference's
signature and arithmetic for callers that want elementary nodes (the generic row-reduction
lowering accepts either form).  einsum is not decomposed (the reference leaves it to its ND-GEMM
code generator unless ``TILELANG_FRONTEND_DECOMPOSE_EINSUM=1``, :17-27).
"""
from __future__ import annotations

import operator
from typing import Optional, Tuple

import torch
import torch.fx as fx


def _fname(n) -> str:
    if not isinstance(n, fx.Node):
        return ""
    if n.op == "call_function":
        return getattr(n.target, "__name__", None) or str(n.target)
    if n.op == "call_method":
        return str(n.target)
    return ""


def _is_softmax_call(node: fx.Node) -> bool:
    if node.op == "call_function":
        return node.target in (torch.nn.functional.softmax, torch.softmax)
    return node.op == "call_method" and str(node.target) == "softmax"


def _softmax_args(node: fx.Node):
    x = node.args[0] if node.args else node.kwargs.get("input")
    dim = node.args[1] if len(node.args) > 1 else node.kwargs.get("dim", -1)
    dtype = node.kwargs.get("dtype")
    if node.op == "call_function" and node.target is torch.nn.functional.softmax and len(node.args) > 3:
        dtype = node.args[3]
    return x, dim, dtype


def decompose_ops(gm: fx.GraphModule) -> fx.GraphModule:
    """softmax(x, dim) -> exp(x - amax(x)) / sum(exp(x - amax(x))) (decomposition.py:167-198).
    Nodes with a ``dtype=`` argument keep their composite form (the cast is part of their meaning)."""
    for node in list(gm.graph.nodes):
        if not _is_softmax_call(node):
            continue
        x, dim, dtype = _softmax_args(node)
        if not isinstance(x, fx.Node) or dtype is not None or not isinstance(dim, int):
            continue
        with gm.graph.inserting_before(node):
            mx = gm.graph.call_function(torch.amax, (x,), {"dim": dim, "keepdim": True})
            centred = gm.graph.call_function(torch.sub, (x, mx))
            ex = gm.graph.call_function(torch.exp, (centred,))
            total = gm.graph.call_function(torch.sum, (ex,), {"dim": dim, "keepdim": True})
            out = gm.graph.call_function(torch.div, (ex, total))
        out.meta = dict(node.meta)
        node.replace_all_uses_with(out)
        gm.graph.erase_node(node)
    gm.graph.lint()
    gm.recompile()
    return gm


def _reduce_dim(node: fx.Node) -> Optional[Tuple[object, bool]]:
    """(dim, keepdim) of an amax / max / sum node over a single axis."""
    dim = node.args[1] if len(node.args) > 1 else node.kwargs.get("dim")
    keep = node.args[2] if len(node.args) > 2 else node.kwargs.get("keepdim", False)
    if isinstance(dim, (list, tuple)) and len(dim) == 1:
        dim = dim[0]
    if not isinstance(dim, int):
        return None
    return dim, bool(keep)


def recompose_softmax(gm: fx.GraphModule) -> int:
    """``div(e, sum(e, dim, keepdim=True))`` with ``e = exp(x - amax(x, dim, keepdim=True))`` becomes
    ``softmax(x, dim)`` when nothing else reads the intermediate nodes.  ``x.max(dim, keepdim=True)[0]``
    is accepted for the maximum as well.  Returns the number of chains folded."""
    folded = 0
    for div in list(gm.graph.nodes):
        if _fname(div) not in ("div", "truediv", "true_divide") or len(div.args) != 2:
            continue
        ex, total = div.args
        if not (isinstance(ex, fx.Node) and isinstance(total, fx.Node)):
            continue
        if _fname(ex) != "exp" or _fname(total) != "sum" or not total.args or total.args[0] is not ex:
            continue
        red = _reduce_dim(total)
        if red is None or not red[1]:
            continue
        dim = red[0]
        centred = ex.args[0] if ex.args else None
        if _fname(centred) != "sub" or len(centred.args) != 2:
            continue
        x, mx = centred.args
        if not (isinstance(x, fx.Node) and isinstance(mx, fx.Node)):
            continue
        if _fname(mx) == "getitem" and mx.args[1] == 0:  # values of x.max(dim, keepdim=True)
            mx_src = mx.args[0]
            if _fname(mx_src) != "max":
                continue
        else:
            mx_src = mx
            if _fname(mx_src) != "amax":
                continue
        if not mx_src.args or mx_src.args[0] is not x:
            continue
        mred = _reduce_dim(mx_src)
        if mred is None or not mred[1]:
            continue
        shp = None
        val = x.meta.get("example_value", x.meta.get("val", None))
        if val is not None and hasattr(val, "dim"):
            shp = val.dim()

        def norm(d):
            return d if (d >= 0 or shp is None) else d + shp

        if norm(mred[0]) != norm(dim):
            continue
        # the intermediates may only feed this chain
        if set(ex.users) != {total, div} or len(total.users) != 1 or len(centred.users) != 1 or len(mx.users) != 1:
            continue
        if mx_src is not mx and len(mx_src.users) != 1:
            continue
        with gm.graph.inserting_before(div):
            sm = gm.graph.call_function(torch.softmax, (x, dim))
        sm.meta = dict(div.meta)
        div.replace_all_uses_with(sm)
        folded += 1
    if folded:
        gm.graph.eliminate_dead_code()
        gm.graph.lint()
        gm.recompile()
    return folded
