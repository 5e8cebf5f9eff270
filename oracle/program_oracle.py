"""CPU restatement of the rowwise op-code program that ``hb_rowwise_program`` interprets.

TEST INFRASTRUCTURE ONLY: imported by ``tests/`` (and nothing in the product path).

The reference generates source text for pointwise chains and for row reductions and compiles it at
run time; this module restates the arithmetic of those generated kernels for one program:
  * the op table — Heddle/heddle/frontend/codegen.py:1577-1609 (``_map_op``: add, mul, sub, div,
    exp, sigmoid = 1/(1+exp(-x)), relu, silu = x * 1/(1+exp(-x)), tanh-GELU with 0.7978845608 and
    0.044715, tanh, log, log2, sqrt, rsqrt = 1/sqrt, neg, abs, pow);
  * row reductions — codegen.py:1246-1455: sum / mean / max over the last axis, results kept in
    fp32 (:1438-1440), the expression in front of a reduction recomputed per pass with earlier
    results substituted (:1406-1414), mean = sum / cols (:1433-1434).
Whole rows are evaluated at once here, which is the same function as the kernel's pass structure
(pass r recomputes the prefix in front of reduction r): a prefix never depends on its own reduction.
Pinned against eager PyTorch by ``tests/test_partitioner_cpu.py``: every lowered partition is run
through this interpreter and compared with the module it was captured from.
"""
from __future__ import annotations

from typing import Sequence, Tuple

import torch


def run_program(program: Sequence[Tuple[str, str, int, float]], inputs: Sequence[torch.Tensor] = (),
                rowvecs: Sequence[torch.Tensor] = (), rowscalars: Sequence[torch.Tensor] = (), n_outputs: int = 1):
    """Evaluate ``program`` (tuples ``(op, src, index, imm)``) in fp32 on CPU tensors.

    Returns ``n_outputs`` tensors in the dtype of ``inputs[0]`` (a tuple when more than one)."""
    x0 = inputs[0]
    dtype = x0.dtype
    shape = x0.shape
    cols = shape[-1]
    ins = [t.reshape(-1, cols).float() for t in inputs]
    rows = ins[0].shape[0]
    vecs = [t.reshape(1, cols).to(dtype).float() for t in rowvecs]
    scal = [t.reshape(rows, 1).float() for t in rowscalars]
    acc = None
    tmp = [None] * 4
    red = [None] * 4
    outs = [None] * n_outputs

    def operand(src, index, imm):
        if src == "input":
            return ins[index]
        if src == "rowvec":
            return vecs[index]
        if src == "rowscalar":
            return scal[index]
        if src == "tmp":
            return tmp[index]
        if src == "reduced":
            return red[index]
        return torch.full((1, 1), float(imm), dtype=torch.float32)

    for op, src, index, imm in program:
        if op in ("load", "add", "sub", "rsub", "mul", "div", "rdiv", "max", "min", "pow"):
            v = operand(src, index, imm)
            if op == "load":
                acc = v.expand(rows, cols).clone()
            elif op == "add":
                acc = acc + v
            elif op == "sub":
                acc = acc - v
            elif op == "rsub":
                acc = v - acc
            elif op == "mul":
                acc = acc * v
            elif op == "div":
                acc = acc / v
            elif op == "rdiv":
                acc = v / acc
            elif op == "max":
                acc = torch.maximum(acc, v.expand_as(acc))
            elif op == "min":
                acc = torch.minimum(acc, v.expand_as(acc))
            else:
                acc = torch.pow(acc, v)
        elif op == "neg":
            acc = -acc
        elif op == "abs":
            acc = acc.abs()
        elif op == "exp":
            acc = torch.exp(acc)
        elif op == "log":
            acc = torch.log(acc)
        elif op == "log2":
            acc = torch.log2(acc)
        elif op == "sqrt":
            acc = torch.sqrt(acc)
        elif op == "rsqrt":
            acc = 1.0 / torch.sqrt(acc)
        elif op == "recip":
            acc = 1.0 / acc
        elif op == "sigmoid":
            acc = 1.0 / (1.0 + torch.exp(-acc))
        elif op == "silu":
            acc = acc * (1.0 / (1.0 + torch.exp(-acc)))
        elif op == "relu":
            acc = torch.clamp_min(acc, 0.0)
        elif op == "gelu_tanh":
            acc = acc * 0.5 * (1.0 + torch.tanh(0.7978845608 * (acc + 0.044715 * acc * acc * acc)))
        elif op == "gelu_erf":
            acc = acc * 0.5 * (1.0 + torch.erf(acc * 0.7071067811865476))
        elif op == "tanh":
            acc = torch.tanh(acc)
        elif op == "round":
            acc = acc.to(dtype).float()
        elif op == "store_tmp":
            tmp[index] = acc
        elif op == "reduce_sum":
            red[index] = acc.sum(dim=-1, keepdim=True)
        elif op == "reduce_max":
            red[index] = acc.amax(dim=-1, keepdim=True)
        elif op == "reduce_mean":
            red[index] = acc.sum(dim=-1, keepdim=True) / cols
        elif op == "store_out":
            outs[index] = acc.to(dtype).reshape(shape)
        else:
            raise ValueError(f"unknown op {op!r}")
    return outs[0] if n_outputs == 1 else tuple(outs)
