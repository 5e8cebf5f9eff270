"""Generate the golden fixtures of tests/golden/ by running the REFERENCE.

Run in a container that holds the reference checkout (it cannot travel to the GPU box):

    HEDDLE_REFERENCE=/path/to/reference/Heddle python tests/golden/make_golden.py

Each case is a module captured by the reference's own ``torch.compile`` backend
(``heddle.frontend.tilelang_backend``, Heddle/heddle/frontend/backend.py:1421) with
kernel generation switched off (TILELANG_FRONTEND_ENABLE_FLASHATTN_PATTERN=0,
TILELANG_FRONTEND_ENABLE_H2O_FUSE=0, TILELANG_FRONTEND_EXECUTE_PARTITIONS=0), so the
decomposed / canonicalised FX graph is executed eagerly in fp32 on the CPU — the
parity oracle the benchmark configuration names.  Inputs come from the seeded
generators in oracle/attention_oracle.py; only outputs (and an input checksum) are
stored.
"""
from __future__ import annotations

import math
import os
import sys
from pathlib import Path

os.environ["TILELANG_FRONTEND_ENABLE_FLASHATTN_PATTERN"] = "0"
os.environ["TILELANG_FRONTEND_ENABLE_H2O_FUSE"] = "0"
os.environ["TILELANG_FRONTEND_EXECUTE_PARTITIONS"] = "0"

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
if "HEDDLE_REFERENCE" not in os.environ:
    raise SystemExit("set HEDDLE_REFERENCE to the directory of the reference checkout that holds the heddle package")
sys.path.insert(0, os.environ["HEDDLE_REFERENCE"])

import torch  # noqa: E402

import heddle  # noqa: E402  (the reference)
from heddle.frontend import tilelang_backend  # noqa: E402

from oracle import attention_oracle as O  # noqa: E402

heddle.init()


def _first(x):
    return x[0] if isinstance(x, (tuple, list)) else x


def run_reference(module: torch.nn.Module, *inputs: torch.Tensor) -> torch.Tensor:
    torch._dynamo.reset()
    compiled = torch.compile(module, backend=tilelang_backend)
    with torch.no_grad():
        return _first(compiled(*inputs)).detach().clone()


class Attn(torch.nn.Module):
    """softmax(Q K^T / sqrt(D) [+ causal mask]) V on [B,H,S,D]."""

    def __init__(self, causal: bool):
        super().__init__()
        self.causal = causal

    def forward(self, q, k, v):
        s = torch.matmul(q, k.transpose(-2, -1)) / math.sqrt(q.shape[-1])
        if self.causal:
            Sq, Skv = q.shape[-2], k.shape[-2]
            s = s + torch.triu(torch.full((Sq, Skv), float("-inf")), diagonal=Skv - Sq + 1)
        return torch.matmul(torch.softmax(s, dim=-1), v)


class H2O(torch.nn.Module):
    """The H2O structure the reference fuses (Heddle/heddle/frontend/backend.py:1316-1419): causal attention whose
    probabilities also feed a sum over the query axis.  With the fusion switched off the reference executes
    this graph eagerly, which is the same arithmetic as the PyTorch fallback of its fused leaf (:186-201)."""

    def forward(self, q, k, v):
        Sq, Skv = q.shape[-2], k.shape[-2]
        s = torch.matmul(q, k.transpose(-2, -1)) / math.sqrt(q.shape[-1])
        s = s + torch.triu(torch.full((Sq, Skv), float("-inf")), diagonal=Skv - Sq + 1)
        p = torch.softmax(s, dim=-1)
        return torch.matmul(p, v), p.sum(dim=-2)


def run_reference_all(module: torch.nn.Module, *inputs: torch.Tensor):
    torch._dynamo.reset()
    compiled = torch.compile(module, backend=tilelang_backend)
    with torch.no_grad():
        return tuple(t.detach().clone() for t in compiled(*inputs))


class LinearAct(torch.nn.Module):
    def __init__(self, w, act):
        super().__init__()
        self.w = torch.nn.Parameter(w)
        self.act = act

    def forward(self, x):
        y = torch.nn.functional.linear(x, self.w)
        return {"none": lambda t: t, "silu": torch.nn.functional.silu, "relu": torch.relu,
                "gelu_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh"),
                "sigmoid": torch.sigmoid, "tanh": torch.tanh}[self.act](y)


class SwiGLU(torch.nn.Module):
    def __init__(self, wg, wu):
        super().__init__()
        self.wg, self.wu = torch.nn.Parameter(wg), torch.nn.Parameter(wu)

    def forward(self, x):
        return torch.nn.functional.silu(torch.nn.functional.linear(x, self.wg)) * torch.nn.functional.linear(x, self.wu)


def main() -> None:
    out = {}
    # config 1: B1 H4 S256 D64 fp32 non-causal, seed 0
    q, k, v = O.make_qkv(1, 4, 4, 256, 256, 64, seed=0)
    out["c1"] = dict(shape=(1, 4, 4, 256, 256, 64), seed=0, causal=False, in_dtype="float32",
                     checksum=float(q.double().sum() + k.double().sum() + v.double().sum()),
                     out=run_reference(Attn(False), q, k, v))
    # ragged causal prefill-with-past on bf16-rounded inputs (seed 1), D=128
    q, k, v = O.make_qkv(1, 2, 2, 192, 320, 128, seed=1, dtype=torch.bfloat16)
    out["causal_ragged"] = dict(shape=(1, 2, 2, 192, 320, 128), seed=1, causal=True, in_dtype="bfloat16",
                                checksum=float(q.double().sum() + k.double().sum() + v.double().sum()),
                                out=run_reference(Attn(True), q.float(), k.float(), v.float()))
    # causal self-attention, two 256-row blocks (seed 2)
    q, k, v = O.make_qkv(2, 2, 2, 512, 512, 128, seed=2, dtype=torch.bfloat16)
    out["causal_512"] = dict(shape=(2, 2, 2, 512, 512, 128), seed=2, causal=True, in_dtype="bfloat16",
                             checksum=float(q.double().sum() + k.double().sum() + v.double().sum()),
                             out=run_reference(Attn(True), q.float(), k.float(), v.float()).to(torch.bfloat16))
    # GEMM + epilogue graphs (seed 3): x [96, 128], w [192, 128] on bf16-rounded values
    g = torch.Generator().manual_seed(3)
    x = torch.randn(96, 128, generator=g).to(torch.bfloat16)
    w = (torch.randn(192, 128, generator=g) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(192, 128, generator=g) * 0.05).to(torch.bfloat16)
    gemm = dict(seed=3, checksum=float(x.double().sum() + w.double().sum() + w2.double().sum()))
    for act in ("none", "silu", "relu", "gelu_tanh", "sigmoid", "tanh"):
        gemm[act] = run_reference(LinearAct(w.float(), act), x.float())
    gemm["swiglu"] = run_reference(SwiGLU(w.float(), w2.float()), x.float())
    out["gemm"] = gemm
    # a small Llama-style layer (hidden 256, 2 heads of 128, inter 512), B2 S128, seed 4
    layer = O.LlamaLayer(hidden=256, heads=2, inter=512).init_weights(seed=4)
    for p in layer.parameters():
        p.data = p.data.to(torch.bfloat16).float()
    gx = torch.Generator().manual_seed(5)
    xs = torch.randn(2, 128, 256, generator=gx).to(torch.bfloat16).float()
    out["llama_small"] = dict(seed=4, x_seed=5, checksum=float(xs.double().sum()),
                              out=run_reference(layer, xs))
    # H2O: causal attention + column sums of the probabilities, keys longer than queries (seed 6)
    q, k, v = O.make_qkv(1, 2, 2, 160, 288, 64, seed=6, dtype=torch.bfloat16)
    h2o_out, h2o_score = run_reference_all(H2O(), q.float(), k.float(), v.float())
    out["h2o"] = dict(shape=(1, 2, 2, 160, 288, 64), seed=6, causal=True, in_dtype="bfloat16",
                      checksum=float(q.double().sum() + k.double().sum() + v.double().sum()),
                      out=h2o_out, score=h2o_score)
    torch.save(out, HERE / "reference_outputs.pt")
    for name, case in out.items():
        o = case.get("out")
        print(name, None if o is None else (tuple(o.shape), o.dtype))


if __name__ == "__main__":
    main()
