"""Device-resident timings of the secondary configurations (one JSON line each):

    python -m heddle_b200.bench_configs --config NAME [--steps N] [--warmup W] [--check]

  c3    BF16 causal GQA, the whole of B=8 Hq=64 Hkv=8 S=8192 D=128 on one GPU (2.4 GB)
  c3_shard  one GPU's share of it at 8 GPUs (one KV head with its 8 query heads, all 8 batches)
  c4    FP8 e4m3 non-causal, B=4 H=32 S=8192 D=128, per-tensor scales amax/448
  c5    Llama-style decoder layer through torch.compile(backend=tilelang_backend):
        hidden 4096, 32 x 128 heads, SwiGLU 11008, B=8 S=2048, bf16
  gemm  the layer's gate/up projection as one SwiGLU GEMM: M=16384 N=2x11008 K=4096
  gemm_plain  the layer's plain projection shapes and 8192^3, each next to torch.matmul (cuBLAS) in the same run
  bmm   a batched product (64 x [2048,128] x [128,2048]) next to torch.bmm
  rowprog  hb_rowwise_program: a pointwise chain and a two-reduction program on 32768 x 4096 bf16 (GB/s)
  h2o   H2O score on the headline attention shape (B=4 H=32 S=4096 D=128, causal)
  bwd   attention backward (preprocess + dK/dV + dQ kernels) on the headline shape, causal; TFLOP/s in
        the usual convention of five matrix products (2.5 x the forward count); the seven products
        the two kernels really issue (each recomputes S and dP) are reported as executed_tflops
  softmax  row softmax of a 32768 x 4096 bf16 score matrix (HBM-bound, GB/s of algorithmic bytes)
  rowstat  RMSNorm row statistic fused with the residual add on the layer's activations
        (16384 x 4096 bf16): HBM-bound, reported in GB/s of algorithmic bytes

``bench.py`` carries the headline metric and calls ``run_config`` for its ``secondary`` object; this module
also gives every kernel a one-command workload for timing and profiling.  ``--check`` adds a comparison of
sampled heads with fp32 eager attention computed on the same GPU (TF32 off).  Inputs are synthetic N(0,1) / N(0,0.02).
"""
from __future__ import annotations

import argparse
import json

import torch


def _time(fn, steps: int, warmup: int) -> float:
    for _ in range(max(warmup, 3)):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


CONFIGS = ["c3", "c3_shard", "c4", "c5", "gemm", "gemm_plain", "bmm", "h2o", "bwd", "rowstat", "softmax", "rowprog"]

# MUFU roofline of an exponential-bound kernel: 16 ex2 per clock and SM (4 per sub-partition)
MUFU_PER_CLK_SM = 16
NUM_SMS = 148


def _fp32_attention_check(q, k, v, out, lse, causal, heads, tol, scale=None):
    """Sampled (batch, head) pairs against fp32 eager attention computed on the same GPU with TF32
    off: max |O - ref| and max |LSE - ref| and whether both are inside the stated tolerance."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        B, Hq, Sq, D = q.shape
        group = Hq // k.shape[1]
        Skv = k.shape[2]
        sm = scale if scale is not None else D ** -0.5
        worst_o = worst_l = 0.0
        for (b, h) in heads:
            qq, kk, vv = q[b, h].float(), k[b, h // group].float(), v[b, h // group].float()
            s = (qq @ kk.t()) * sm
            if causal:
                s = s.masked_fill(torch.ones(Sq, Skv, dtype=torch.bool, device=q.device).triu(1 + Skv - Sq), float("-inf"))
            ref_l = torch.logsumexp(s, -1)
            ref_o = torch.softmax(s, -1) @ vv
            worst_o = max(worst_o, float((out[b, h].float() - ref_o).abs().max()))
            if lse is not None:
                worst_l = max(worst_l, float((lse[b, h] - ref_l).abs().max()))
            del s, ref_o, ref_l
        return {"against": "fp32 eager attention on the same GPU (TF32 off)", "heads": [list(x) for x in heads],
                "max_abs_err": worst_o, "lse_max_err": worst_l if lse is not None else None, "tolerance": tol,
                "pass": bool(worst_o <= tol and (lse is None or worst_l <= 1e-3))}
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def llama_layer():
    """The Llama-style decoder layer of configuration 5 (hidden 4096, 32 heads, SwiGLU 11008), weights N(0, 0.02) from
    seed 0, bf16, on the current CUDA device."""
    import torch.nn.functional as F

    class Layer(torch.nn.Module):
        """Pre-norm Llama block (RMSNorm eps 1e-5, rotate-half RoPE theta 10000, causal attention, SwiGLU)."""

        def __init__(self, hidden=4096, heads=32, inter=11008):
            super().__init__()
            lin = lambda i, o: torch.nn.Linear(i, o, bias=False)
            self.h, self.nh, self.hd = hidden, heads, hidden // heads
            self.wq, self.wk, self.wv, self.wo = lin(hidden, hidden), lin(hidden, hidden), lin(hidden, hidden), lin(hidden, hidden)
            self.wg, self.wu, self.wd = lin(hidden, inter), lin(hidden, inter), lin(inter, hidden)
            self.g1, self.g2 = torch.nn.Parameter(torch.ones(hidden)), torch.nn.Parameter(torch.ones(hidden))

        def rms(self, x, g):
            return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * g

        def rope(self, x, cos, sin):
            d = self.hd // 2
            x1, x2 = x[..., :d], x[..., d:]
            return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)

        def forward(self, x):
            B, S, _ = x.shape
            h = self.rms(x, self.g1)
            q, k, v = (w(h).view(B, S, self.nh, self.hd).transpose(1, 2) for w in (self.wq, self.wk, self.wv))
            inv = 1.0 / (10000.0 ** (torch.arange(0, self.hd, 2, dtype=torch.float32, device=x.device) / self.hd))
            ang = torch.arange(S, dtype=torch.float32, device=x.device)[:, None] * inv[None, :]
            cos, sin = torch.cos(ang).to(x.dtype), torch.sin(ang).to(x.dtype)
            a = F.scaled_dot_product_attention(self.rope(q, cos, sin), self.rope(k, cos, sin), v, is_causal=True)
            x = x + self.wo(a.transpose(1, 2).reshape(B, S, self.h))
            h = self.rms(x, self.g2)
            return x + self.wd(F.silu(self.wg(h)) * self.wu(h))

    torch.manual_seed(0)
    layer = Layer()
    with torch.no_grad():
        for prm in layer.parameters():
            if prm.dim() == 2:
                prm.normal_(0.0, 0.02)
    return layer.to(torch.bfloat16).cuda()


LLAMA_LAYER_FLOPS_B8_S2048 = 6.907e12  # algorithmic FLOPs of the layer at batch 8, sequence 2048


def run_config(name: str, steps: int = 20, warmup: int = 3, check: bool = False) -> dict:
    """Time one secondary configuration; returns its JSON-able record."""
    import types

    args = types.SimpleNamespace(config=name, steps=steps, warmup=warmup)
    from . import ops

    gen = torch.Generator(device="cuda").manual_seed(0)
    rnd = lambda *shape: torch.randn(*shape, generator=gen, device="cuda")
    line = {"config": args.config, "steps": args.steps, "unit": "TFLOP/s", "data": "synthetic"}
    if args.config in ("c3", "c3_shard"):
        B, Hq, Hkv, S, D = (8, 64, 8, 8192, 128) if args.config == "c3" else (8, 8, 1, 8192, 128)
        q, k, v = rnd(B, Hq, S, D).bfloat16(), rnd(B, Hkv, S, D).bfloat16(), rnd(B, Hkv, S, D).bfloat16()
        out = torch.empty_like(q)
        ms = _time(lambda: ops.fa_fwd(q, k, v, causal=True, out=out), args.steps, args.warmup)
        flops = 2.0 * B * Hq * S * S * D
        line.update(workload=f"bf16_causal_gqa_B{B}_Hq{Hq}_Hkv{Hkv}_S{S}_D{D}" + ("" if args.config == "c3" else " (1/8 of config 3)"),
                    dtype="bf16")
        if check:
            o, lse = ops.fa_fwd(q, k, v, causal=True, return_lse=True)
            line.update(tolerance_check=_fp32_attention_check(q, k, v, o, lse, True, [(0, 0), (B - 1, Hq - 1), (B // 2, Hq // 2 + 1)], 2e-2))
            del o, lse
    elif args.config == "c4":
        B, H, S, D = 4, 32, 8192, 128
        q, k, v = rnd(B, H, S, D), rnd(B, H, S, D), rnd(B, H, S, D)
        sc = [float(t.abs().max()) / 448.0 for t in (q, k, v)]
        qq, kq, vq = ((t / s).to(torch.float8_e4m3fn) for t, s in zip((q, k, v), sc))
        del q, k, v
        ms = _time(lambda: ops.fa_fwd(qq, kq, vq, causal=False, scales=sc), args.steps, args.warmup)
        flops = 4.0 * B * H * S * S * D
        line.update(workload="fp8_e4m3_noncausal_B4_H32_S8192_D128", dtype="e4m3",
                    mufu_roofline_tflops=_mufu_roofline_tflops(4.0 * D), mufu_note="B*H*S*S exponentials at 16 ex2/clk/SM x 148 SMs at "
                    "1.9 GHz, expressed in attention TFLOP/s (4*D flops per exponential); a quarter of them run on the FMA pipe")
        if check:
            o = ops.fa_fwd(qq, kq, vq, causal=False, scales=sc)
            deq = [t.float() * s_ for t, s_ in zip((qq, kq, vq), sc)]
            line.update(tolerance_check=_fp32_attention_check(deq[0], deq[1], deq[2], o, None, False, [(0, 0), (B - 1, H - 1)], 6e-2))
            del o, deq
        # an FP8 tensor-core reference measured in the same run (no FP8 peak is on file): cuBLASLt
        # e4m3 x e4m3 -> bf16 at 8192^3 through torch._scaled_mm
        try:
            n = 8192
            a8 = torch.randn(n, n, device="cuda").to(torch.float8_e4m3fn)
            b8 = torch.randn(n, n, device="cuda").to(torch.float8_e4m3fn).t()
            one = torch.ones((), device="cuda")
            mm_ms = _time(lambda: torch._scaled_mm(a8, b8, scale_a=one, scale_b=one, out_dtype=torch.bfloat16), 20, 5)
            line.update(fp8_gemm_reference_tflops=2.0 * n ** 3 / mm_ms / 1e9)
        except Exception as exc:  # the reference is informative only
            line.update(fp8_gemm_reference_tflops=None, fp8_gemm_reference_error=str(exc)[:80])
    elif args.config == "h2o":
        B, H, S, D = 4, 32, 4096, 128
        q, k, v = rnd(B, H, S, D).bfloat16(), rnd(B, H, S, D).bfloat16(), rnd(B, H, S, D).bfloat16()
        _, lse = ops.fa_fwd(q, k, v, causal=True, return_lse=True)
        ms = _time(lambda: ops.h2o_score(q, k, lse, causal=True), args.steps, args.warmup)
        flops = 1.0 * B * H * S * S * D  # one causal Q K^T product
        line.update(workload="h2o_score_bf16_causal_B4_H32_S4096_D128", dtype="bf16",
                    mufu_roofline_tflops=_mufu_roofline_tflops(2.0 * D), mufu_note="one exponential per score (2*D flops each) at 16 ex2/clk/SM x "
                    "148 SMs at 1.9 GHz: the bound of this kernel next to the tensor peak; a quarter of them run on the FMA pipe")
    elif args.config == "bwd":
        B, H, S, D = 4, 32, 4096, 128
        q, k, v, g = (rnd(B, H, S, D).bfloat16() for _ in range(4))
        out, lse = ops.fa_fwd(q, k, v, causal=True, return_lse=True)
        ms = _time(lambda: ops.fa_bwd(q, k, v, out, g, lse, causal=True), args.steps, args.warmup)
        delta = ops.fa_bwd_preprocess(out, g)
        parts = {
            "preprocess_ms": _time(lambda: ops.fa_bwd_preprocess(out, g), args.steps, args.warmup),
            "dkdv_ms": _time(lambda: ops.fa_bwd_dkdv(q, k, v, g, lse, delta, causal=True), args.steps, args.warmup),
            "dq_ms": _time(lambda: ops.fa_bwd_dq(q, k, v, g, lse, delta, causal=True), args.steps, args.warmup),
        }
        flops = 5.0 * B * H * S * S * D  # five causal products of 2 S^2 D / 2 flops each
        line.update(workload="fa_bwd_bf16_causal_B4_H32_S4096_D128", dtype="bf16", **parts,
                    executed_tflops=7.0 * B * H * S * S * D / ms / 1e9)
    elif args.config == "softmax":
        R, Cn = 32768, 4096
        xs = [rnd(R, Cn).bfloat16() for _ in range(3)]  # 3 x 268 MB in rotation: no launch finds its input in L2
        it = [0]

        def run():
            i = it[0] = (it[0] + 1) % 3
            ops.row_softmax(xs[i], 0.125)

        ms = _time(run, args.steps, args.warmup)
        nbytes = 2.0 * R * Cn * 2
        torch_ms = _time(lambda: torch.softmax(xs[0] * 0.125, dim=-1), args.steps, args.warmup)
        line.update(workload="row_softmax_R32768_C4096", dtype="bf16", unit="GB/s", ms=ms, value=nbytes / ms / 1e6,
                    algorithmic_mb=nbytes / 1e6, torch_mul_softmax_ms=torch_ms, device_status_word=ops.status_word())
        return line
    elif args.config == "rowstat":
        M, N = 16384, 4096
        # several activation buffers in rotation so that no launch finds its input in L2 (126 MB)
        xs = [rnd(M, N).bfloat16() for _ in range(4)]
        rs = [rnd(M, N).bfloat16() for _ in range(4)]
        it = [0]

        def fused():
            i = it[0] = (it[0] + 1) % 4
            ops.rms_rowstat(xs[i], rs[i])

        def plain():
            i = it[0] = (it[0] + 1) % 4
            ops.rms_rowstat(xs[i])

        ms_plain = _time(plain, args.steps, args.warmup)
        ms = _time(fused, args.steps, args.warmup)
        bytes_fused, bytes_plain = 3.0 * M * N * 2 + 4.0 * M, 1.0 * M * N * 2 + 4.0 * M
        line.update(workload="rms_rowstat_residual_M16384_N4096", dtype="bf16", unit="GB/s", ms=ms, value=bytes_fused / ms / 1e6,
                    algorithmic_mb=bytes_fused / 1e6, plain_statistic_ms=ms_plain, plain_statistic_gbs=bytes_plain / ms_plain / 1e6,
                    device_status_word=ops.status_word())
        return line
    elif args.config == "gemm_plain":
        # the projection shapes of the decoder layer and the reference's 8192^3, each next to torch.matmul (cuBLAS)
        shapes = [(16384, 4096, 4096), (16384, 12288, 4096), (16384, 4096, 11008), (8192, 8192, 8192)]
        rows = []
        for (M, N, K) in shapes:
            a, w = rnd(M, K).bfloat16(), (rnd(N, K) * 0.02).bfloat16()
            ours = _time(lambda: ops.gemm_epilogue(a, w, "none"), args.steps, args.warmup)
            wt = w.t()
            lib = _time(lambda: torch.matmul(a, wt), args.steps, args.warmup)
            fl = 2.0 * M * N * K
            rows.append({"M": M, "N": N, "K": K, "ms": ours, "tflops": fl / ours / 1e9, "cublas_ms": lib,
                         "cublas_tflops": fl / lib / 1e9, "ratio": lib / ours})
            del a, w, wt
        line.update(workload="plain_gemm_projection_shapes", dtype="bf16", shapes=rows, ms=sum(r["ms"] for r in rows),
                    value=sum(2.0 * r["M"] * r["N"] * r["K"] for r in rows) / sum(r["ms"] for r in rows) / 1e9,
                    device_status_word=ops.status_word())
        return line
    elif args.config == "bmm":
        Bn, M, N, K = 64, 2048, 2048, 128   # per-head score-like products: [64, 2048, 128] x [64, 128, 2048]
        a, b = rnd(Bn, M, K).bfloat16(), rnd(Bn, K, N).bfloat16()
        ms = _time(lambda: ops.bmm(a, b), args.steps, args.warmup)
        lib = _time(lambda: torch.bmm(a, b), args.steps, args.warmup)
        flops = 2.0 * Bn * M * N * K
        line.update(workload=f"bmm_B{Bn}_M{M}_N{N}_K{K}", dtype="bf16", torch_bmm_ms=lib, torch_bmm_tflops=flops / lib / 1e9)
    elif args.config == "rowprog":
        # a pointwise chain and a row-reduction program on a [32768, 4096] bf16 matrix (HBM-bound, GB/s of
        # algorithmic bytes: every input read once, the output written once)
        R, Cn = 32768, 4096
        xs = [rnd(R, Cn).bfloat16() for _ in range(3)]
        ys = [rnd(R, Cn).bfloat16() for _ in range(3)]
        it = [0]
        chain = (("load", "input", 0, 0.0), ("silu", None, 0, 0.0), ("mul", "input", 1, 0.0), ("add", "imm", 0, 1.5),
                 ("store_out", None, 0, 0.0))
        norm = (("load", "input", 0, 0.0), ("reduce_mean", None, 0, 0.0), ("sub", "reduced", 0, 0.0), ("store_tmp", None, 0, 0.0),
                ("mul", "tmp", 0, 0.0), ("reduce_mean", None, 1, 0.0), ("load", "reduced", 1, 0.0), ("add", "imm", 0, 1e-5),
                ("rsqrt", None, 0, 0.0), ("mul", "tmp", 0, 0.0), ("store_out", None, 0, 0.0))

        def run_chain():
            i = it[0] = (it[0] + 1) % 3
            ops.rowwise_program(chain, [xs[i], ys[i]])

        def run_norm():
            i = it[0] = (it[0] + 1) % 3
            ops.rowwise_program(norm, [xs[i]])

        def torch_chain():
            i = it[0] = (it[0] + 1) % 3
            return torch.nn.functional.silu(xs[i]) * ys[i] + 1.5

        ms = _time(run_chain, args.steps, args.warmup)
        ms_norm = _time(run_norm, args.steps, args.warmup)
        ms_torch = _time(torch_chain, args.steps, args.warmup)
        b_chain, b_norm = 3.0 * R * Cn * 2, 2.0 * R * Cn * 2
        line.update(workload="rowwise_program_R32768_C4096", dtype="bf16", unit="GB/s", ms=ms, value=b_chain / ms / 1e6,
                    algorithmic_mb=b_chain / 1e6, what="silu(x) * y + 1.5 (fp32 chain, one rounding), two inputs, one output",
                    torch_eager_ms=ms_torch, layernorm_like={"ms": ms_norm, "gbs": b_norm / ms_norm / 1e6,
                                                             "what": "(x - mean) * rsqrt(var + eps): two reductions, three passes over L1/L2"},
                    device_status_word=ops.status_word())
        return line
    elif args.config == "gemm":
        M, N, K = 16384, 2 * 11008, 4096
        a, w = rnd(M, K).bfloat16(), (rnd(N, K) * 0.02).bfloat16()
        ms = _time(lambda: ops.gemm_epilogue(a, w, "swiglu"), args.steps, args.warmup)
        flops = 2.0 * M * N * K
        line.update(workload="swiglu_gemm_M16384_N22016_K4096", dtype="bf16")
    else:
        from .frontend import tilelang_backend

        layer = llama_layer()
        x = rnd(8, 2048, 4096).bfloat16()
        with torch.no_grad():
            eager_ms = _time(lambda: layer(x), args.steps, args.warmup)
            torch._dynamo.reset()
            comp = torch.compile(layer, backend=tilelang_backend)
            ms = _time(lambda: comp(x), args.steps, args.warmup)
        flops = LLAMA_LAYER_FLOPS_B8_S2048
        line.update(workload="llama_layer_h4096_heads32_inter11008_B8_S2048", dtype="bf16", eager_pytorch_ms=eager_ms,
                    eager_pytorch_tflops=flops / eager_ms / 1e9)
        if check:
            import copy

            prev = torch.backends.cuda.matmul.allow_tf32
            torch.backends.cuda.matmul.allow_tf32 = False
            try:
                with torch.no_grad():
                    got = comp(x)[:1].float()
                    ref = copy.deepcopy(layer).float()(x[:1].float())
                err = float((got - ref).abs().max())
                line.update(tolerance_check={"against": "the same layer in fp32 eager PyTorch on the same GPU (TF32 off), batch element 0",
                                             "max_abs_err": err, "tolerance": 2e-2 * max(1.0, float(ref.abs().max())),
                                             "pass": bool(err <= 2e-2 * max(1.0, float(ref.abs().max())))})
                del got, ref
            finally:
                torch.backends.cuda.matmul.allow_tf32 = prev
    line.update(ms=ms, value=flops / ms / 1e9, algorithmic_tflop=flops / 1e12, device_status_word=ops.status_word())
    if line.get("fp8_gemm_reference_tflops"):
        line.update(frac_of_fp8_gemm_reference=line["value"] / line["fp8_gemm_reference_tflops"])
    if line.get("mufu_roofline_tflops"):
        line.update(frac_of_mufu_roofline=line["value"] / line["mufu_roofline_tflops"])
    return line


def _mufu_roofline_tflops(flops_per_exponential: float, ghz: float = 1.9) -> float:
    """Throughput at which the MUFU alone bounds a kernel that needs one exponential per
    ``flops_per_exponential`` flops of the metric."""
    return MUFU_PER_CLK_SM * NUM_SMS * ghz * 1e9 * flops_per_exponential / 1e12


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", choices=CONFIGS, required=True)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--check", action="store_true", help="also compare sampled heads with fp32 eager attention on the GPU")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device: the heddle_b200 kernels have no CPU path")
    print(json.dumps(run_config(args.config, args.steps, args.warmup, args.check)), flush=True)


if __name__ == "__main__":
    main()
