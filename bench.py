#!/usr/bin/env python
"""Benchmark of the attention-forward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one FlashAttention-forward pass over one synthetic batch of the headline
workload: BF16 causal multi-head attention, B=4, H=32, S=4096, D=128 (per GPU).  With
N > 1 (launched under torchrun, one rank per GPU) every rank runs the same-sized shard
of a global batch of 4*N — attention shards by batch x head with no collective — so the
scaling is weak and ``value`` is the whole-job TFLOP/s: total algorithmic FLOPs over
the slowest rank's time.

Printed by rank 0 as ONE JSON line:
  value      device-resident throughput (inputs already in HBM), CUDA events, max over ranks
  e2e        same metric through the public op with HOST buffers: pinned H2D of q,k,v and
             D2H of O and LSE inside the timed region, every step
  roofline   dominant kernel (fa_fwd) against the measured dense-bf16 tensor peak
  cpu_baseline  the CPU oracle (the reference's eager fp32 graph) on a bounded slice
  clocks     SM clock / throttle reasons sampled during the timed region

  secondary  (N = 1) short runs of the other configurations: GQA (config 3, whole), FP8 (config 4), the fused
             decoder layer (config 5), the plain projection GEMMs next to cuBLAS, H2O, the rowwise program
  strong     (N > 1) the FIXED config-2 and config-3 problems split over the ranks by batch x KV head

``--impl reference`` times the reference's own CPU path for the same metric/config: the attention
module captured by the reference's ``tilelang_backend`` (from ``baseline/_ref``) with kernel generation
off, i.e. its FX graph executed eagerly in fp32 on the host cores; when that package cannot be
imported, the oracle port of the same graph.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

WORKLOAD = dict(B=4, H=32, S=4096, D=128, causal=True)
METRIC = "attention_fwd_bf16_causal_tflops"
UNIT = "TFLOP/s"


def config_dict(world: int) -> dict:
    """The workload description both arms print (identical for ``--impl ours`` and ``--impl reference``)."""
    return {"workload": "bf16_causal_mha_B4_H32_S4096_D128", "global_batch": WORKLOAD["B"] * world,
            "seq_len": WORKLOAD["S"], "heads": WORKLOAD["H"], "head_dim": WORKLOAD["D"], "causal": True,
            "parallelism": f"dp{world}_batch_x_head_no_collective",
            "l2": "inputs+outputs (268 MB per step) exceed the 126 MB L2; no explicit flush"}


def algorithmic_flops(B, H, S, D, causal) -> float:
    # 4*B*H*Sq*Skv*D for both GEMMs; causal with Sq == Skv counts half (masked tiles are not work)
    return 4.0 * B * H * S * S * D * (0.5 if causal else 1.0)


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(burst=float(d["bf16_tflops"]), sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    hbm=float(d["hbm_gbs"]), source="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, source="fallback")


# ----------------------------------------------------------------------------------------
# clock sampling during the timed region (read-only NVML queries)
# ----------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x0000000000000004: "sw_power_cap",
        0x0000000000000008: "hw_slowdown",
        0x0000000000000020: "sw_thermal_slowdown",
        0x0000000000000040: "hw_thermal_slowdown",
        0x0000000000000080: "hw_power_brake_slowdown",
    }

    def __init__(self, device_index: int, period_s: float = 0.001):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        self.period = period_s
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            # honour CUDA_VISIBLE_DEVICES: map through the PCI bus id of the torch device
            bus = torch.cuda.get_device_properties(device_index).pci_bus_id if hasattr(
                torch.cuda.get_device_properties(device_index), "pci_bus_id") else None
            self._h = None
            if bus is not None:
                for i in range(pynvml.nvmlDeviceGetCount()):
                    h = pynvml.nvmlDeviceGetHandleByIndex(i)
                    info = pynvml.nvmlDeviceGetPciInfo(h)
                    if int(info.bus) == int(bus):
                        self._h = h
                        break
            if self._h is None:
                self._h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._h = None

    def _loop(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------
# CPU legs (the oracle is only ever the thing compared against or timed as the baseline)
# ----------------------------------------------------------------------------------------
def use_all_host_threads() -> int:
    """torchrun exports OMP_NUM_THREADS=1; the CPU legs use every core this process may run on."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def cpu_slice_tflops(heads: int = 8, reps: int = 31):
    """Reference eager fp32 attention on the host cores for a slice of the workload:
    one batch element x ``heads`` query heads at full sequence length, repeated until about ten
    seconds of CPU work are sampled (median reported)."""
    from oracle import attention_oracle as O

    use_all_host_threads()

    S, D = WORKLOAD["S"], WORKLOAD["D"]
    q, k, v = O.make_qkv(1, heads, heads, S, S, D, seed=0, dtype=torch.bfloat16)
    O.attention_eager(q, k, v, causal=True)  # warm-up
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        O.attention_eager(q, k, v, causal=True)
        times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    fl = algorithmic_flops(1, heads, S, D, True)
    return fl / t / 1e12, t, f"B=1 x {heads} heads x S={S} D={D} causal, eager fp32, median of {reps}"


def reference_gpu_kernel(B, H, S, D, causal):
    """The reference's own generated kernel on this GPU, when its package is present under
    baseline/_ref (a git-ignored pip --target install of the reference) and TileLang can JIT it:
    Heddle's `_build_fa_kernel` template (fp16, the only dtype it has; tile 128x128, 2 stages, 256
    threads = its heuristic's choice), timed with the reference's own protocol (10 warm-up, 50
    launches, CUDA events, median).  Any failure is reported, never fatal."""
    ref_dir = ROOT / "baseline" / "_ref"
    if not (ref_dir / "heddle").exists():
        return {"unavailable": "baseline/_ref/heddle not present"}
    try:
        os.environ.setdefault("TILELANG_DISABLE_CACHE", "1")
        sys.path.insert(0, str(ref_dir))
        import contextlib
        import io

        with contextlib.redirect_stdout(io.StringIO()):
            import heddle
            heddle.init()
            from heddle.frontend.backend import _build_fa_kernel
            kern = _build_fa_kernel(B, H, S, S, D, is_causal=causal, block_M=128, block_N=128, num_stages=2, threads=256)
        g = torch.Generator(device="cuda").manual_seed(7)
        q, k, v = (torch.randn(B, H, S, D, generator=g, device="cuda").to(torch.float16) for _ in range(3))
        for _ in range(10):
            kern(q, k, v)
        torch.cuda.synchronize()
        times = []
        for _ in range(50):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            kern(q, k, v)
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        ms = statistics.median(times)
        return {"value": algorithmic_flops(B, H, S, D, causal) / (ms * 1e-3) / 1e12, "unit": UNIT, "ms": ms,
                "dtype": "fp16", "what": "Heddle _build_fa_kernel through TileLang JIT (mma.sync path), median of 50"}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
    finally:
        if str(ref_dir) in sys.path:
            sys.path.remove(str(ref_dir))


class _EagerCausalAttention(torch.nn.Module):
    """The attention of the workload written out as user code writes it; what the reference captures."""

    def forward(self, q, k, v):
        S = q.shape[-2]
        s = torch.matmul(q, k.transpose(-2, -1)) / (q.shape[-1] ** 0.5)
        s = s + torch.triu(torch.full((S, S), float("-inf")), diagonal=1)
        return torch.matmul(torch.softmax(s, dim=-1), v)


def _reference_cpu_callable():
    """The reference's own CPU path: the module above compiled with the reference's torch.compile
    backend (Heddle/heddle/frontend/backend.py:1421) from baseline/_ref, attention-kernel generation and
    partition execution switched off, so that its decomposed FX graph runs eagerly in fp32.  Returns
    (callable, kind) or (None, reason)."""
    ref_dir = ROOT / "baseline" / "_ref"
    if not (ref_dir / "heddle").exists():
        return None, "baseline/_ref/heddle not present"
    import contextlib

    os.environ["TILELANG_FRONTEND_ENABLE_FLASHATTN_PATTERN"] = "0"
    os.environ["TILELANG_FRONTEND_ENABLE_H2O_FUSE"] = "0"
    os.environ["TILELANG_FRONTEND_EXECUTE_PARTITIONS"] = "0"
    os.environ.setdefault("TILELANG_DISABLE_CACHE", "1")
    try:
        sys.path.insert(0, str(ref_dir))
        with contextlib.redirect_stdout(sys.stderr):  # the reference prints its graphs; stdout carries one JSON line
            import heddle
            heddle.init()
            from heddle.frontend import tilelang_backend as reference_backend

        torch._dynamo.reset()
        compiled = torch.compile(_EagerCausalAttention(), backend=reference_backend)

        def call(q, k, v):
            with contextlib.redirect_stdout(sys.stderr), torch.no_grad():
                out = compiled(q, k, v)
            return out[0] if isinstance(out, (tuple, list)) else out

        return call, "reference"
    except Exception as e:  # noqa: BLE001
        return None, f"{type(e).__name__}: {str(e)[:160]}"
    finally:
        if str(ref_dir) in sys.path:
            sys.path.remove(str(ref_dir))


def run_reference(args):
    """Reference arm: the reference's CPU implementation of the path on all host threads, a bounded
    sample (a slice of the workload) per step.  Only rank 0 works."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    heads = 2
    use_all_host_threads()
    S, D = WORKLOAD["S"], WORKLOAD["D"]
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(1, heads, S, D, generator=g).to(torch.bfloat16).float() for _ in range(3))
    fn, kind = _reference_cpu_callable()
    note = None
    if fn is not None:
        try:
            fn(q, k, v)
        except Exception as e:  # noqa: BLE001
            fn, note = None, f"{type(e).__name__}: {str(e)[:160]}"
    else:
        note = kind
    if fn is None:
        from oracle import attention_oracle as O

        kind = "port"

        def fn(q, k, v):
            return O.attention_eager(q, k, v, causal=True)[0]

    steps = max(1, min(args.steps, 20))
    warm = max(1, min(args.warmup, 2))
    for _ in range(warm):
        fn(q, k, v)
    t0 = time.perf_counter()
    for _ in range(steps):
        fn(q, k, v)
    dt = (time.perf_counter() - t0) / steps
    val = algorithmic_flops(1, heads, S, D, True) / dt / 1e12
    sample = f"each step = B=1 x {heads} heads x S={S} D={D} causal slice of the workload (1/{4 * 32 // heads} of it)"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": config_dict(args.gpus),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind, "sample": sample,
                         "how": ("the attention module captured by the reference's tilelang_backend (baseline/_ref), kernel "
                                 "generation off: its FX graph run eagerly in fp32" if kind == "reference" else
                                 "oracle port of the reference's eager fp32 graph" + (f" (reference package unusable: {note})" if note else ""))},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------
# secondary configurations and the fixed-problem split
# ----------------------------------------------------------------------------------------
def run_secondary(peaks) -> dict:
    """Short device-resident runs (at most 20 launches each) of the configurations the headline does not
    cover, each with its time, throughput, fraction of the stated peak and a tolerance check of sampled
    heads against fp32 eager attention computed on the same GPU (TF32 off)."""
    from heddle_b200 import bench_configs

    out = {}
    plan = [("c3", True), ("c4", True), ("c5", True), ("gemm", False), ("gemm_plain", False), ("bmm", False),
            ("h2o", False), ("rowprog", False)]
    for name, check in plan:
        try:
            # every configuration is a burst measurement like the headline: a short pause lets the part
            # leave the power-capped state the previous configuration left it in (without it the runs at the
            # end of the list read 30-45 % low), and the clocks seen during the run are reported with it
            torch.cuda.synchronize()
            time.sleep(0.5)
            with ClockSampler(torch.cuda.current_device()) as cs:
                r = bench_configs.run_config(name, steps=10 if name in ("c3", "c5", "gemm_plain") else 20, warmup=3, check=check)
            r["clocks"] = cs.summary()
            if r.get("unit") == "TFLOP/s":
                if name == "c4" and r.get("fp8_gemm_reference_tflops"):
                    r["frac"] = r["value"] / r["fp8_gemm_reference_tflops"]
                    r["peak"] = "cuBLASLt e4m3 GEMM 8192^3 through torch._scaled_mm, measured in the same run"
                else:
                    r["frac"] = r["value"] / peaks["burst"]
                    r["peak"] = f"dense bf16 burst, of {peaks['source']}"
            elif r.get("unit") == "GB/s":
                r["frac"] = r["value"] / peaks["hbm"]
                r["peak"] = f"HBM copy bandwidth, of {peaks['source']}"
            out[name] = r
        except Exception as exc:  # noqa: BLE001 — a secondary run never takes the headline down
            out[name] = {"error": f"{type(exc).__name__}: {str(exc)[:200]}"}
        torch.cuda.empty_cache()
    return out


def strong_scaling(which: str, world: int, rank: int, dev, barrier, max_over_ranks, steps: int = 20) -> dict:
    """One FIXED problem split over the ranks with no collective: every rank builds the same tensors
    from the same seed on its own GPU and runs the kernel on its block of (batch, KV head) units.
      c2: B=4 H=32 S=4096 D=128 causal — the 128 (batch, head) units in contiguous blocks
          (``sharding.shard_batch_kvheads``);
      c3: B=8 Hq=64 Hkv=8 S=8192 D=128 causal GQA — by KV head: a rank owns Hkv/N KV heads with their
          query heads, all batches;
      c4: FP8 e4m3 non-causal B=4 H=32 S=8192 D=128 — split like c2;
      c5: the Llama-style layer, batch 8 x sequence 2048 — data-parallel over the batch (8 / N sequences per
          rank, the same weights on every rank).
    Aggregate = the whole problem's algorithmic FLOPs over the slowest rank's time."""
    from heddle_b200 import ops, sharding

    if which == "c5":
        return _strong_layer(world, rank, dev, barrier, max_over_ranks, steps=min(steps, 10))

    gen = torch.Generator(device=dev).manual_seed(2024)
    if which == "c2":
        B, Hq, Hkv, S, D = 4, 32, 32, 4096, 128
    elif which == "c4":
        B, Hq, Hkv, S, D = 4, 32, 32, 8192, 128
    else:
        B, Hq, Hkv, S, D = 8, 64, 8, 8192, 128
    causal = which != "c4"
    group = Hq // Hkv
    q = torch.randn(B, Hq, S, D, generator=gen, device=dev).to(torch.bfloat16)
    k = torch.randn(B, Hkv, S, D, generator=gen, device=dev).to(torch.bfloat16)
    v = torch.randn(B, Hkv, S, D, generator=gen, device=dev).to(torch.bfloat16)
    o = torch.empty_like(q)
    scales = None
    if which == "c4":  # per-tensor scales, e4m3 operands, bf16 output
        scales = [float(t.abs().max()) / 448.0 for t in (q, k, v)]
        q, k, v = ((t / s_).to(torch.float8_e4m3fn) for t, s_ in zip((q, k, v), scales))
    if which in ("c2", "c4"):
        runs = sharding.shard_batch_kvheads(B, Hkv, world, rank)  # (batch, kv_head_start, kv_head_stop)
        if runs and all(h0 == 0 and h1 == Hkv for (_, h0, h1) in runs):
            # whole batch elements: one launch on the [b0:b1] slice
            b0, b1 = runs[0][0], runs[-1][0] + 1
            views = [(q[b0:b1], k[b0:b1], v[b0:b1], o[b0:b1])]
        else:
            views = [(q[b:b + 1, h0 * group:h1 * group], k[b:b + 1, h0:h1], v[b:b + 1, h0:h1], o[b:b + 1, h0 * group:h1 * group])
                     for (b, h0, h1) in runs]
        units = sum(h1 - h0 for (_, h0, h1) in runs)
        split = "contiguous blocks of the 128 (batch, head) units"
    else:
        h0, h1 = sharding.shard_units(Hkv, world, rank)
        views = [(q[:, h0 * group:h1 * group], k[:, h0:h1], v[:, h0:h1], o[:, h0 * group:h1 * group])] if h1 > h0 else []
        units = B * (h1 - h0)
        split = "by KV head (a rank owns Hkv/N KV heads with their query heads, all batches)"

    def step():
        for (qq, kk, vv, oo) in views:
            if scales is None:
                ops.fa_fwd(qq, kk, vv, causal=causal, out=oo)
            else:
                ops.fa_fwd(qq, kk, vv, causal=False, scales=scales, out=oo)

    for _ in range(3):
        step()
    a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    a.record()
    for _ in range(steps):
        step()
    b_.record()
    barrier()
    ms = max_over_ranks(a.elapsed_time(b_)) / steps
    total = (2.0 if causal else 4.0) * B * Hq * S * S * D
    nqb = (S + 255) // 256
    pairs = units * group * ((nqb + 1) // 2 if causal else nqb)
    res = {"value": total / (ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms, "steps": steps, "scaling": "strong",
           "problem": f"B{B}_Hq{Hq}_Hkv{Hkv}_S{S}_D{D}_" + ("causal" if causal else "noncausal_e4m3"), "split": split,
           "kv_units_this_rank": units,
           "launches_per_step_this_rank": len(views), "work_items_this_rank": pairs,
           "note": f"{pairs} equal-cost work items for 148 persistent CTAs on this rank"
                   + (" (less than one wave: the split, not the kernel, bounds the time)" if pairs < 148 else "")}
    del q, k, v, o
    torch.cuda.empty_cache()
    return res


def _strong_layer(world: int, rank: int, dev, barrier, max_over_ranks, steps: int = 10) -> dict:
    """Configuration 5 data-parallel over the batch: every rank holds the same layer (same seed) and runs its
    8 / N sequences through ``torch.compile(backend=tilelang_backend)``; no collective (forward only)."""
    from heddle_b200 import bench_configs, sharding
    from heddle_b200.frontend import tilelang_backend

    B, S, Hd = 8, 2048, 4096
    layer = bench_configs.llama_layer()
    gen = torch.Generator(device=dev).manual_seed(2025)
    x = torch.randn(B, S, Hd, generator=gen, device=dev).to(torch.bfloat16)
    b0, b1 = sharding.shard_units(B, world, rank)
    mine = x[b0:b1]
    ms_local = 0.0
    if b1 > b0:
        torch._dynamo.reset()
        comp = torch.compile(layer, backend=tilelang_backend)
        with torch.no_grad():
            for _ in range(3):
                comp(mine)
    a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    a.record()
    if b1 > b0:
        with torch.no_grad():
            for _ in range(steps):
                comp(mine)
    b_.record()
    barrier()
    ms_local = a.elapsed_time(b_)
    ms = max_over_ranks(ms_local) / steps
    res = {"value": bench_configs.LLAMA_LAYER_FLOPS_B8_S2048 / (ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms, "steps": steps,
           "scaling": "strong", "problem": "llama_layer_h4096_heads32_inter11008_B8_S2048", "split": "data-parallel over the batch",
           "sequences_this_rank": b1 - b0}
    del layer, x
    torch.cuda.empty_cache()
    return res


# ----------------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------------
def run_ours(args):
    from heddle_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    distributed = world > 1
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if distributed:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if not distributed:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    B, H, S, D, causal = (WORKLOAD[k] for k in ("B", "H", "S", "D", "causal"))
    flops_rank = algorithmic_flops(B, H, S, D, causal)
    # this rank's shard of the global batch: same generator stream, distinct seed per rank
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    q = torch.randn(B, H, S, D, generator=gen, device=dev).to(torch.bfloat16)
    k = torch.randn(B, H, S, D, generator=gen, device=dev).to(torch.bfloat16)
    v = torch.randn(B, H, S, D, generator=gen, device=dev).to(torch.bfloat16)
    out = torch.empty_like(q)

    # ---- device-resident throughput -----------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        ops.fa_fwd(q, k, v, causal=causal, out=out)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(local_rank) as clocks:
        start.record()
        for _ in range(args.steps):
            ops.fa_fwd(q, k, v, causal=causal, out=out)
        stop.record()
        barrier()
    ms_local = start.elapsed_time(stop)
    ms_total = max_over_ranks(ms_local)
    ms_step = ms_total / args.steps
    value = flops_rank * world / (ms_step * 1e-3) / 1e12
    status = ops.status_word()

    # ---- per-launch duration of the dominant kernel (for the roofline) ---------------------
    n_ev = min(args.steps, 50)
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_ev)]
    for a, b in evs:
        a.record()
        ops.fa_fwd(q, k, v, causal=causal, out=out)
        b.record()
    torch.cuda.synchronize()
    per_launch = sorted(a.elapsed_time(b) for a, b in evs)
    launch_ms_bracketed = statistics.median(per_launch)
    launch_stats = {"median": launch_ms_bracketed, "min": per_launch[0], "p90": per_launch[int(0.9 * (len(per_launch) - 1))],
                    "launches": len(per_launch)}
    # Only this kernel launches inside the timed region, back to back on one stream, so its average
    # launch duration is the region's device time over its launches (events around every single
    # launch add the gap between an event and the next launch; that figure is kept beside it).
    launch_ms = ms_local / args.steps
    peaks = load_peaks()
    # Which measured peak applies: the burst figure for a kernel timed alone at full clocks, the
    # sustained one when the timed region ran under the power cap (reduced SM clock), as a long
    # back-to-back loop does on this 1 kW part.  Both fractions are reported.
    clk = clocks.summary()
    capped = "sw_power_cap" in clk["reasons"] or (clk["sm_mhz"] is not None and clk["sm_max_mhz"]
                                                  and clk["sm_mhz"] < 0.92 * clk["sm_max_mhz"])
    sustained_run = ms_total > 1000.0 or capped
    peak = peaks["sustained"] if sustained_run else peaks["burst"]
    achieved = flops_rank / (launch_ms * 1e-3) / 1e12
    traffic = None
    tfile = ROOT / "profiles" / "fa_fwd_dram_traffic.json"
    if tfile.exists():
        try:
            traffic = json.loads(tfile.read_text()).get("bytes_per_launch_full_workload")
        except Exception:
            traffic = None
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": traffic, "kernel": "fa_fwd_kernel<bf16,128>",
                "peak_kind": f"{'sustained (power-capped clocks during the timed region)' if sustained_run else 'burst'}"
                             f" dense bf16, of {peaks['source']}",
                "frac_of_burst_peak": achieved / peaks["burst"], "frac_of_sustained_peak": achieved / peaks["sustained"],
                "launch_ms": launch_ms, "launch_ms_events_around_each_launch": launch_stats,
                # time x median SM clock sampled during the region: lets burst, sustained and profiler runs be compared
                "cycles_per_launch": (launch_ms * 1e-3 * clk["sm_mhz"] * 1e6) if clk["sm_mhz"] else None}

    # ---- the same launch in a long back-to-back loop ----------------------------------------
    # A 1 kW part drops its SM clock under the power cap after a few hundred milliseconds of this
    # kernel; the default timed region (like the reference's 50-launch protocol) ends before that.
    # The long loop is reported next to it so that both regimes are on the line.
    n_long = 1000
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(local_rank) as clocks_long:
        s0.record()
        for _ in range(n_long):
            ops.fa_fwd(q, k, v, causal=causal, out=out)
        s1.record()
        barrier()
    ms_long = max_over_ranks(s0.elapsed_time(s1)) / n_long
    clk_long = clocks_long.summary()
    sustained = {"value": flops_rank * world / (ms_long * 1e-3) / 1e12, "unit": "TFLOP/s", "steps": n_long,
                 "ms_per_step": ms_long, "clocks": clk_long,
                 "frac_of_sustained_peak": flops_rank / (ms_long * 1e-3) / 1e12 / peaks["sustained"],
                 "cycles_per_launch": (ms_long * 1e-3 * clk_long["sm_mhz"] * 1e6) if clk_long["sm_mhz"] else None}

    # ---- end to end through the public op with host buffers --------------------------------
    # Every step moves that step's q, k, v from pinned host memory to the device and its O and
    # LSE back.  The batch is cut into per-batch-element chunks on three streams (H2D, compute,
    # D2H) with double-buffered device staging, so copies of one chunk overlap the kernel of
    # another; the result of every chunk is read back inside the timed region.
    hq, hk, hv = (torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t) for t in (q, k, v))
    ho = torch.empty(q.shape, dtype=q.dtype, pin_memory=True)
    hl = torch.empty((B, H, S), dtype=torch.float32, pin_memory=True)
    e2e = None
    if not args.kernel_only:
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        s_main = torch.cuda.current_stream(dev)
        nbuf = 2
        dq = [torch.empty((1, H, S, D), dtype=q.dtype, device=dev) for _ in range(nbuf)]
        dk = [torch.empty_like(dq[0]) for _ in range(nbuf)]
        dv = [torch.empty_like(dq[0]) for _ in range(nbuf)]
        do = [torch.empty_like(dq[0]) for _ in range(nbuf)]
        dl = [None] * nbuf
        ev_in = [torch.cuda.Event() for _ in range(nbuf)]
        ev_done = [torch.cuda.Event() for _ in range(nbuf)]
        ev_out = [torch.cuda.Event() for _ in range(nbuf)]
        counter = [0]

        def e2e_step():
            for b in range(B):
                i = counter[0] % nbuf
                counter[0] += 1
                with torch.cuda.stream(s_in):
                    s_in.wait_event(ev_done[i])      # staging buffers free again (kernel that read them is done)
                    dq[i].copy_(hq[b:b + 1], non_blocking=True)
                    dk[i].copy_(hk[b:b + 1], non_blocking=True)
                    dv[i].copy_(hv[b:b + 1], non_blocking=True)
                    ev_in[i].record(s_in)
                s_main.wait_event(ev_in[i])
                s_main.wait_event(ev_out[i])         # previous result of this slot has left the device
                _, dl[i] = ops.fa_fwd(dq[i], dk[i], dv[i], causal=causal, return_lse=True, out=do[i])
                ev_done[i].record(s_main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[i])
                    ho[b:b + 1].copy_(do[i], non_blocking=True)
                    hl[b:b + 1].copy_(dl[i], non_blocking=True)
                    ev_out[i].record(s_out)

        def e2e_sync():
            s_main.wait_stream(s_in)
            s_main.wait_stream(s_out)

        e2e_steps = max(3, min(args.steps, 20))
        for _ in range(2):
            e2e_step()
        e2e_sync()
        barrier()
        start.record()
        for _ in range(e2e_steps):
            e2e_step()
        e2e_sync()
        stop.record()
        barrier()
        e2e_ms = max_over_ranks(start.elapsed_time(stop)) / e2e_steps
        h2d = 3 * q.numel() * q.element_size()
        d2h = ho.numel() * ho.element_size() + hl.numel() * 4
        # bytes of the whole job per step (every rank moves its own shard), like `value`
        e2e = {"value": flops_rank * world / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d * world,
               "d2h_bytes_per_step": d2h * world, "bytes_per_rank": {"h2d": h2d, "d2h": d2h}, "ms_per_step": e2e_ms,
               "how": "ops.fa_fwd per batch element, pinned host buffers, H2D / kernel / D2H on three streams"}

    # ---- CPU baseline (rank 0, N = 1 only) -------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.kernel_only:
        v_cpu, t_cpu, sample = cpu_slice_tflops()
        cpu = {"value": v_cpu, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
               "sample": sample + f" ({t_cpu:.3f} s per slice)"}

    ref_gpu = None
    if rank == 0 and world == 1 and not args.kernel_only and not args.no_reference_gpu:
        ref_gpu = reference_gpu_kernel(B, H, S, D, causal)

    # ---- attention backward on the same shape (informative; not part of the headline metric) ----
    backward = None
    if rank == 0 and world == 1 and not args.kernel_only:
        try:
            _, lse = ops.fa_fwd(q, k, v, causal=causal, out=out, return_lse=True)
            d_o = torch.randn_like(q)
            for _ in range(3):
                ops.fa_bwd(q, k, v, out, d_o, lse, causal=causal)
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            ev0.record()
            for _ in range(20):
                ops.fa_bwd(q, k, v, out, d_o, lse, causal=causal)
            ev1.record()
            torch.cuda.synchronize()
            bwd_ms = ev0.elapsed_time(ev1) / 20
            prod = 2.0 * B * H * S * S * D * (0.5 if causal else 1.0)  # flops of one S x S x D product
            backward = {"ms": bwd_ms, "value": 5.0 * prod / (bwd_ms * 1e-3) / 1e12, "unit": UNIT,
                        "executed_tflops": 7.0 * prod / (bwd_ms * 1e-3) / 1e12,
                        "what": "hb_fa_bwd_preprocess + hb_fa_bwd_dkdv + hb_fa_bwd_dq, 20 backward passes; value counts the "
                                "usual five products, executed_tflops the seven the two kernels issue",
                        "device_status_word": ops.status_word()}
        except Exception as exc:  # informative only
            backward = {"error": str(exc)[:120]}

    # ---- strong scaling: the FIXED problems of configurations 2 and 3 split over the ranks ---------
    strong = None
    if distributed and not args.kernel_only:
        strong = {name: strong_scaling(name, world, rank, dev, barrier, max_over_ranks) for name in ("c2", "c3", "c4", "c5")}

    # ---- the other configurations, short runs (N = 1) ---------------------------------------------
    secondary = None
    if rank == 0 and world == 1 and not args.kernel_only and not args.no_secondary:
        secondary = run_secondary(peaks)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_dict(world),
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": args.steps * world,
            "clocks": clocks.summary(), "sustained": sustained, "device_status_word": status, "reference_gpu_kernel": ref_gpu,
            "backward": backward, "secondary": secondary, "strong": strong,
            "pct_of_nominal_dense_bf16_peak_2250": 100.0 * value / world / 2250.0,
        }
        print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-reference-gpu", action="store_true",
                    help="skip timing the reference's own generated kernel (needs baseline/_ref and TileLang)")
    ap.add_argument("--no-secondary", action="store_true", help="skip the short runs of the secondary configurations")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end and CPU-baseline legs (for profiler runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the heddle_b200 kernels have no CPU path")
    run_ours(args)


if __name__ == "__main__":
    main()
