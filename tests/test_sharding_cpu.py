"""Multi-GPU partitioning logic, exercised with world_size-2 gloo ranks on the CPU: every rank
computes its shard with the CPU oracle (stand-in for the kernel: the product has no CPU path),
the shards tile the full problem exactly, and a failing rank surfaces as an error, not a hang."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent

from heddle_b200 import sharding


def test_shard_units_tile_the_range():
    for total in (0, 1, 7, 128, 129):
        for world in (1, 2, 3, 8):
            blocks = [sharding.shard_units(total, world, r) for r in range(world)]
            assert blocks[0][0] == 0 and blocks[-1][1] == total
            assert all(blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in blocks]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_units(4, 2, 2)


def test_runs_are_views_and_gqa_groups_stay_together():
    runs = [sharding.shard_batch_kvheads(4, 8, 8, r) for r in range(8)]
    assert all(len(r) == 1 and r[0][2] - r[0][1] == 4 for r in runs)   # config 2 at 8 GPUs on KV heads
    runs = [sharding.shard_batch_kvheads(8, 8, 8, r) for r in range(8)]
    assert all(r == [(i, 0, 8)] for i, r in enumerate(runs))
    runs = sharding.shard_batch_kvheads(2, 3, 4, 1)                     # ragged: spans a batch boundary
    assert runs == [(0, 2, 3), (1, 0, 1)] or sum(h1 - h0 for _, h0, h1 in runs) in (1, 2)


def test_aggregate_uses_slowest_rank():
    assert sharding.aggregate_tflops([1e12, 1e12], [1000.0, 2000.0]) == pytest.approx(1.0)


def _worker(rank, world, port, fail_rank, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import attention_oracle as O
        B, Hq, Hkv, S, D = 2, 6, 3, 96, 64
        q, k, v = O.make_qkv(B, Hq, Hkv, S, S, D, seed=0)   # every rank derives the same full tensors
        g = Hq // Hkv
        out = torch.zeros(B, Hq, S, D)
        status = torch.zeros(1)
        try:
            if rank == fail_rank:
                raise RuntimeError("injected failure before launch")
            for b, h0, h1 in sharding.shard_batch_kvheads(B, Hkv, world, rank):
                o, _ = O.attention_eager(q[b:b + 1, h0 * g:h1 * g], k[b:b + 1, h0:h1], v[b:b + 1, h0:h1], causal=True)
                out[b, h0 * g:h1 * g] = o[0]
        except RuntimeError:
            status[0] = 1
        # host-side health exchange before anyone would wait on the data
        dist.all_reduce(status, op=dist.ReduceOp.MAX)
        if status.item() == 0:
            dist.all_reduce(out)   # only to check the result; the data path itself has no collective
            ref, _ = O.attention_eager(q, k, v, causal=True)
            ok = torch.allclose(out, ref, atol=2e-5)   # slices and the full problem may block their fp32 sums differently
        else:
            ok = False
        Path(out_dir, f"rank{rank}.txt").write_text(f"{int(status.item())} {int(ok)}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fail_rank", [-1, 1])
def test_two_ranks_tile_the_problem_or_report_failure(tmp_path, fail_rank):
    port = 29500 + (os.getpid() % 2000) + (7 if fail_rank >= 0 else 0)
    mp.spawn(_worker, args=(2, port, fail_rank, str(tmp_path)), nprocs=2, join=True)
    res = [Path(tmp_path, f"rank{r}.txt").read_text().split() for r in range(2)]
    if fail_rank < 0:
        assert res == [["0", "1"], ["0", "1"]]
    else:
        assert res == [["1", "0"], ["1", "0"]]   # every rank learnt of the failure, none hung


def _bwd_worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import attention_oracle as O
        B, Hq, Hkv, S, D = 2, 4, 2, 64, 32
        q, k, v = O.make_qkv(B, Hq, Hkv, S, S, D, seed=3)
        d_o = torch.randn(B, Hq, S, D, generator=torch.Generator().manual_seed(4))
        g = Hq // Hkv
        dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
        # the backward shards exactly like the forward: a (batch, kv head) run owns its query heads' dQ and its own
        # dK, dV (the sum over the group's query heads stays inside the run), so no rank needs another rank's data
        for b, h0, h1 in sharding.shard_batch_kvheads(B, Hkv, world, rank):
            rq, rk, rv, _ = O.attention_backward(q[b:b + 1, h0 * g:h1 * g], k[b:b + 1, h0:h1], v[b:b + 1, h0:h1],
                                                 d_o[b:b + 1, h0 * g:h1 * g], causal=True)
            dq[b, h0 * g:h1 * g], dk[b, h0:h1], dv[b, h0:h1] = rq[0], rk[0], rv[0]
        for t in (dq, dk, dv):
            dist.all_reduce(t)   # only to check the result; the data path itself has no collective
        fq, fk, fv, _ = O.attention_backward(q, k, v, d_o, causal=True)
        ok = all(torch.allclose(a, b_, atol=2e-5) for a, b_ in ((dq, fq), (dk, fk), (dv, fv)))
        Path(out_dir, f"bwd_rank{rank}.txt").write_text(str(int(ok)))
    finally:
        dist.destroy_process_group()


def test_two_ranks_tile_the_backward(tmp_path):
    port = 29500 + (os.getpid() % 2000) + 13
    mp.spawn(_bwd_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert [Path(tmp_path, f"bwd_rank{r}.txt").read_text() for r in range(2)] == ["1", "1"]
