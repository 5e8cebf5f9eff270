"""Failure detection on the GPU without a fault or a hang: a wait that nothing satisfies runs out
of its (short) limit, the CTA's roles leave their loops, the kernel ends normally and the host reads
a status code; the context stays usable."""
import pytest
import torch

from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_reports(built_lib):
    from heddle_b200 import ops

    status, (ok0, ns0, ok1, ns1) = ops.debug_wait_timeout(200)
    # kStatusWaitTimeout (0x100) | the role of the warp whose wait ran out (0x70)
    assert status == 0x170
    assert ok0 == 0 and ok1 == 0  # the timed-out warp and the warp that only saw the abort flag
    assert 200_000 <= ns0 <= 50_000_000  # gave up after the limit, long before the 2 s of the product kernels
    assert ns1 <= 60_000_000  # left through the flag, not through its own (1000 x longer) limit
    # the scratch status of the probe is not the library's status word, and the context still works
    assert ops.status_word() == 0
    q, k, v = O.make_qkv(1, 2, 2, 256, 256, 128, seed=1, dtype=torch.bfloat16)
    out = ops.fa_fwd(q.cuda(), k.cuda(), v.cuda(), causal=True)
    ref, _ = O.attention_eager(q, k, v, causal=True)
    assert (out.float().cpu() - ref).abs().max().item() <= 2e-2
    assert ops.status_word() == 0


def test_probe_rejects_bad_limits(built_lib):
    from heddle_b200 import ops

    with pytest.raises(RuntimeError, match="limit"):
        ops.debug_wait_timeout(0)
    with pytest.raises(RuntimeError, match="limit"):
        ops.debug_wait_timeout(10_000_000)
