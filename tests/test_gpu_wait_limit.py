"""A bounded device wait that runs out: the kernel returns, the status word names the site, the context stays usable.

The cross-rank barrier kernel is launched for a two-rank layout on ONE GPU in which the "peer" is just a second local flag
buffer that nothing ever writes. No other rank, no fault: the wait simply reaches its (shortened) limit. This is the
device half of failure detection; the host half (ranks that leave, watchdog, truncated checkpoints) is tested on CPU.
"""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_barrier_wait_runs_out_and_the_next_launch_works():
    from picotron_b200.ops import _ext
    C = _ext.load()
    torch.cuda.set_device(0)
    C.kernel_status()                                    # clear anything an earlier test left behind
    mine = torch.zeros(131072 // 4, dtype=torch.int32, device="cuda")       # flag region of "rank 0"
    silent_peer = torch.zeros_like(mine)                                    # flag region of a rank that never arrives
    default = C.get_wait_limit_ns()
    assert default >= 1_000_000_000
    try:
        C.set_wait_limit_ns(1_000_000)                   # 1 ms
        t0 = time.perf_counter()
        C.symm_barrier([mine.data_ptr(), silent_peer.data_ptr()], 0, 2)
        torch.cuda.synchronize()
        waited = time.perf_counter() - t0
        status = C.kernel_status()
        assert status != 0, "the wait should have run out"
        assert status >> 24 == 5 and (status >> 16) & 0xFF == 1, hex(status)   # all-reduce/barrier family, start barrier
        assert waited < 1.0, f"a 1 ms limit took {waited:.3f} s"
        assert C.kernel_status() == 0                    # fetch-and-clear
        # the call counter advanced although the wait failed, and the rank told its peer that it had arrived
        assert int(mine[8192 // 4].item()) == 1 and int(silent_peer[0].item()) == 1
        # a later launch on the same buffers works: as a single-rank group the barrier has nobody to wait for
        C.symm_barrier([mine.data_ptr()], 0, 1)
        # and so does real work on the device
        a = torch.randn(256, 256, device="cuda").to(torch.bfloat16)
        out = C.gemm(a, a, False, False, None, False)
        torch.cuda.synchronize()
        assert C.kernel_status() == 0
        assert int(mine[8192 // 4].item()) == 2
        torch.testing.assert_close(out.float(), a.float() @ a.float().t(), rtol=2e-2, atol=0.5)
    finally:
        C.set_wait_limit_ns(0)
    assert C.get_wait_limit_ns() == default
