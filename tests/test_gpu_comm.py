"""Peer-memory all-reduce kernels on symmetric buffers against a host-side sum (2+ GPUs)."""
import pytest
import torch

from dist_utils import run_distributed

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _worker(rank, world, use_multicast):
    import torch.distributed as dist
    from picotron_b200.comm.workspace import SymmetricWorkspace
    from picotron_b200.ops import _ext
    C = _ext.load()
    ws = SymmetricWorkspace(dist.group.WORLD, 64 << 20, num_blocks=16, use_multicast=use_multicast)
    out = {"multicast": ws.mc_ptr != 0}
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    # fp32 with fused averaging, odd length and an offset into the buffer
    n = 3 * 1000 * 1000 + 3
    x = ws.view(4096, (n,), torch.float32)
    mine = torch.randn(n, device="cuda", generator=g)
    x.copy_(mine)
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    want = torch.stack(gathered).sum(0) / world
    ws.all_reduce_(x, scale=1.0 / world)
    torch.cuda.synchronize()
    out["f32_err"] = float((x - want).abs().max())
    # bf16, several calls in a row on ring slots
    ws.configure_ring(4, 8 << 20)
    errs = []
    for it in range(6):
        t = ws.ring_alloc((1024, 2048), torch.bfloat16)
        mine = (torch.randn(1024, 2048, device="cuda", generator=g)).to(torch.bfloat16)
        t.copy_(mine)
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        want = torch.stack([t_.float() for t_ in gathered]).sum(0)
        ws.all_reduce_(t)
        torch.cuda.synchronize()
        errs.append(float((t.float() - want).abs().max()))
    out["bf16_err"] = max(errs)
    out["status"] = int(C.kernel_status())
    return out


@pytest.mark.parametrize("use_multicast", [False, True])
def test_symmetric_all_reduce(use_multicast):
    world = min(torch.cuda.device_count(), 4)
    res = run_distributed(_worker, world, use_multicast, backend="nccl")
    for r in res:
        assert r["status"] == 0
        assert r["f32_err"] < 1e-5, r
        assert r["bf16_err"] < 0.07, r     # one bf16 rounding of a sum of `world` N(0,1) values
