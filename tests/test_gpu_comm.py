"""Peer-memory all-reduce kernels on symmetric buffers against a host-side sum (2+ GPUs)."""
import pytest
import torch

from dist_utils import run_distributed

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _worker(rank, world, mode):
    import torch.distributed as dist
    from picotron_b200.comm.workspace import SymmetricWorkspace
    from picotron_b200.ops import _ext
    C = _ext.load()
    # "push": peer stores into a staging area that is smaller than the fp32 message below (several pieces per call)
    ws = SymmetricWorkspace(dist.group.WORLD, 64 << 20, num_blocks=16, use_multicast=mode == "multimem",
                            staging_bytes=(3 << 20) if mode == "push" else 0)
    out = {"multicast": ws.mc_ptr != 0}
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    # fp32 with fused averaging, an offset into the buffer and (pull / multimem kernels) an odd length
    n = 3 * 1000 * 1000 + (0 if mode == "push" else 3)
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
    dist.barrier()
    ws.check_canaries()                                   # nothing wrote behind the flag or data region of this rank
    # the guard words do catch a stray write
    ws.storage[-1:].fill_(0)
    try:
        ws.check_canaries()
        out["canary_detects"] = False
    except RuntimeError:
        out["canary_detects"] = True
    return out


@pytest.mark.parametrize("mode", ["pull", "multimem", "push"])
def test_symmetric_all_reduce(mode):
    world = min(torch.cuda.device_count(), 4)
    res = run_distributed(_worker, world, mode, backend="nccl")
    for r in res:
        assert r["status"] == 0
        assert r["canary_detects"]
        assert r["f32_err"] < 1e-5, r
        assert r["bf16_err"] < 0.07, r     # one bf16 rounding of a sum of `world` N(0,1) values


def _ring_worker(rank, world, hq, hkv, d, s, causal):
    import math
    import torch.distributed as dist
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.ops import _ext, reference as ref
    from picotron_b200.parallel import context_parallel as cpar
    C = _ext.load()
    pgm.setup_process_group_manager(tp_size=1, cp_size=world, pp_size=1, dp_size=1)
    cpar.FUSED = True
    B = 2
    g = torch.Generator(device="cuda").manual_seed(7 + rank)
    mk = lambda *sh: torch.randn(*sh, device="cuda", generator=g).to(torch.bfloat16)
    q, k, v, do = mk(B, s, hq, d), mk(B, s, hkv, d), mk(B, s, hkv, d), mk(B, s, hq, d)
    scale = 1.0 / math.sqrt(d)

    def gather(t):
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous())
        return torch.cat(parts, dim=1)

    Q, K, V, DO = gather(q), gather(k), gather(v), gather(do)
    o_ref, lse_ref = ref.attention_fwd(Q, K, V, causal, scale)
    dq_ref, dk_ref, dv_ref = ref.attention_bwd(DO, Q, K, V, o_ref, lse_ref, causal, scale)
    sl = slice(rank * s, (rank + 1) * s)
    errs = {}
    for it in range(2):                                   # twice: slot alternation and epochs
        o, lse = cpar.ring_attention_forward_blocks(q, k, v, scale, causal)
        dq, dk, dv = cpar.ring_attention_backward_blocks(do, q, k, v, o, lse, scale, causal)
        torch.cuda.synchronize()
        rel = lambda a, b: float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))
        errs[f"o{it}"] = rel(o, o_ref[:, sl])
        errs[f"lse{it}"] = float((lse - lse_ref[:, :, sl]).abs().max())
        errs[f"dq{it}"] = rel(dq, dq_ref[:, sl])
        errs[f"dk{it}"] = rel(dk, dk_ref[:, sl])
        errs[f"dv{it}"] = rel(dv, dv_ref[:, sl])
    errs["status"] = int(C.kernel_status())
    return errs


@pytest.mark.parametrize("hq,hkv,d,s,causal", [(4, 2, 64, 256, True), (2, 2, 128, 192, True), (4, 1, 64, 128, False)])
def test_fused_ring_attention_reads_peer_kv_in_kernel(hq, hkv, d, s, causal):
    world = min(torch.cuda.device_count(), 4)
    res = run_distributed(_ring_worker, world, hq, hkv, d, s, causal, backend="nccl")
    for r in res:
        assert r["status"] == 0, r
        for k_, v_ in r.items():
            if k_.startswith("lse"):
                assert v_ < 5e-3, r
            elif k_ != "status":
                assert v_ < 2.5e-2, r


def _gemm_ar_worker(rank, world, M, N, K, dgrad):
    import torch.distributed as dist
    from picotron_b200.comm.workspace import SymmetricWorkspace
    from picotron_b200.ops import _ext
    C = _ext.load()
    ws = SymmetricWorkspace(dist.group.WORLD, 4 * M * N * 2 + (1 << 20), num_blocks=32)
    ws.configure_ring(4, M * N * 2)
    ws_push = SymmetricWorkspace(dist.group.WORLD, 2 * M * N * 2, num_blocks=32, use_multicast=False, staging_bytes=M * N * 2)
    ws_push.configure_ring(2, M * N * 2)
    g = torch.Generator(device="cuda").manual_seed(11 + rank)
    a = (torch.randn(M, K, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    b = (torch.randn((K, N) if dgrad else (N, K), device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    local = a.float() @ (b.float() if dgrad else b.float().t())
    want = local.clone()
    dist.all_reduce(want)
    errs, times = [], {}
    for it in range(3):                                   # consecutive calls: ring slots, epochs, flag reuse
        out = ws.ring_alloc((M, N), torch.bfloat16)
        ws.gemm_all_reduce(a, b, dgrad, out)
        torch.cuda.synchronize()
        errs.append(float((out.float() - want).norm() / want.norm()))
    dist.barrier()
    ws.check_canaries()

    def timed(fn, iters=10):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    def unfused():
        out = ws.ring_alloc((M, N), torch.bfloat16)
        C.gemm(a, b, False, dgrad, out, False)
        ws.all_reduce_(out)

    def nccl():
        y = C.gemm(a, b, False, dgrad, None, False)
        dist.all_reduce(y)

    def push():
        out = ws_push.ring_alloc((M, N), torch.bfloat16)
        C.gemm(a, b, False, dgrad, out, False)
        ws_push.all_reduce_(out)

    out = ws_push.ring_alloc((M, N), torch.bfloat16)
    C.gemm(a, b, False, dgrad, out, False)
    ws_push.all_reduce_(out)
    torch.cuda.synchronize()
    errs.append(float((out.float() - want).norm() / want.norm()))
    times["gemm_then_push_allreduce_ms"] = timed(push)
    times["push_allreduce_only_ms"] = timed(lambda: ws_push.all_reduce_(out))
    nccl_buf = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    times["nccl_allreduce_only_ms"] = timed(lambda: dist.all_reduce(nccl_buf))
    times["fused_ms"] = timed(lambda: ws.gemm_all_reduce(a, b, dgrad, ws.ring_alloc((M, N), torch.bfloat16)))
    times["gemm_then_symm_allreduce_ms"] = timed(unfused)
    times["gemm_then_nccl_ms"] = timed(nccl)
    times["gemm_only_ms"] = timed(lambda: C.gemm(a, b, False, dgrad, None, False))
    return {"err": max(errs), "status": int(C.kernel_status()), **times}


@pytest.mark.parametrize("world", [2, 4])               # 2: plain peer loads/stores; 4: the NVSwitch multimem reducer
@pytest.mark.parametrize("M,N,K,dgrad", [(512, 768, 256, False), (4096, 4096, 2048, False), (4096, 4096, 5504, True)])
def test_gemm_fused_with_all_reduce(M, N, K, dgrad, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    res = run_distributed(_gemm_ar_worker, world, M, N, K, dgrad, backend="nccl")
    print({k: round(v, 4) if isinstance(v, float) else v for k, v in res[0].items()})
    for r in res:
        assert r["status"] == 0, r
        assert r["err"] < 1e-2, r


def _graph_replay_worker(rank, world):
    """Collectives captured in a CUDA graph: the call counter lives in device memory, so replays, eager calls and replays
    again stay in step with the peers."""
    import torch.distributed as dist
    from picotron_b200.comm.workspace import SymmetricWorkspace
    from picotron_b200.ops import _ext
    C = _ext.load()
    ws = SymmetricWorkspace(dist.group.WORLD, 16 << 20, num_blocks=16)
    n = 1 << 20
    x = ws.view(0, (n,), torch.float32)
    src = torch.empty(n, device="cuda")
    ws.all_reduce_(x.zero_())                              # warm-up outside capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        x.copy_(src)
        ws.all_reduce_(x, scale=1.0 / world)
        ws.barrier()
    errs = []
    total = sum(range(world))

    def check(it):
        want = (it * world + total) / world                # ranks hold it + rank
        errs.append(float((x - want).abs().max()))

    for it in range(3):
        src.fill_(float(it + rank))
        graph.replay()
        torch.cuda.synchronize()
        check(it)
    x.fill_(float(10 + rank))                              # an eager call between replays
    ws.all_reduce_(x, scale=1.0 / world)
    torch.cuda.synchronize()
    check(10)
    src.fill_(float(20 + rank))
    graph.replay()
    torch.cuda.synchronize()
    check(20)
    return {"err": max(errs), "status": int(C.kernel_status()), "calls": ws.calls()}


def test_collectives_replay_from_a_cuda_graph():
    world = 2
    res = run_distributed(_graph_replay_worker, world, backend="nccl")
    for r in res:
        assert r["status"] == 0, r
        assert r["err"] < 1e-6, r
        assert r["calls"] == 1 + 4 * 2 + 1, r               # warm-up, 4 replays of (all-reduce + barrier), 1 eager call
