"""Collective timings on N GPUs of one node: peer-memory all-reduce kernels (plain P2P and NVSwitch multimem) vs NCCL,
and the fused GEMM+all-reduce kernel vs GEMM followed by an all-reduce.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 bench_comm.py

Every number is device time (CUDA events), max over ranks, mean of 20 back-to-back calls after 3 warm-up calls.
Roofline of an all-reduce of S bytes on n ranks: each rank must send and receive S*(n-1)/n bytes; at the measured
770 GB/s per direction that is S*(n-1)/n / 770e9 seconds.
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def timed(fn, iters=20, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    from picotron_b200.comm.workspace import SymmetricWorkspace
    from picotron_b200.ops import _ext
    C = _ext.load()
    log = (lambda *a: print(*a, flush=True)) if rank == 0 else (lambda *a: None)
    cap = 256 << 20
    ws_p2p = SymmetricWorkspace(dist.group.WORLD, cap, num_blocks=128, use_multicast=False)
    ws_mc = SymmetricWorkspace(dist.group.WORLD, cap, num_blocks=128, use_multicast=True)
    log(f"world {world}; multicast mapping available: {ws_mc.mc_ptr != 0}")
    log(f"{'all-reduce':24s} {'MiB':>6s} {'p2p ms':>8s} {'multimem ms':>12s} {'NCCL ms':>8s} {'roofline ms':>12s} {'best/roofline':>14s}")
    for name, dtype, nbytes in [("bf16 TP activation", torch.bfloat16, 32 << 20), ("bf16 TP activation", torch.bfloat16, 16 << 20),
                                ("fp32 DDP bucket", torch.float32, 64 << 20), ("fp32 DDP bucket", torch.float32, 256 << 20)]:
        n = nbytes // torch.empty(0, dtype=dtype).element_size()
        a, b = ws_p2p.view(0, (n,), dtype), ws_mc.view(0, (n,), dtype)
        a.zero_(), b.zero_()
        c = torch.zeros(n, dtype=dtype, device="cuda")
        scale = 1.0 / world if dtype == torch.float32 else 1.0
        tp = timed(lambda: ws_p2p.all_reduce_(a, scale))
        tm = timed(lambda: ws_mc.all_reduce_(b, scale)) if ws_mc.mc_ptr else float("nan")
        tn = timed(lambda: dist.all_reduce(c))
        roof = nbytes * (world - 1) / world / 770e9 * 1e3
        best = min(tp, tm) if ws_mc.mc_ptr else tp
        log(f"{name:24s} {nbytes >> 20:6d} {tp:8.3f} {tm:12.3f} {tn:8.3f} {roof:12.3f} {roof / best:14.2f}")
    log("")
    log(f"{'GEMM + all-reduce':24s} {'M':>5s} {'N':>5s} {'K':>6s} {'fused ms':>9s} {'gemm+symm':>10s} {'gemm+NCCL':>10s} {'gemm only':>10s} "
        f"{'roofline ms':>12s} {'roofline/fused':>15s}")
    ws_mc.configure_ring(4, 64 << 20)
    for M, N, K, dgrad in [(4096, 4096, 2048, False), (4096, 4096, 5504, False), (4096, 4096, 11008 // 2, True),
                           (8192, 4096, 7168, False)]:
        g = torch.Generator(device="cuda").manual_seed(rank)
        x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
        w = torch.randn((K, N) if dgrad else (N, K), device="cuda", generator=g).to(torch.bfloat16)
        tf = timed(lambda: ws_mc.gemm_all_reduce(x, w, dgrad, ws_mc.ring_alloc((M, N), torch.bfloat16)))

        def unfused():
            out = ws_mc.ring_alloc((M, N), torch.bfloat16)
            C.gemm(x, w, False, dgrad, out, False)
            ws_mc.all_reduce_(out)

        def nccl():
            y = C.gemm(x, w, False, dgrad, None, False)
            dist.all_reduce(y)

        tu, tn = timed(unfused), timed(nccl)
        tg = timed(lambda: C.gemm(x, w, False, dgrad, None, False))
        roof = max(2.0 * M * N * K / 1.7017e15, M * N * 2 * (world - 1) / world / 770e9) * 1e3
        log(f"{'dgrad' if dgrad else 'row-parallel fwd':24s} {M:5d} {N:5d} {K:6d} {tf:9.3f} {tu:10.3f} {tn:10.3f} {tg:10.3f} "
            f"{roof:12.3f} {roof / tf:15.2f}")
    torch.cuda.synchronize()
    log("kernel status:", C.kernel_status())
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
