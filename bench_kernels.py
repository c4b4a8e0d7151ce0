"""Per-kernel timings against their rooflines (CUDA events, L2 flushed between iterations).

    python bench_kernels.py gemm            # model GEMM shapes vs the cuBLAS twin
    python bench_kernels.py gemm --small    # one small case, a few launches (what an ncu capture should run)
    python bench_kernels.py elementwise
    python bench_kernels.py attention
    python bench_kernels.py attention --phases   # cycle counters of the kernels' consumer threads, per phase
    python bench_kernels.py microbatch      # eager forward+backward micro-batches of the 24-layer SmolLM-1.7B; the last one runs
                                            # between cudaProfilerStart/Stop (for `ncu --profile-from-start off`: launch list)

Peaks come from MEASURED_PEAKS.json in the repository root when present.
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


_FLUSH = None


def flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


def time_ms(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def bench_gemm(small: bool):
    from picotron_b200.ops import _ext
    C = _ext.load()
    _, flops_peak, src = peaks()
    T = 4096
    shapes = [("qkv fwd", "fwd", T, 6144, 2048), ("out fwd", "fwd", T, 2048, 2048), ("gate_up fwd", "fwd", T, 16384, 2048),
              ("down fwd", "fwd", T, 2048, 8192), ("head fwd", "fwd", 2048, 49152, 2048),
              ("gate_up dgrad", "dgrad", T, 2048, 16384), ("down dgrad", "dgrad", T, 8192, 2048),
              ("gate_up wgrad", "wgrad", 16384, 2048, T), ("down wgrad", "wgrad", 2048, 8192, T),
              ("qkv wgrad", "wgrad", 6144, 2048, T), ("qkv dgrad", "dgrad", T, 2048, 6144),
              ("out wgrad", "wgrad", 2048, 2048, T), ("llama7b mlp fwd", "fwd", T, 22016, 4096),
              ("8192^3", "fwd", 8192, 8192, 8192)]
    if small:   # the ncu case: 160 MB of operands and output (larger than L2), 512 tiles = 7 per CTA pair, ~0.2 ms
        shapes = [("ncu case fwd", "fwd", 4096, 8192, 4096)]
    print(f"{'shape':18s} {'kind':6s} {'M':>6s} {'N':>6s} {'K':>6s} {'ours ms':>9s} {'TFLOP/s':>9s} {'of peak':>8s} "
          f"{'cuBLAS ms':>10s} {'ours/cuBLAS':>11s}{'direct-store ms':>16s}   (peak: {flops_peak / 1e12:.0f} TFLOP/s {src}; "
          f"direct-store = epilogue with per-thread stores instead of TMA store / reduce-add)")
    for name, kind, M, N, K in shapes:
        g = torch.Generator(device="cuda").manual_seed(0)
        rnd = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)
        if kind == "fwd":
            a, b = rnd(M, K), rnd(N, K)
            ours = lambda: C.gemm(a, b, False, False)
            lib = lambda: torch.matmul(a, b.t())
        elif kind == "dgrad":
            a, b = rnd(M, K), rnd(K, N)
            ours = lambda: C.gemm(a, b, False, True)
            lib = lambda: torch.matmul(a, b)
        else:
            a, b = rnd(K, M), rnd(K, N)
            acc = torch.zeros(M, N, device="cuda")
            ours = lambda: C.gemm(a, b, True, True, acc, True)
            lib = lambda: torch.matmul(a.t(), b)
        iters = 3 if small else 10
        t = time_ms(ours, iters=iters, warmup=1 if small else 3)
        tl = time_ms(lib, iters=iters, warmup=1 if small else 3)
        C.set_gemm_tma_epilogue(False)
        td = time_ms(ours, iters=iters, warmup=1 if small else 3)
        C.set_gemm_tma_epilogue(True)
        fl = 2.0 * M * N * K
        print(f"{name:18s} {kind:6s} {M:6d} {N:6d} {K:6d} {t:9.3f} {fl / t / 1e9:9.1f} {fl / (t * 1e-3) / flops_peak:8.2f} "
              f"{tl:10.3f} {tl / t:11.2f} {td:16.3f}")
    torch.cuda.synchronize()
    print("kernel status:", C.kernel_status())


def bench_fused_epilogues(small: bool):
    """GEMMs with fused epilogues against the same GEMM followed by the kernel(s) the epilogue replaces."""
    from picotron_b200.ops import _ext
    C = _ext.load()
    T, H, I, V = 4096, 2048, 8192, 49152
    g = torch.Generator(device="cuda").manual_seed(0)
    rnd = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)
    x, a_mid, res = rnd(T, H), rnd(T, I), rnd(T, H)
    w_gu, w_d, w_qkv = rnd(2 * I, H), rnd(H, I), rnd(3 * H, H)
    gu, dy = rnd(T, 2 * I), rnd(T, H)
    hc, w_head = rnd(2048, H), rnd(V, H)
    tg = torch.randint(0, V, (2048,), device="cuda")
    cos, sin = [t.cuda() for t in __import__("picotron_b200.ops", fromlist=["rope_tables"]).rope_tables(1024, 64, 1e4)]

    def unfused_rope():
        q = C.gemm(x, w_qkv, False, False)
        C.rope_(q, cos, sin, 64, 64, 1024, False)

    def unfused_ce():
        lg = C.gemm(hc, w_head, False, False)
        C.ce_stats(lg, tg, 0)

    cases = [("gate/up + SwiGLU", lambda: C.gemm_swiglu(x, w_gu), lambda: C.swiglu_fwd(C.gemm(x, w_gu, False, False))),
             ("qkv + RoPE", lambda: C.gemm_rope(x, w_qkv, cos, sin, 64, 64, 1024), unfused_rope),
             ("down + residual add", lambda: C.gemm_add(a_mid, w_d, res), lambda: C.add(res, C.gemm(a_mid, w_d, False, False))),
             ("down dgrad + SwiGLU bwd", lambda: C.gemm_dgrad_swiglu_bwd(dy, w_d, gu),
              lambda: C.swiglu_bwd(gu, C.gemm(dy, w_d, False, True))),
             ("head + CE statistics", lambda: C.gemm_ce_stats(hc, w_head, tg, 0), unfused_ce)]
    if small:
        cases = cases[3:4]
    print(f"{'GEMM + epilogue':26s} {'fused ms':>9s} {'separate ms':>12s} {'saved':>7s}")
    for name, fused, separate in cases:
        it = 3 if small else 10
        tf, ts = time_ms(fused, iters=it, warmup=1 if small else 3), time_ms(separate, iters=it, warmup=1 if small else 3)
        print(f"{name:26s} {tf:9.3f} {ts:12.3f} {100 * (1 - tf / ts):6.1f}%")
    torch.cuda.synchronize()
    print("kernel status:", C.kernel_status())


def bench_elementwise(small: bool = False):
    from picotron_b200.ops import _ext
    C = _ext.load()
    bw_peak, _, src = peaks()
    T, H, I, V = 4096, 2048, 8192, 49152
    g = torch.Generator(device="cuda").manual_seed(0)
    rnd = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)
    x, d, w = rnd(T, H), rnd(T, H), rnd(H)
    gu, da = rnd(T, 2 * I), rnd(T, I)
    logits = rnd(2048, V)
    tgt = torch.randint(0, V, (2048,), device="cuda")
    y, rstd = C.rmsnorm_fwd(x, w, 1e-5)
    lse = torch.zeros(2048, device="cuda") + 12.0
    qkv = rnd(T, 3 * H)
    cos, sin = [t.cuda() for t in __import__("picotron_b200.ops", fromlist=["rope_tables"]).rope_tables(1024, 64, 1e4)]
    cases = [("rmsnorm_fwd", lambda: C.rmsnorm_fwd(x, w, 1e-5), 2 * T * H * 2),
             ("add_rmsnorm_fwd", lambda: C.add_rmsnorm_fwd(x, d, w, 1e-5), 4 * T * H * 2),
             ("rmsnorm_bwd(+res)", lambda: C.rmsnorm_bwd(d, x, w, rstd, y), 4 * T * H * 2),
             ("rope (q,k)", lambda: C.rope_(qkv, cos, sin, 64, 64, 1024, False), 2 * T * 2 * H * 2),
             ("swiglu_fwd", lambda: C.swiglu_fwd(gu), 3 * T * I * 2),
             ("swiglu_bwd", lambda: C.swiglu_bwd(gu, da), 5 * T * I * 2),
             ("ce_stats", lambda: C.ce_stats(logits, tgt, 0), 2048 * V * 2),
             ("ce_grad_", lambda: C.ce_grad_(logits, tgt, lse, 1.0, 0), 2 * 2048 * V * 2),
             ("add", lambda: C.add(x, d), 3 * T * H * 2)]
    # the remaining bandwidth-bound kernels of a training step
    dw_acc = torch.zeros(H, device="cuda")
    ids = torch.randint(0, V, (T,), device="cuda")
    emb_w = rnd(V, H)
    emb_g = torch.zeros(V, H, device="cuda")
    n_adam = 64 << 20                                         # 64 Mi parameters: bf16 param + fp32 grad, m, v, master
    ap = [rnd(n_adam)]
    ag, am, av, aw = (torch.zeros(n_adam, device="cuda") for _ in range(4))
    acc32, g16 = torch.zeros(T * I, device="cuda"), rnd(T * I)
    mo, ml = torch.zeros(4, 1024, 32, 64, device="cuda"), torch.zeros(4, 32, 1024, device="cuda")
    mbo, mbl = rnd(4, 1024, 32, 64), torch.zeros(4, 32, 1024, device="cuda")
    cases += [("rmsnorm_bwd(+res,dw+=)", lambda: C.rmsnorm_bwd(d, x, w, rstd, y, dw_acc), 4 * T * H * 2),
              ("embedding_fwd", lambda: C.embedding_fwd(ids, emb_w, 0), 2 * T * H * 2),
              ("embedding_bwd", lambda: C.embedding_bwd(ids, x, emb_g, 0), T * H * 2 + 2 * T * H * 4),
              ("accumulate_ (fp32+=bf16)", lambda: C.accumulate_(acc32, g16), T * I * (2 + 8)),
              ("adamw (64 Mi params)", lambda: C.adamw_multi_(ap, [ag], [am], [av], [aw], 1, 1e-3, 0.9, 0.999, 1e-8, 0.01),
               n_adam * (4 + 8 + 8 + 8 + 2)),
              ("merge_attention_", lambda: C.merge_attention_(mo, ml, mbo, mbl), mo.numel() * (8 + 2) + 3 * ml.numel() * 4)]
    print(f"{'kernel':20s} {'ms':>8s} {'GB/s':>9s} {'of peak':>8s}   (peak: {bw_peak / 1e9:.0f} GB/s {src})")
    for name, fn, nbytes in cases:
        t = time_ms(fn, iters=2, warmup=1) if small else time_ms(fn)
        print(f"{name:20s} {t:8.4f} {nbytes / t / 1e6:9.1f} {nbytes / (t * 1e-3) / bw_peak:8.2f}")


def _library_attention_fwd(q, k, v, causal, scale):
    """flash-attn 2 (the reference's attention kernel), timed next to ours as the library baseline."""
    from flash_attn.flash_attn_interface import _flash_attn_forward
    out, lse, _, _ = _flash_attn_forward(q.contiguous(), k.contiguous(), v.contiguous(), 0.0, scale,
                                         causal=causal, window_size_left=-1, window_size_right=-1,
                                         softcap=0.0, alibi_slopes=None, return_softmax=False)
    return out, lse


def _library_attention_bwd(do, q, k, v, o, lse, causal, scale):
    from flash_attn.flash_attn_interface import _flash_attn_backward
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    _flash_attn_backward(do.contiguous(), q, k, v, o, lse, dq, dk, dv, 0.0, scale, causal, -1, -1, 0.0,
                         None, False)
    return dq, dk, dv


def bench_attention(small: bool):
    """Attention forward/backward vs the flash-attn 2 library twin; FLOPs counted as 4*B*h*Sq*Sk*d (x0.5 causal), bwd x2.5."""
    import math
    from picotron_b200.ops import _ext
    import picotron_b200.ops as ops
    C = _ext.load()
    _, flops_peak, src = peaks()
    cases = [(4, 1024, 32, 32, 64), (1, 4096, 32, 8, 64), (4, 1024, 32, 32, 128), (1, 8192, 32, 8, 128)]
    if small:   # the ncu case: q, k, v, o, dO of 32 MiB each (working set larger than L2)
        cases = [(4, 2048, 32, 32, 64)]
    print(f"{'B':>2s} {'S':>5s} {'hq':>3s} {'hkv':>3s} {'d':>4s} | {'fwd ms':>8s} {'TFLOP/s':>8s} {'lib ms':>8s} | {'bwd ms':>8s} "
          f"{'TFLOP/s':>8s} {'lib ms':>8s}   (peak {flops_peak / 1e12:.0f} TFLOP/s {src})")
    for B, S, hq, hkv, d in cases:
        g = torch.Generator(device="cuda").manual_seed(0)
        rnd = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)
        q, k, v, do = rnd(B, S, hq, d), rnd(B, S, hkv, d), rnd(B, S, hkv, d), rnd(B, S, hq, d)
        scale = 1 / math.sqrt(d)
        o, lse = C.attention_fwd(q, k, v, True, scale)
        fl = 4.0 * B * hq * S * S * d * 0.5
        it = 3 if small else 10
        tf = time_ms(lambda: C.attention_fwd(q, k, v, True, scale), iters=it, warmup=1)
        tb = time_ms(lambda: C.attention_bwd(do, q, k, v, o, lse, True, scale), iters=it, warmup=1)
        tlf = time_ms(lambda: _library_attention_fwd(q, k, v, True, scale), iters=it, warmup=1)
        tlb = time_ms(lambda: _library_attention_bwd(do, q, k, v, o, lse, True, scale), iters=it, warmup=1)
        print(f"{B:2d} {S:5d} {hq:3d} {hkv:3d} {d:4d} | {tf:8.3f} {fl / tf / 1e9:8.1f} {tlf:8.3f} | {tb:8.3f} "
              f"{2.5 * fl / tb / 1e9:8.1f} {tlb:8.3f}")
    torch.cuda.synchronize()
    print("kernel status:", C.kernel_status())


def bench_attention_phases():
    """Where the consumer threads of the attention kernels spend their cycles (clock64 counters inside the kernels)."""
    import math
    from picotron_b200.ops import _ext
    C = _ext.load()
    cases = [(4, 1024, 32, 32, 64), (1, 4096, 32, 8, 64), (4, 1024, 32, 32, 128), (1, 8192, 32, 8, 128)]
    print("cycles per key block (forward) / per query-block step (backward), thread 0 of every CTA, averaged over all CTAs")
    for B, S, hq, hkv, d in cases:
        g = torch.Generator(device="cuda").manual_seed(0)
        rnd = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)
        q, k, v, do = rnd(B, S, hq, d), rnd(B, S, hkv, d), rnd(B, S, hkv, d), rnd(B, S, hq, d)
        scale = 1 / math.sqrt(d)
        o, lse = C.attention_fwd(q, k, v, True, scale)
        C.attention_bwd(do, q, k, v, o, lse, True, scale)                 # warm-up of both kernels
        counters = torch.zeros(16, dtype=torch.int64, device="cuda")
        C.attention_set_profile(counters)
        try:
            C.attention_fwd(q, k, v, True, scale)
            C.attention_bwd(do, q, k, v, o, lse, True, scale)
            torch.cuda.synchronize()
        finally:
            C.attention_set_profile(None)
        c = [float(x) for x in counters.tolist()]
        print(f"B={B} S={S} hq={hq} hkv={hkv} d={d}")
        print(f"  fwd: wait S {c[14] / c[11]:6.0f} | read S + row max {c[8] / c[11]:6.0f} | wait O / rescale {c[9] / c[11]:6.0f} | "
              f"exp + store P {c[10] / c[11]:6.0f} | blocks per CTA {c[11] / c[13]:5.1f} | loop lifetime {c[12] / c[13]:9.0f}")
        print(f"  bwd: wait S, dP {c[0] / c[4]:6.0f} | read + exp + store P, dS {c[1] / c[4]:6.0f} | wait dQ {c[2] / c[4]:6.0f} | "
              f"drain dQ {c[3] / c[4]:6.0f} | steps per CTA {c[4] / c[6]:5.1f} | loop lifetime {c[5] / c[6]:9.0f}")
    print("kernel status:", C.kernel_status())


def bench_microbatch(small: bool):
    """Eager micro-batches (forward + backward, gradient accumulation into the fp32 buckets) of the headline model."""
    import time
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    for k, v in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1")):
        os.environ.setdefault(k, v)
    from picotron_b200.ops import _ext
    from picotron_b200.trainer import build_trainer
    layers = 2 if small else 24
    cfg = {"distributed": {"tp_size": 1, "cp_size": 1, "pp_size": 1, "dp_size": 1, "use_cpu": False, "bucket_cap_mb": 64},
           "model": {"name": "HuggingFaceTB/SmolLM-1.7B", "num_hidden_layers": layers, "num_attention_heads": 32,
                     "num_key_value_heads": 32, "init": "normal"},
           "training": {"seed": 42, "learning_rate": 3e-4, "total_train_steps": 10 ** 9, "seq_length": 1024,
                        "micro_batch_size": 4, "gradient_accumulation_steps": 4, "num_samples": None, "master_weights": True,
                        "cuda_graph": False},
           "dataset": {"name": "synthetic"}}
    tr = build_trainer(cfg)
    C = _ext.load()
    model, dev = tr.model, tr.device
    model.require_backward_grad_sync = False
    batch = next(tr.data_loader)
    ids, tgt = batch["input_ids"].to(dev), batch["target_ids"].to(dev)

    def micro():
        model(input_ids=ids, target_ids=tgt, loss_scale=0.25).backward()

    for _ in range(3):
        micro()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n0, t0 = C.launch_count(), time.perf_counter()
    e0.record()
    for _ in range(4):
        micro()
    e1.record()
    torch.cuda.synchronize()
    print(f"eager micro-batch ({layers} layers, 4 x 1024 tokens): {e0.elapsed_time(e1) / 4:.2f} ms device, "
          f"{(time.perf_counter() - t0) * 250:.2f} ms wall, {(C.launch_count() - n0) // 4} kernels of this library")
    torch.cuda.profiler.start()
    micro()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print("kernel status:", C.kernel_status())


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "fused", "elementwise", "attention", "microbatch"])
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--single-cta", action="store_true", help="GEMM on single CTAs instead of CTA pairs")
    ap.add_argument("--phases", action="store_true", help="attention: per-phase cycle counters instead of timings")
    a = ap.parse_args()
    if a.single_cta:
        from picotron_b200.ops import _ext
        _ext.load().set_gemm_pair(False)
    if a.what == "gemm":
        bench_gemm(a.small)
    elif a.what == "attention":
        bench_attention_phases() if a.phases else bench_attention(a.small)
    elif a.what == "microbatch":
        bench_microbatch(a.small)
    elif a.what == "fused":
        bench_fused_epilogues(a.small)
    else:
        bench_elementwise(a.small)
