"""Headline benchmark: SmolLM-1.7B pre-training throughput, pure data parallel over N GPUs of one node.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref, same metric and config

Config (the reference's DP example): 24-layer SmolLM-1.7B shape (hidden 2048, intermediate 8192, 32/32 heads,
vocab 49152, untied head as the reference always builds it), bf16 compute, micro-batch 4 x 1024 tokens,
32 gradient-accumulation steps per optimizer step, dp = N (weak scaling), synthetic uniform-random token ids,
random-init weights. One "step" is a full optimizer step: 32 forward/backward micro-batches, gradient
all-reduce, AdamW update.

Two timed regions of K steps each, both bracketed by barrier + synchronize and taken as the max over ranks:
  value  device time (CUDA events) with the step's inputs already resident on the device;
  e2e    wall clock through the public API (Trainer.step): every micro-batch is copied from pinned host
         memory and the step's loss is read back to the host.
Inputs, weights, gradients and optimizer state of a step are several GB, far larger than the 126 MB L2, so
no explicit L2 flush is needed between iterations.

With ``--gpus 8`` the JSON line carries one more object, ``secondary``: the other model of the benchmark definition,
Llama-2-7B on a dp2 x tp2 x pp2 grid (1F1B, micro-batch 4 x 1024, 32 gradient-accumulation steps), measured after the
headline on the same ranks by ``bench_configs.measure_ours`` / ``measure_reference`` (a few optimizer steps, CUDA-event
time, max over ranks, own clock record). It runs under a deadline: if it fails or does not finish in time the line is
printed with ``secondary.error`` instead, so the headline number never depends on it. ``--no-secondary`` skips it.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
MODEL = "HuggingFaceTB/SmolLM-1.7B"
MBS, SEQ, GRAD_ACC = 4, 1024, 32
# tokens/s/GPU implied by the reference's published "nearly 50% MFU" for SmolLM-1.7B on 8xH100
# (0.5 * 989.5e12 / (6*1,812,039,680 + 12*24*2048*1024) FLOP/token)
PUBLISHED_TOKENS_PER_S_PER_GPU = 43.1e3
SECONDARY = {"config": "llama7b_3d", "steps": 3, "warmup": 2, "deadline_s": 420}
# architecture cards of the benchmark's models for the reference arm (which must not import this repository's package)
REFERENCE_SHAPES = {
    "meta-llama/Llama-2-7b-hf": dict(hidden_size=4096, intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32,
                                     num_key_value_heads=32, vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0),
    "meta-llama/Llama-3.2-1B": dict(hidden_size=2048, intermediate_size=8192, num_hidden_layers=16, num_attention_heads=32,
                                    num_key_value_heads=8, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0),
    "meta-llama/Meta-Llama-3-8B": dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                                       num_key_value_heads=8, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0),
}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    p.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (result is then marked invalid)")
    p.add_argument("--grad-acc", type=int, default=GRAD_ACC)
    p.add_argument("--no-secondary", action="store_true", help="--gpus 8: skip the Llama-2-7B dp2.tp2.pp2 measurement")
    return p.parse_args()


def setup_env(n_gpus: int):
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("OMP_NUM_THREADS", "1")
    os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "1")
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    world = int(os.environ["WORLD_SIZE"])
    if world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {n_gpus}")
    return int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), world


# ------------------------------------------------------------------------------------------- clocks
_CLOCK_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
                "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
                "clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs (rank 0 only)."""

    def __init__(self, enabled: bool):
        self.proc, self.path = None, None
        if not enabled:
            return
        self.path = f"/tmp/picotron_clocks_{os.getpid()}.csv"
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={_CLOCK_QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:  # noqa: BLE001
            self.proc = None

    def stop(self, n_gpus: int):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        self.out.close()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [x.strip() for x in line.split(",")]
                if len(parts) < 8:
                    continue
                try:
                    idx = int(parts[0])
                    if idx >= n_gpus:
                        continue
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                    power.append(float(parts[3]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[4:8]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        try:
            os.remove(self.path)
        except OSError:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "power_w_max": max(power), "samples": len(sm)}


# ------------------------------------------------------------------------------------------- timing
def timed_region(torch, dist, world, fn, steps: int, device_timed: bool) -> float:
    """Seconds for ``steps`` calls of ``fn`` (max over ranks); barrier + synchronize on both sides."""
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if device_timed:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    if device_timed:
        e1.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    secs = e0.elapsed_time(e1) / 1e3 if device_timed else wall
    if world > 1:
        t = torch.tensor([secs], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        secs = float(t.item())
    return secs


class DeviceResidentLoader:
    """Serves a pre-staged pool of micro-batches that already live on the device (device-timed region)."""

    def __init__(self, loader, device, pool: int):
        self.__dict__.update({k: getattr(loader, k) for k in ("micro_batch_size", "seq_length", "grad_acc_steps",
                                                              "global_batch_size", "num_global_micro_batches",
                                                              "seq_length_per_gpu")})
        self.batches = []
        for _ in range(pool):
            b = next(loader)
            self.batches.append({k: (v.to(device) if v is not None else None) for k, v in b.items()})
        self.i = 0

    def __iter__(self):
        return self

    def __next__(self):
        b = self.batches[self.i % len(self.batches)]
        self.i += 1
        return b


def result_line(args, world, secs_value, secs_e2e, clocks, launches, impl, extra_cfg, num_params, layers):
    tokens_per_step = MBS * SEQ * args.grad_acc * world
    value = tokens_per_step * args.steps / secs_value
    e2e = tokens_per_step * args.steps / secs_e2e
    flops_per_token = 6 * num_params + 12 * layers * 2048 * SEQ
    peak = float(os.environ.get("PICOTRON_PEAK_FLOPS", 2.25e15))
    ids_bytes = MBS * SEQ * 8
    out = {
        "metric": "tokens_per_second", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": secs_value / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": (value / world) / PUBLISHED_TOKENS_PER_S_PER_GPU, "dtype": "bf16",
        "data": "synthetic uniform-random token ids, random-init weights", "impl": impl,
        "tokens_per_second_per_gpu": value / world, "mfu_pct": value / world * flops_per_token / peak * 100,
        "mfu_peak_flops": peak,
        "config": {"model": f"SmolLM-1.7B ({layers} layers, untied head)", "global_batch": MBS * args.grad_acc * world,
                   "micro_batch": MBS, "grad_acc_steps": args.grad_acc, "seq_len": SEQ, "parallelism": f"dp{world}",
                   "l2": "inputs larger than L2 (multi-GB working set per step), no explicit flush", **extra_cfg},
        "clocks": clocks,
        "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": secs_e2e / args.steps * 1e3,
                "h2d_bytes_per_step": 2 * ids_bytes * args.grad_acc * world, "d2h_bytes_per_step": 4 * world},
        "gpu_launches": launches,
    }
    if layers != 24 or args.grad_acc != GRAD_ACC:
        out["invalid"] = "debug run on a reduced config"
    return out


def with_secondary(out, rank, world, args, impl):
    """At 8 GPUs: measure the Llama-2-7B 3D configuration on the same ranks and attach it to ``out`` (rank 0 prints).

    A timer on every rank bounds the attempt: when it fires, rank 0 prints the headline line with ``secondary.error`` and
    every rank leaves with exit code 0, so that a stuck collective in the second measurement cannot cost the first.
    """
    import threading
    printed = threading.Lock()

    def emit(secondary):
        if rank == 0 and printed.acquire(blocking=False):
            if secondary is not None:
                out["secondary"] = secondary
            print(json.dumps(out), flush=True)

    if world != 8 or args.no_secondary or args.layers or args.grad_acc != GRAD_ACC:
        emit(None)
        return

    def on_deadline():
        emit({"config": SECONDARY["config"], "impl": impl, "error": f"not finished within {SECONDARY['deadline_s']} s"})
        sys.stdout.flush()
        os._exit(0)

    timer = threading.Timer(SECONDARY["deadline_s"], on_deadline)
    timer.daemon = True
    timer.start()
    try:
        import bench_configs
        fn = bench_configs.measure_ours if impl == "ours" else bench_configs.measure_reference
        sec = fn(SECONDARY["config"], SECONDARY["steps"], SECONDARY["warmup"])
    except BaseException as e:  # noqa: BLE001
        sec = {"config": SECONDARY["config"], "impl": impl, "error": f"{type(e).__name__}: {e}"[:300]}
    timer.cancel()
    emit(sec)


# ------------------------------------------------------------------------------------------- our arm
def run_ours(args):
    rank, local_rank, world = setup_env(args.gpus)
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from picotron_b200.ops import _ext
    from picotron_b200.trainer import build_trainer

    layers = args.layers or 24
    cfg = {
        "distributed": {"tp_size": 1, "cp_size": 1, "pp_size": 1, "dp_size": world, "use_cpu": False,
                        "bucket_cap_mb": 64},
        "model": {"name": MODEL, "num_hidden_layers": layers, "num_attention_heads": 32, "num_key_value_heads": 32,
                  "init": "normal"},
        "training": {"seed": 42, "learning_rate": 3e-4, "total_train_steps": 10 ** 9, "seq_length": SEQ,
                     "micro_batch_size": MBS, "gradient_accumulation_steps": args.grad_acc, "num_samples": None,
                     "master_weights": True},
        "dataset": {"name": "synthetic"},
    }
    trainer = build_trainer(cfg)
    C = _ext.load()
    host_loader = trainer.data_loader
    dev_loader = DeviceResidentLoader(host_loader, trainer.device, pool=args.grad_acc * 2)

    def step_device():
        trainer.data_loader = dev_loader
        trainer.step()

    def step_e2e():
        trainer.data_loader = host_loader
        trainer.step()

    for _ in range(args.warmup):
        step_e2e()
    status = C.kernel_status()
    if status:
        raise SystemExit(f"a kernel reported a timed-out wait during warm-up (status {status:#x})")

    sampler = ClockSampler(rank == 0)
    n0 = C.launch_count()
    secs_value = timed_region(torch, dist, world, step_device, args.steps, device_timed=True)
    launches = C.launch_count() - n0
    secs_e2e = timed_region(torch, dist, world, step_e2e, args.steps, device_timed=False)
    clocks = sampler.stop(world)
    status = C.kernel_status()
    if rank == 0:
        out = result_line(args, world, secs_value, secs_e2e, clocks, launches, "ours",
                          {"gemm": "tcgen05", "attention": "tcgen05",
                           "precision": "bf16 params/activations, fp32 grad buckets, fp32 Adam moments + master weights"},
                          trainer.num_params, layers)
        if status:
            out["invalid"] = f"kernel status {status:#x}"
    else:
        out = {}
    del trainer, dev_loader, host_loader
    if world == 8 and not args.no_secondary:
        import bench_configs
        bench_configs.release()
    with_secondary(out, rank, world, args, "ours")
    if dist.is_initialized():
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------- reference arm
def run_reference(args):
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "picotron")) or not os.path.exists(os.path.join(ref_root, "train.py")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref holds no reference sources (picotron/ and train.py)"}))
        return
    rank, local_rank, world = setup_env(args.gpus)
    os.environ["FLASH_ATTEN"] = "1"
    os.environ["DEVICE"] = "cuda"
    os.environ["DTYPE"] = "bfloat16"
    os.environ.setdefault("HF_TOKEN", "offline")
    os.environ.setdefault("WANDB_MODE", "disabled")
    import datetime
    from types import SimpleNamespace
    import torch
    import torch.distributed as dist
    try:
        sys.path.insert(0, ref_root)
        import picotron.process_group_manager as pgm
        from picotron.process_group_manager import setup_process_group_manager
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"reference import failed: {type(e).__name__}: {e}"[:300]}))
        return

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group(rank=rank, world_size=world, backend="nccl", init_method="env://",
                            timeout=datetime.timedelta(minutes=3))
    setup_process_group_manager(tp_size=1, cp_size=1, pp_size=1, dp_size=world)
    try:
        import train as ref_train                                   # the reference's train.py (train_step)
        from picotron.model import Llama
        from picotron.data_parallel.data_parallel import DataParallelBucket
        from picotron.utils import average_loss_across_dp_cp_ranks, set_all_seed
        from torch.optim import AdamW
    except Exception as e:  # noqa: BLE001
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"reference import failed: {type(e).__name__}: {e}"[:300]}))
        dist.destroy_process_group()
        return

    layers = args.layers or 24
    set_all_seed(42)
    model_config = SimpleNamespace(hidden_size=2048, intermediate_size=8192, num_hidden_layers=layers,
                                   num_attention_heads=32, num_key_value_heads=32, vocab_size=49152,
                                   rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=SEQ)
    with torch.device(device):                                       # random init straight on the GPU (untimed set-up)
        model = Llama(config=model_config)
    model.to(torch.bfloat16).to(device)
    if world > 1:
        model = DataParallelBucket(model)
    model.train()
    optimizer = AdamW(model.parameters(), lr=3e-4)                   # what train.py:203-209 ends up constructing
    num_params = sum(p.numel() for p in model.parameters())

    class SyntheticLoader:
        """Offline stand-in for MicroBatchDataLoader: pinned uniform-random ids of the same shape."""
        grad_acc_steps = args.grad_acc
        micro_batch_size = MBS
        seq_length_per_gpu = SEQ

        def __init__(self):
            self.gen = torch.Generator().manual_seed(42 + rank)

        def __iter__(self):
            return self

        def __next__(self):
            ids = torch.randint(0, 49152, (MBS, SEQ + 1), generator=self.gen, dtype=torch.int64)
            return {"input_ids": ids[:, :-1].contiguous().pin_memory(), "target_ids": ids[:, 1:].contiguous().pin_memory(),
                    "position_ids": torch.arange(SEQ).unsqueeze(0).expand(MBS, -1).contiguous(), "hidden_states": None}

    loader = SyntheticLoader()

    def step():                                                      # body of the loop at train.py:219-240
        optimizer.zero_grad()
        loss = ref_train.train_step(model, loader, device)
        loss = average_loss_across_dp_cp_ranks(loss, device)
        optimizer.step()
        if hasattr(model, "reset"):
            model.reset()
        return loss

    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(rank == 0)
    secs_value = timed_region(torch, dist, world, step, args.steps, device_timed=True)
    secs_e2e = timed_region(torch, dist, world, step, args.steps, device_timed=False)
    clocks = sampler.stop(world)
    if rank == 0:
        out = result_line(args, world, secs_value, secs_e2e, clocks, None, "reference",
                          {"precision": "bf16 params/grads/Adam states (reference default), fp32 grad buckets when dp>1",
                           "note": "both timed regions run the reference's own train_step (H2D + .item() per micro-batch)"},
                          num_params, layers)
    else:
        out = {}
    del model, optimizer, loader
    torch.cuda.empty_cache()
    with_secondary(out, rank, world, args, "reference")
    dist.destroy_process_group()


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
