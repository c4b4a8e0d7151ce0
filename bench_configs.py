"""Throughput of the multi-axis configurations on 8 GPUs, for this framework and for the unmodified reference.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench_configs.py --config llama7b_3d
    ... --config llama1b_cp8 | llama8b_4d            ... --impl reference

Configs (shapes, grids and batch sizes of the benchmark definition):
  llama7b_3d    Llama-2-7B shape, dp2 x tp2 x pp2, 1F1B, micro-batch 4 x 1024, 32 grad-acc steps
  llama1b_cp8   Llama-3.2-1B shape (32q/8kv heads), cp8 ring attention, 1 x 32768 tokens, 8 grad-acc steps
  llama8b_4d    Llama-3-8B shape, tp2 x cp2 x pp2, 1F1B, 1 x 8192 tokens, 16 grad-acc steps
Synthetic uniform-random tokens, random-init weights, bf16. W warm-up optimizer steps (default 3), K timed (default 5);
CUDA-event time, max over ranks, SM clocks and throttle reasons sampled during the timed steps. One JSON line on rank 0.
The reference arm runs the reference's own modules and schedules from baseline/_ref; only the HF I/O is replaced
(see bench.py). ``measure_ours`` / ``measure_reference`` are also what ``bench.py --gpus 8`` calls for the Llama-2-7B
entry it appends to its own line.
"""
import argparse
import datetime
import json
import os
import sys
from types import SimpleNamespace

ROOT = os.path.dirname(os.path.abspath(__file__))
CONFIGS = {
    "llama7b_3d": dict(preset="meta-llama/Llama-2-7b-hf", tp=2, cp=1, pp=2, dp=2, engine="1f1b", mbs=4, seq=1024, ga=32),
    "llama1b_cp8": dict(preset="meta-llama/Llama-3.2-1B", tp=1, cp=8, pp=1, dp=1, engine="1f1b", mbs=1, seq=32768, ga=8),
    "llama8b_4d": dict(preset="meta-llama/Meta-Llama-3-8B", tp=2, cp=2, pp=2, dp=1, engine="1f1b", mbs=1, seq=8192, ga=16),
}
PEAK_FLOPS = 2.25e15       # nominal dense bf16 of a B200: the MFU denominator used for both arms


def timed_steps(torch, dist, step, warmup, steps):
    """(seconds for ``steps`` calls, clock record): device time, max over ranks, barrier + synchronize on both sides."""
    from bench import ClockSampler
    for _ in range(warmup):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(dist.get_rank() == 0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop(dist.get_world_size())
    dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1) / 1e3], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()), clocks


def result(name, c, secs, steps, warmup, impl, num_params, shape, clocks, extra=None):
    world = c["tp"] * c["cp"] * c["pp"] * c["dp"]
    tokens = c["mbs"] * c["seq"] * c["ga"] * c["dp"] * steps
    tps_gpu = tokens / secs / world
    fpt = 6 * num_params + 12 * shape["num_hidden_layers"] * shape["hidden_size"] * c["seq"]
    out = {"config": name, "impl": impl, "n_gpus": world, "tokens_per_second_per_gpu": tps_gpu,
           "tokens_per_second": tps_gpu * world, "mfu_pct": tps_gpu * fpt / PEAK_FLOPS * 100, "mfu_peak_flops": PEAK_FLOPS,
           "ms_per_step": secs / steps * 1e3, "steps": steps, "warmup": warmup,
           "grid": f"dp{c['dp']}.tp{c['tp']}.pp{c['pp']}.cp{c['cp']}", "pp_engine": c["engine"], "micro_batch": c["mbs"],
           "seq_len": c["seq"], "grad_acc_steps": c["ga"], "num_params": num_params,
           "data": "synthetic uniform-random token ids, random-init weights", "dtype": "bf16", "clocks": clocks}
    if extra:
        out.update(extra)
    return out


def resolve(name, overrides=None):
    c = dict(CONFIGS[name])
    for k, v in (overrides or {}).items():
        if v is not None:
            c[k] = v
    return c


def release(trainer=None):
    """Forget the process grid and the peer-memory workspaces of a finished run so that another grid can be built in the
    same process (the NCCL process group itself stays)."""
    import torch
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.comm import ring, symmetric
    from picotron_b200.parallel import pp_communications
    torch.cuda.synchronize()
    for rw in list(ring._CACHE.values()):
        rw.close()
    ring._CACHE.clear()
    symmetric.clear()
    pp_communications._P2P = None
    pgm.reset()
    torch.cuda.empty_cache()


def measure_ours(name, steps, warmup, overrides=None, extra_training=None, comm=None, extra_distributed=None):
    """Build the trainer of config ``name`` on the already launched ranks, time it, return the result dict (all ranks)."""
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from picotron_b200.config import MODEL_PRESETS
    from picotron_b200.ops import _ext
    from picotron_b200.trainer import build_trainer
    c = resolve(name, overrides)
    cfg = {"distributed": {"tp_size": c["tp"], "cp_size": c["cp"], "pp_size": c["pp"], "dp_size": c["dp"],
                           "pp_engine": c["engine"], "use_cpu": False, "bucket_cap_mb": 64,
                           # layers per stage chosen so that the LM head counts as work of the last stage (the reference always
                           # splits evenly); the split that was used is reported as `pp_layers`
                           "pp_layer_split": os.environ.get("PICOTRON_PP_SPLIT", "balanced"),
                           "cp_layout": os.environ.get("PICOTRON_CP_LAYOUT", "contiguous"),
                           **({"comm": comm} if comm else {}), **(extra_distributed or {})},
           # every shape field explicitly: the config template carries layer/head overrides of its own
           "model": {"name": c["preset"], "init": "normal", **{k: MODEL_PRESETS[c["preset"]][k] for k in
                     ("num_hidden_layers", "num_attention_heads", "num_key_value_heads")},
                     **({"num_hidden_layers": c["layers"]} if c.get("layers") else {})},
           "training": {"seed": 42, "learning_rate": 3e-4, "total_train_steps": 10 ** 9, "seq_length": c["seq"],
                        "micro_batch_size": c["mbs"], "gradient_accumulation_steps": c["ga"], "num_samples": None,
                        **(extra_training or {})},
           "dataset": {"name": "synthetic"},
           "logging": {"phase_timers": bool(os.environ.get("PICOTRON_PHASE_TIMERS"))}}
    tr = build_trainer(cfg)
    C = _ext.load()
    n0 = C.launch_count()
    secs, clocks = timed_steps(torch, dist, tr.step, warmup, steps)
    status = C.kernel_status()
    shape = dict(MODEL_PRESETS[c["preset"]])
    if c.get("layers"):
        shape["num_hidden_layers"] = c["layers"]
    extra = {"gpu_launches": int(C.launch_count() - n0), "cuda_graph": tr.graphed is not None}
    if c["pp"] > 1:
        from picotron_b200.parallel.pipeline_parallel import balanced_layer_split
        split = cfg["distributed"]["pp_layer_split"]
        extra["pp_layers"] = balanced_layer_split(tr.model_config, c["pp"]) if split == "balanced" else split
    if status:
        extra["invalid"] = f"kernel status {status:#x}"
    if tr.timers.enabled:
        from picotron_b200 import process_group_manager as pgm
        g = pgm.get()
        mine = {"coords": f"dp{g.dp_rank}.pp{g.pp_rank}.cp{g.cp_rank}.tp{g.tp_rank}",
                **{k: round(v, 1) for k, v in tr.timers.summary().items()}}
        every = [None] * dist.get_world_size()
        dist.all_gather_object(every, mine)
        extra["phase_ms_total_over_warmup_and_timed_steps"] = every
    out = result(name, c, secs, steps, warmup, "ours", tr.num_params, shape, clocks, extra)
    del tr
    release()
    return out


def measure_reference(name, steps, warmup, overrides=None):
    """The same measurement on the unmodified reference of baseline/_ref (its model, wrappers, schedules, AdamW)."""
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    os.environ.update(FLASH_ATTEN="1", DEVICE="cuda", DTYPE="bfloat16")
    os.environ.setdefault("HF_TOKEN", "offline")
    import torch
    import torch.distributed as dist
    c = resolve(name, overrides)
    from bench import REFERENCE_SHAPES
    if ref_root not in sys.path:
        sys.path.insert(0, ref_root)
    rank = dist.get_rank()
    device = torch.device("cuda", torch.cuda.current_device())
    import picotron.process_group_manager as pgm
    pgm.setup_process_group_manager(tp_size=c["tp"], cp_size=c["cp"], pp_size=c["pp"], dp_size=c["dp"])
    import train as ref_train
    from picotron.context_parallel.context_parallel import apply_context_parallel
    from picotron.data_parallel.data_parallel import DataParallelBucket
    from picotron.model import Llama
    from picotron.pipeline_parallel.pipeline_parallel import PipelineParallel, train_step_pipeline_1f1b
    from picotron.tensor_parallel.tensor_parallel import apply_tensor_parallel
    from picotron.utils import average_loss_across_dp_cp_ranks, set_all_seed
    from torch.optim import AdamW
    g = pgm.process_group_manager
    shape = dict(REFERENCE_SHAPES[c["preset"]])
    shape["max_position_embeddings"] = c["seq"]
    if c.get("layers"):
        shape["num_hidden_layers"] = c["layers"]
    model_config = SimpleNamespace(**shape)
    set_all_seed(42)
    # build order of train.py:174-193; the meta-device + safetensors detour is replaced by direct random init on the GPU
    with torch.device(device):
        model = Llama(config=model_config)
        if g.tp_world_size > 1:
            model = apply_tensor_parallel(model)
        if g.pp_world_size > 1:
            model = PipelineParallel(model, model_config)
    if g.cp_world_size > 1:
        model = apply_context_parallel(model)
    else:
        os.environ.pop("CONTEXT_PARALLEL", None)
    model.to(torch.bfloat16).to(device)
    torch.cuda.empty_cache()
    if g.dp_world_size > 1:
        model = DataParallelBucket(model)
    model.train()
    optimizer = AdamW(model.parameters(), lr=3e-4)
    s_local = c["seq"] // c["cp"]
    tensor_shapes = (c["mbs"], s_local, model_config.hidden_size)

    class Loader:
        grad_acc_steps = c["ga"]
        micro_batch_size = c["mbs"]
        seq_length_per_gpu = s_local

        def __init__(self):
            self.gen = torch.Generator().manual_seed(42 + g.dp_rank)

        def __iter__(self):
            return self

        def __next__(self):
            ids = torch.randint(0, model_config.vocab_size, (c["mbs"], c["seq"] + 1), generator=self.gen, dtype=torch.int64)
            lo = g.cp_rank * s_local
            return {"input_ids": ids[:, lo:lo + s_local].contiguous(), "target_ids": ids[:, lo + 1:lo + s_local + 1].contiguous(),
                    "position_ids": torch.arange(lo, lo + s_local).unsqueeze(0).expand(c["mbs"], -1).contiguous(),
                    "hidden_states": None}

    loader = Loader()

    def step():
        optimizer.zero_grad()
        if g.pp_world_size > 1:
            loss = train_step_pipeline_1f1b(model, loader, tensor_shapes, device, torch.bfloat16)
        else:
            loss = ref_train.train_step(model, loader, device)
        average_loss_across_dp_cp_ranks(loss, device)
        optimizer.step()
        if hasattr(model, "reset"):
            model.reset()

    secs, clocks = timed_steps(torch, dist, step, warmup, steps)
    n_local = sum(p.numel() * (g.tp_world_size if any(k in n.lower() for k in ("attention", "mlp", "embed", "final_proj")) else 1)
                  for n, p in model.named_parameters())
    t = torch.tensor([n_local], dtype=torch.int64, device=device)
    dist.all_reduce(t, group=g.pp_group)
    return result(name, c, secs, steps, warmup, "reference", int(t.item()), shape, clocks)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", choices=sorted(CONFIGS), required=True)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    for k in ("tp", "cp", "pp", "dp", "ga", "seq", "mbs", "layers"):      # smoke-test overrides (the result is then not the named config)
        ap.add_argument(f"--{k}", type=int, default=None)
    ap.add_argument("--no-graph", action="store_true", help="ours: run every micro-batch eagerly")
    ap.add_argument("--comm", choices=["fused", "nccl"], default=None, help="ours: peer-memory kernels (default) or NCCL")
    ap.add_argument("--sequence-parallel", action="store_true", help="ours: distributed.sequence_parallel")
    ap.add_argument("--zero1", action="store_true", help="ours: optimizer state sharded over the data-parallel replicas")
    a = ap.parse_args()
    os.environ.setdefault("OMP_NUM_THREADS", "1")
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    import torch
    import torch.distributed as dist
    rank, local_rank, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local_rank)
    dist.init_process_group(rank=rank, world_size=world, backend="nccl", init_method="env://",
                            timeout=datetime.timedelta(minutes=3), device_id=torch.device("cuda", local_rank))
    overrides = {k: getattr(a, k) for k in ("tp", "cp", "pp", "dp", "ga", "seq", "mbs", "layers")}
    named = all(v is None for v in overrides.values())
    if a.impl == "reference":
        out = measure_reference(a.config, a.steps, a.warmup, overrides)
    else:
        extra = {**({"cuda_graph": False} if a.no_graph else {}), **({"zero1": True} if a.zero1 else {})}
        out = measure_ours(a.config, a.steps, a.warmup, overrides, extra, a.comm,
                           {"sequence_parallel": True} if a.sequence_parallel else None)
        if a.sequence_parallel or a.zero1:
            out["options"] = {"sequence_parallel": a.sequence_parallel, "zero1": a.zero1}
    if not named:
        out["invalid"] = out.get("invalid", "smoke-test overrides: not the named configuration")
    if rank == 0:
        print(json.dumps(out), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
