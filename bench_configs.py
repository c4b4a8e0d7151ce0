"""Throughput of the multi-axis configurations on 8 GPUs, for this framework and for the unmodified reference.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench_configs.py --config llama7b_3d
    ... --config llama1b_cp8 | llama8b_4d            ... --impl reference

Configs (shapes, grids and batch sizes of the benchmark definition):
  llama7b_3d    Llama-2-7B shape, dp2 x tp2 x pp2, 1F1B, micro-batch 4 x 1024, 32 grad-acc steps
  llama1b_cp8   Llama-3.2-1B shape (32q/8kv heads), cp8 ring attention, 1 x 32768 tokens, 8 grad-acc steps
  llama8b_4d    Llama-3-8B shape, tp2 x cp2 x pp2, 1F1B, 1 x 8192 tokens, 16 grad-acc steps
Synthetic uniform-random tokens, random-init weights, bf16. W warm-up optimizer steps, K timed; CUDA-event time, max over
ranks. One JSON line on rank 0. The reference arm runs the reference's own modules and schedules from baseline/_ref; only
the HF I/O is replaced (see bench.py).
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


def timed_steps(torch, dist, step, warmup, steps):
    for _ in range(warmup):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1) / 1e3], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def report(args, c, secs, impl, num_params, shape):
    world = c["tp"] * c["cp"] * c["pp"] * c["dp"]
    tokens = c["mbs"] * c["seq"] * c["ga"] * c["dp"] * args.steps
    tps_gpu = tokens / secs / world
    fpt = 6 * num_params + 12 * shape["num_hidden_layers"] * shape["hidden_size"] * c["seq"]
    print(json.dumps({"config": args.config, "impl": impl, "n_gpus": world, "tokens_per_second_per_gpu": tps_gpu,
                      "tokens_per_second": tps_gpu * world, "mfu_pct": tps_gpu * fpt / 2.25e15 * 100, "ms_per_step":
                      secs / args.steps * 1e3, "steps": args.steps, "warmup": args.warmup, "grid":
                      f"dp{c['dp']}.tp{c['tp']}.pp{c['pp']}.cp{c['cp']}", "num_params": num_params,
                      "data": "synthetic uniform-random token ids, random-init weights", "dtype": "bf16"}), flush=True)


def run_ours(args, c):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from picotron_b200.config import MODEL_PRESETS
    from picotron_b200.trainer import build_trainer
    cfg = {"distributed": {"tp_size": c["tp"], "cp_size": c["cp"], "pp_size": c["pp"], "dp_size": c["dp"],
                           "pp_engine": c["engine"], "use_cpu": False, "bucket_cap_mb": 64},
           # every shape field explicitly: the config template carries layer/head overrides of its own
           "model": {"name": c["preset"], "init": "normal", **{k: MODEL_PRESETS[c["preset"]][k] for k in
                     ("num_hidden_layers", "num_attention_heads", "num_key_value_heads")},
                     **({"num_hidden_layers": c["layers"]} if c.get("layers") else {})},
           "training": {"seed": 42, "learning_rate": 3e-4, "total_train_steps": 10 ** 9, "seq_length": c["seq"],
                        "micro_batch_size": c["mbs"], "gradient_accumulation_steps": c["ga"], "num_samples": None},
           "dataset": {"name": "synthetic"}}
    tr = build_trainer(cfg)
    secs = timed_steps(torch, dist, tr.step, args.warmup, args.steps)
    from picotron_b200.ops import _ext
    status = _ext.load().kernel_status()
    if dist.get_rank() == 0:
        if status:
            print(json.dumps({"config": args.config, "impl": "ours", "invalid": f"kernel status {status:#x}"}))
        report(args, c, secs, "ours", tr.num_params, MODEL_PRESETS[c["preset"]])
    dist.destroy_process_group()


def run_reference(args, c):
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    os.environ.update(FLASH_ATTEN="1", DEVICE="cuda", DTYPE="bfloat16")
    os.environ.setdefault("HF_TOKEN", "offline")
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from picotron_b200.config import MODEL_PRESETS
    sys.path.insert(0, ref_root)
    rank, local_rank, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group(rank=rank, world_size=world, backend="nccl", init_method="env://",
                            timeout=datetime.timedelta(minutes=3))
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
    shape = dict(MODEL_PRESETS[c["preset"]])
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

    secs = timed_steps(torch, dist, step, args.warmup, args.steps)
    n_local = sum(p.numel() * (g.tp_world_size if any(k in n.lower() for k in ("attention", "mlp", "embed", "final_proj")) else 1)
                  for n, p in model.named_parameters())
    t = torch.tensor([n_local], dtype=torch.int64, device=device)
    dist.all_reduce(t, group=g.pp_group)
    if rank == 0:
        report(args, c, secs, "reference", int(t.item()), MODEL_PRESETS[c["preset"]])
    dist.destroy_process_group()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", choices=sorted(CONFIGS), required=True)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=2)
    for k in ("tp", "cp", "pp", "dp", "ga", "seq", "layers"):      # smoke-test overrides (the result is then not the named config)
        ap.add_argument(f"--{k}", type=int, default=None)
    a = ap.parse_args()
    os.environ.setdefault("OMP_NUM_THREADS", "1")
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    cfg = dict(CONFIGS[a.config])
    for k in ("tp", "cp", "pp", "dp", "ga", "seq"):
        if getattr(a, k) is not None:
            cfg[k] = getattr(a, k)
    cfg["layers"] = a.layers
    (run_reference if a.impl == "reference" else run_ours)(a, cfg)
