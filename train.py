"""Training entry point.

    torchrun --nproc_per_node N train.py --config <path/to/config.json>

Same command line, JSON schema, step-log line and stopping rules as the reference's ``train.py:57-281``;
the work is done by :mod:`picotron_b200.trainer`. Step time is measured with CUDA events on the
device and reduced as the maximum over ranks (the reference uses the host wall clock of one rank).
"""
import argparse
import os
import signal
import time

import torch
import torch.distributed as dist

from picotron_b200 import process_group_manager as pgm
from picotron_b200.config import load_config
from picotron_b200.trainer import build_trainer, train_step  # noqa: F401  (train_step is part of the public surface)
from picotron_b200.utils import (MetricsWriter, format_step_line, get_mfu, print, to_readable_format)
from picotron_b200.utils.tracing import ProfilerWindow
from picotron_b200.utils.watchdog import StepWatchdog


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--config", type=str, default="", help="Path to config file")
    parser.add_argument("--dry_run", action="store_true",
                        help="no GPU, no process group: print what each pipeline stage would hold (layers, parameters, "
                             "memory against 180 GB) and exit; an impossible grid fails here as it would at start-up")
    args = parser.parse_args()
    config = load_config(args.config)
    if args.dry_run:
        from picotron_b200.utils.memory import describe_run
        for line in describe_run(config):
            print(line)
        return

    start = time.time()
    trainer = build_trainer(config)
    g = pgm.get()
    device = trainer.device
    world_size = g.world_size
    is_log_rank = g.tp_rank == 0 and g.dp_rank == 0 and g.cp_rank == 0 and g.pp_is_last_stage
    print(f"init time: {time.time() - start:.2f}s | {g} | params: {to_readable_format(trainer.num_params)} | "
          f"Tokens per step: {to_readable_format(trainer.tokens_per_step)}", is_print_rank=is_log_rank)

    use_wandb = bool(config["logging"]["use_wandb"]) and is_log_rank
    if use_wandb:
        import wandb
        wandb.init(project=config["logging"].get("project_name") or "picotron",
                   name=f"{config['logging']['run_name']}_{to_readable_format(trainer.tokens_per_step)}_{g}",
                   config={"tensor_parallel_size": g.tp_world_size, "context_parallel_size": g.cp_world_size,
                           "pipeline_parallel_size": g.pp_world_size, "data_parallel_size": g.dp_world_size,
                           "model": config["model"]["name"], "dataset": config["dataset"]["name"],
                           "max_tokens": config["training"]["max_tokens"],
                           "learning_rate": config["training"]["learning_rate"], "seed": config["training"]["seed"],
                           "micro_batch_size": trainer.data_loader.micro_batch_size,
                           "global_batch_size": trainer.data_loader.global_batch_size,
                           "gradient_accumulation": trainer.data_loader.grad_acc_steps})
    metrics = MetricsWriter(config["logging"].get("metrics_jsonl") if is_log_rank else None)
    watchdog = StepWatchdog(timeout_s=float(config["training"].get("step_timeout_s", 0) or 0))
    profiler = ProfilerWindow(config["logging"].get("profile"), rank=g.global_rank)
    max_tokens = config["training"]["max_tokens"]
    cuda = device.type == "cuda"
    # checkpoint.save_on_signal: SIGUSR1 (e.g. `#SBATCH --signal=USR1@120` before a time limit or a preemption) or SIGTERM
    # on ANY rank makes all ranks finish the current step, save it and exit cleanly; `load_path: "latest"` then resumes it
    stop_requested = {"signal": None}
    save_on_signal = bool(config["checkpoint"].get("save_on_signal", False))
    if save_on_signal:
        for sig in (signal.SIGUSR1, signal.SIGTERM):
            signal.signal(sig, lambda signum, frame: stop_requested.update(signal=signum))

    while max_tokens is None or trainer.trained_tokens < max_tokens:
        if cuda:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        t0 = time.time()
        with watchdog.step(trainer.step_idx):
            loss = trainer.step()
        profiler.step()
        if cuda:
            ev1.record()
            ev1.synchronize()
            duration = ev0.elapsed_time(ev1) / 1e3
        else:
            duration = time.time() - t0
        if world_size > 1:
            d = torch.tensor([duration], dtype=torch.float64, device=device)
            dist.all_reduce(d, op=dist.ReduceOp.MAX)
            duration = float(d.item())
        tokens_per_second = trainer.tokens_per_step / duration
        tokens_per_second_per_gpu = tokens_per_second / world_size
        mfu = get_mfu(tokens_per_second_per_gpu, trainer.num_params, trainer.model_config)
        mem = torch.cuda.memory_reserved() / 1e9 if cuda else 0.0
        if is_log_rank:
            print(format_step_line(g.global_rank, trainer.step_idx, loss, trainer.tokens_per_step, tokens_per_second,
                                   tokens_per_second_per_gpu, trainer.trained_tokens, max_tokens, mfu, mem))
            fields = {"loss": loss, "tokens_per_step": trainer.tokens_per_step, "tokens_per_second": tokens_per_second,
                      "mfu": mfu, "tokens_per_second_per_gpu": tokens_per_second_per_gpu, "memory_usage": mem,
                      "trained_tokens": trainer.trained_tokens}
            phases = {f"ms_{k}": v for k, v in trainer.timers.summary().items()}      # empty unless logging.phase_timers
            extras = {"lr": trainer.optimizer.param_groups[0]["lr"]}
            if trainer.last_grad_norm is not None:                                    # training.max_grad_norm
                extras["grad_norm"] = float(trainer.last_grad_norm)
            metrics.write(step=trainer.step_idx, step_seconds=duration, **fields, **phases, **extras)
            if use_wandb:
                wandb.log(fields)
        eval_every = int(config["training"].get("eval_every", 0) or 0)
        if eval_every and trainer.step_idx % eval_every == 0:
            val_loss = trainer.evaluate()
            if is_log_rank:
                print(f"[rank {g.global_rank}] Step: {trainer.step_idx:<5d} | Validation loss: {val_loss:6.4f}")
                metrics.write(step=trainer.step_idx, val_loss=val_loss)
                if use_wandb:
                    wandb.log({"val_loss": val_loss})
        saved = trainer.step_idx % config["checkpoint"]["save_frequency"] == 0
        if saved:
            trainer.save(os.path.join(config["checkpoint"]["save_dir"], str(trainer.step_idx)))
        if save_on_signal:
            flag = torch.tensor([1 if stop_requested["signal"] is not None else 0], dtype=torch.int32, device=device)
            if world_size > 1:
                dist.all_reduce(flag, op=dist.ReduceOp.MAX)       # one rank was told: every rank stops after this step
            if int(flag.item()):
                if not saved:
                    trainer.save(os.path.join(config["checkpoint"]["save_dir"], str(trainer.step_idx)))
                print(f"[rank {g.global_rank}] stop signal received: state of step {trainer.step_idx} saved, exiting",
                      is_print_rank=is_log_rank)
                break
        if trainer.step_idx >= config["training"]["total_train_steps"]:
            break

    trainer.checkpoint_manager.wait()                    # a background checkpoint write (checkpoint.async_save) finishes first
    profiler.close()
    if use_wandb:
        wandb.finish()
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
