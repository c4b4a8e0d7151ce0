"""Training engine shared by ``train.py`` and ``bench.py``.

``build_trainer(config)`` performs the start-up sequence of the reference's ``train.py:57-217`` (process
group + 4D grid, seed, dataloader, model on the meta device -> tensor parallel -> pipeline parallel ->
materialise -> context parallel -> dtype/device -> data parallel, optimizer, optional checkpoint
load) and returns a :class:`Trainer` whose ``step()`` runs one optimizer step (``train.py:219-240``):
all micro-batches, loss averaging over the CP x DP group, optimizer update, bucket reset.

Differences that matter for throughput: the loss of a micro-batch never leaves the device (the
reference calls ``.item()`` per micro-batch, ``train.py:53``) and is read once per step; the LM head
and the cross entropy are one fused, chunked node; the data-parallel wrapper (fp32 gradient buckets)
is always applied, also for ``cp * dp == 1`` where it only accumulates; input copies are
``non_blocking`` from pinned memory.

Beyond the reference, all optional and off by default: a learning-rate schedule and global-norm clipping, a skip of
updates with non-finite gradients, a bitwise check that replicas still agree, a validation loss (``Trainer.evaluate``),
a tied embedding / LM head, sequence parallelism, an optimizer sharded over the replicas, background checkpoint writes.
"""
from __future__ import annotations

import datetime
import os
import time
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

from . import process_group_manager as pgm
from .checkpoint import (CheckpointManager, find_latest_checkpoint, init_model_with_dematerialized_weights,
                         init_model_with_materialized_weights)
from .config import load_config, resolve_model_config, world_size_of
from .data import MicroBatchDataLoader
from .models.llama import Llama
from .optim import FusedAdamW, clip_grad_norm_, lr_at
from .parallel.context_parallel import apply_context_parallel
from .parallel.data_parallel import DataParallelBucket
from .parallel.pipeline_parallel import PipelineParallel, train_step_pipeline_1f1b, train_step_pipeline_afab
from .parallel.tensor_parallel import apply_tensor_parallel
from .parallel.tied_embeddings import sync_tied_embedding_grads
from .parallel.tp_communications import sync_sequence_parallel_grads
from .utils import average_loss_across_dp_cp_ranks, get_num_params, print, set_all_seed
from .utils.tracing import PhaseTimer, enable_nvtx, set_active_timer


def train_step(model, data_loader, device) -> float:
    """All micro-batches of one optimizer step without pipeline parallelism (``train.py:29-55``).

    Returns the mean loss of this rank's micro-batches (one device->host read at the end).
    """
    g = pgm.get()
    n = data_loader.grad_acc_steps
    requires_grad_sync = g.cp_dp_world_size > 1 or hasattr(model, "require_backward_grad_sync")
    acc = torch.zeros((), dtype=torch.float32, device=device)
    for i in range(n):
        batch = next(data_loader)
        input_ids = batch["input_ids"].to(device, non_blocking=True)
        target_ids = batch["target_ids"].to(device, non_blocking=True)
        if requires_grad_sync:
            model.require_backward_grad_sync = i == n - 1
        loss = model(input_ids=input_ids, target_ids=target_ids, loss_scale=1.0 / n)
        loss.backward()
        acc += loss.detach()
    return acc.item()


class GraphedMicroBatch:
    """One forward+backward micro-batch of gradient accumulation captured in a CUDA graph.

    A micro-batch of the 1.7B model is ~1100 kernel launches of 15-200 us each; replaying them as one graph removes
    the per-launch host work and most of the inter-kernel gaps. Weight gradients go straight into the static fp32
    buckets, so the graph has no outputs besides the loss accumulator. The last micro-batch of a step, which triggers
    gradient synchronisation callbacks, runs eagerly.

    Tensor- and context-parallel micro-batches are captured too: the peer-memory collectives inside them (fused GEMM +
    all-reduce, activation all-reduce, ring-attention barriers) keep their call counters in device memory, so a replay
    is indistinguishable from an eager run to the peers. Every rank of such a group must replay (or run eagerly) the
    same sequence, which the trainer guarantees by agreeing on the outcome of the capture across all ranks. Pipeline
    stages are not captured (their micro-batches interleave with point-to-point messages in a rank-dependent order).
    """

    def __init__(self, model, micro_batch_size: int, seq_len: int, device, loss_scale: float):
        self.model = model
        self.ids = torch.zeros(micro_batch_size, seq_len, dtype=torch.long, device=device)
        self.tgt = torch.zeros(micro_batch_size, seq_len, dtype=torch.long, device=device)
        self.loss_acc = torch.zeros((), dtype=torch.float32, device=device)
        self.loss_scale = loss_scale
        model.require_backward_grad_sync = False
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):                       # warm-up: lazy initialisation must not happen under capture
            for _ in range(2):
                self._body()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        from .ops import _ext
        self._C = _ext.load()
        self.graph = torch.cuda.CUDAGraph()
        n0 = self._C.launch_count()
        with torch.cuda.graph(self.graph):
            self._body()
        self.kernels_per_replay = int(self._C.launch_count() - n0)   # this library's kernels inside the graph
        torch.cuda.synchronize()
        model.require_backward_grad_sync = True

    def _body(self):
        loss = self.model(input_ids=self.ids, target_ids=self.tgt, loss_scale=self.loss_scale)
        loss.backward()
        self.loss_acc.add_(loss.detach())

    def run(self, input_ids, target_ids):
        self.ids.copy_(input_ids, non_blocking=True)
        self.tgt.copy_(target_ids, non_blocking=True)
        self.graph.replay()
        self._C.count_launches(self.kernels_per_replay)


def train_step_graphed(model, data_loader, device, graphed: GraphedMicroBatch) -> float:
    """`train_step` with the accumulation micro-batches replayed from a CUDA graph."""
    n = data_loader.grad_acc_steps
    graphed.loss_acc.zero_()
    for i in range(n - 1):
        batch = next(data_loader)
        graphed.run(batch["input_ids"], batch["target_ids"])
    batch = next(data_loader)
    model.require_backward_grad_sync = True
    loss = model(input_ids=batch["input_ids"].to(device, non_blocking=True),
                 target_ids=batch["target_ids"].to(device, non_blocking=True), loss_scale=1.0 / n)
    loss.backward()
    return (graphed.loss_acc + loss.detach()).item()


class ReplicaDivergence(RuntimeError):
    """Copies of a parameter that must be identical (data-parallel replicas, weights replicated over a tensor-parallel
    group, the two copies of a tied embedding) differ between ranks."""


def _fingerprints(params) -> torch.Tensor:
    """One int64 per parameter: the sum of its raw bit patterns (wrap-around), equal on two ranks iff, barring a
    collision, the tensors are bitwise equal. Exact where a floating-point checksum would hide rounding differences."""
    bits = {2: torch.int16, 4: torch.int32, 8: torch.int64}
    out = [p.detach().contiguous().view(bits[p.element_size()]).to(torch.int64).sum() for p in params]
    return torch.stack(out) if out else torch.zeros(0, dtype=torch.int64)


def verify_replicas(model) -> None:
    """Raise :class:`ReplicaDivergence` if parameters that should be identical on several ranks are not.

    The reference relies on every rank seeding identically and never checks (``train.py:103``); replicas that drift
    (a missed gradient reduction, a rank that skipped an update, memory corruption) keep training silently. Checked
    here: every parameter over the context/data-parallel group, the norm weights over the tensor-parallel group, a tied
    embedding / LM-head pair over its two pipeline stages. Collective: every rank calls it. Two small all-reduces per
    group that has more than one rank.
    """
    g = pgm.get()
    raw = model
    while hasattr(raw, "module") and hasattr(raw, "require_backward_grad_sync"):
        raw = raw.module
    named = list(raw.named_parameters())
    checks = []
    if g.cp_dp_world_size > 1:
        checks.append(("context/data-parallel replicas", g.cp_dp_group, named))
    if g.tp_world_size > 1:
        checks.append(("tensor-parallel copies", g.tp_group, [(n, p) for n, p in named if p.dim() == 1]))
    tied = getattr(raw, "_tied_embedding", None)
    if tied and tied[1] is not None:
        checks.append(("tied embedding / LM head", tied[1], [("embedding.weight | final_proj.weight", tied[0])]))
    found = []
    for what, group, items in checks:
        if not items:
            continue
        fp = _fingerprints([p for _, p in items])
        lo, hi = fp.clone(), fp.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=group)
        bad = (lo != hi).nonzero().flatten().tolist()
        if bad:
            found.append(f"{what} differ between ranks in {len(bad)} parameter(s), first: {[items[i][0] for i in bad[:5]]}")
    # every rank leaves together: a rank that raised alone would leave its other groups waiting in their collectives
    any_bad = torch.tensor([1 if found else 0], dtype=torch.int32, device=named[0][1].device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(any_bad, op=dist.ReduceOp.MAX)
    if int(any_bad.item()):
        raise ReplicaDivergence("; ".join(found) + f" (seen from rank {g.global_rank})" if found else
                                f"reported by another rank (rank {g.global_rank} saw its own groups agree)")


class KernelWaitTimeout(RuntimeError):
    """A peer-memory kernel of some rank gave up a bounded wait during the step (a peer was late by more than the limit)."""


def _device_status_reader(device):
    """Callable returning this device's kernel status word (0 = every bounded wait of every kernel was satisfied)."""
    if device.type != "cuda":
        return lambda: 0
    from .ops import _ext
    C = _ext.load()
    return lambda: int(C.kernel_status())


class Trainer:
    def __init__(self, config: Dict[str, Any], model, optimizer, data_loader, model_config, device, dtype):
        self.config, self.model, self.optimizer = config, model, optimizer
        self.data_loader, self.model_config, self.device, self.dtype = data_loader, model_config, device, dtype
        self.g = pgm.get()
        # a pipeline message carries this rank's tokens: 1/tp of the micro-batch's under sequence parallelism
        sp = self.g.tp_world_size if config["distributed"].get("sequence_parallel") else 1
        self.tensor_shapes = (data_loader.micro_batch_size, data_loader.seq_length_per_gpu // sp, model_config.hidden_size)
        self.tokens_per_step = data_loader.global_batch_size * config["training"]["seq_length"]
        self.num_params = get_num_params(model)
        self.checkpoint_manager = CheckpointManager()
        self.trained_tokens, self.step_idx = 0, 0
        log_cfg = config.get("logging", {})
        if log_cfg.get("nvtx"):
            enable_nvtx(True)
        # per-phase device timings of a step (logging.phase_timers): read with `self.timers.summary()`
        self.timers = PhaseTimer(device, enabled=bool(log_cfg.get("phase_timers", False)))
        set_active_timer(self.timers if self.timers.enabled else None)
        # read once per step before the optimizer update; tests replace it to inject a status on one rank
        self.status_reader = _device_status_reader(device)
        self.eval_loader = None                          # set by build_trainer when training.eval_every is given
        self.skipped_steps = 0                           # updates skipped by training.skip_nonfinite_steps
        self.last_grad_norm = None                       # global gradient norm of the last step (training.max_grad_norm)
        self.graphed: Optional[GraphedMicroBatch] = None
        g = self.g
        want_graph = bool(config["training"].get("cuda_graph", True)) and device.type == "cuda"
        if want_graph and g.pp_world_size == 1 and data_loader.grad_acc_steps > 1:
            try:
                self.graphed = GraphedMicroBatch(model, data_loader.micro_batch_size, data_loader.seq_length_per_gpu,
                                                 device, 1.0 / data_loader.grad_acc_steps)
            except Exception as e:  # noqa: BLE001
                print(f"[picotron_b200] CUDA graph capture of the micro-batch failed ({type(e).__name__}: {e}); running eagerly")
                self.graphed = None
            if dist.is_initialized() and dist.get_world_size() > 1:
                # ranks that share collectives must all replay or all run eagerly
                ok = torch.tensor([1 if self.graphed is not None else 0], dtype=torch.int32, device=device)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN)
                if int(ok.item()) == 0:
                    self.graphed = None
            if hasattr(model, "reset"):
                model.reset()                                # warm-up and capture accumulated into the buckets

    def step(self) -> float:
        """One optimizer step; returns the loss averaged over the CP x DP group (valid on last-stage ranks)."""
        cfg, g, tm = self.config, self.g, self.timers
        self.optimizer.zero_grad()
        t_host = time.perf_counter()
        with tm.phase("micro_batches"):                      # forward/backward of all micro-batches + gradient sync
            if g.pp_world_size > 1:
                engine = cfg["distributed"]["pp_engine"]
                if engine == "afab":
                    loss = train_step_pipeline_afab(self.model, self.data_loader, self.tensor_shapes, self.device, self.dtype)
                elif engine == "1f1b":
                    loss = train_step_pipeline_1f1b(self.model, self.data_loader, self.tensor_shapes, self.device, self.dtype)
                else:
                    raise ValueError(f"Invalid pipeline parallel engine: {engine}")
            elif self.graphed is not None:
                loss = train_step_graphed(self.model, self.data_loader, self.device, self.graphed)
            else:
                loss = train_step(self.model, self.data_loader, self.device)
        if tm.enabled:
            tm._add("host_wall_micro_batches", (time.perf_counter() - t_host) * 1e3)
        with tm.phase("loss_average"):
            loss = average_loss_across_dp_cp_ranks(loss, self.device)
        if self.model_config.tie_word_embeddings:
            sync_tied_embedding_grads(self.model)        # first + last pipeline stage; no-op when one rank holds both uses
        sync_sequence_parallel_grads(self.model)         # norm-weight gradients over the TP group; no-op unless SP is on
        self.check_kernel_status()
        if cfg["training"].get("skip_nonfinite_steps") and not self._gradients_are_finite(loss):
            self.skipped_steps += 1                      # no update, no step count; the data of this step is spent
            print(f"[picotron_b200] step {self.step_idx + 1}: non-finite loss or gradient on some rank, update skipped "
                  f"({self.skipped_steps} so far)", is_print_rank=self.g.global_rank == 0)
            self.trained_tokens += self.tokens_per_step
            if hasattr(self.model, "reset"):
                self.model.reset()
            return loss
        with tm.phase("optimizer"):
            t = cfg["training"]
            if t.get("max_grad_norm"):
                self.last_grad_norm = clip_grad_norm_(self.model, float(t["max_grad_norm"]))
            if t.get("lr_schedule"):
                schedule = {"total_steps": t.get("total_train_steps", 0), **t["lr_schedule"]}
                for group in self.optimizer.param_groups:
                    group["lr"] = lr_at(self.step_idx, t["learning_rate"], schedule)
            self.optimizer.step()
        self.trained_tokens += self.tokens_per_step
        self.step_idx += 1
        every = int(cfg["training"].get("verify_replicas_every", 0) or 0)
        if every and self.step_idx % every == 0:
            verify_replicas(self.model)
        with tm.phase("bucket_reset"):
            if hasattr(self.model, "reset"):
                self.model.reset()
        return loss

    @torch.no_grad()
    def evaluate(self) -> float:
        """Mean loss over ``training.eval_batches`` micro-batches of the evaluation data (the same batches at every call),
        averaged over the context/data-parallel group; forward passes only, no gradient buffer is touched. Collective:
        every rank calls it. Needs ``training.eval_every`` (the evaluation loader is built with the trainer)."""
        loader = self.eval_loader
        assert loader is not None, "no evaluation data: set training.eval_every in the config"
        loader.load_state_dict({"epoch": 0, "cursor": 0})
        if self.g.pp_world_size > 1:
            from .parallel.pipeline_parallel import evaluate_pipeline
            loss = evaluate_pipeline(self.model, loader, self.tensor_shapes, self.device, self.dtype)
        else:
            acc = torch.zeros((), dtype=torch.float32, device=self.device)
            for _ in range(loader.grad_acc_steps):
                batch = next(loader)
                acc += self.model(input_ids=batch["input_ids"].to(self.device, non_blocking=True),
                                  target_ids=batch["target_ids"].to(self.device, non_blocking=True))
            loss = (acc / loader.grad_acc_steps).item()
        return average_loss_across_dp_cp_ranks(loss, self.device)

    def _gradients_are_finite(self, loss: float) -> bool:
        """True when the loss and every gradient of every rank are finite (one reduction over this rank's gradient
        buffer and one scalar all-reduce over the world, so that all ranks take or skip the update together)."""
        import math
        manager = getattr(self.model, "bucket_manager", None)
        if manager is not None:
            ok = torch.isfinite(manager.flat.sum())
        else:
            grads = [p.grad for p in self.model.parameters() if p.grad is not None]
            ok = torch.isfinite(torch.stack([x.sum() for x in grads]).sum()) if grads else torch.tensor(True)
        bad = torch.tensor([0 if (bool(ok) and math.isfinite(loss)) else 1], dtype=torch.int32, device=self.device)
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        return int(bad.item()) == 0

    def check_kernel_status(self) -> None:
        """Abort the step on EVERY rank if a kernel of ANY rank gave up a bounded wait since the last check.

        The peer-memory collectives (gradient-bucket all-reduce, fused GEMM + all-reduce, ring attention barriers) return
        early with a status code when a peer does not show up within their limit; the gradients of such a step are not
        reduced, so the optimizer must not consume them. The micro-batch loop has already synchronised the device
        (the loss read), so this costs one small all-reduce over the world group per step.
        """
        status = int(self.status_reader())
        if dist.is_initialized() and dist.get_world_size() > 1:
            t = torch.tensor([status], dtype=torch.int64, device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            status = int(t.item())
        if status:
            raise KernelWaitTimeout(
                f"step {self.step_idx}: a kernel gave up a bounded wait on some rank (status {status:#x}: kernel id "
                f"{status >> 24}, site {(status >> 16) & 0xff}, block {status & 0xffff}); the gradients of this step are "
                "not fully reduced, the optimizer step was not applied")

    def save(self, out_dir: str) -> None:
        self.checkpoint_manager.save_checkpoint(self.model, self.optimizer, self.step_idx, self.trained_tokens, out_dir,
                                                extra={"data_loader": self.data_loader.state_dict()},
                                                asynchronous=bool(self.config["checkpoint"].get("async_save", False)))
        # only dp_rank == cp_rank == 0 write: without this barrier the other replicas would run ahead into the next
        # step's collectives while the writers are still in torch.save, and their device-side waits would expire
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()

    def load(self, path: str) -> None:
        self.step_idx, self.trained_tokens = self.checkpoint_manager.load_checkpoint(self.model, self.optimizer, path)
        extra = getattr(self.checkpoint_manager, "last_loaded", {})
        if "data_loader" in extra:
            self.data_loader.load_state_dict(extra["data_loader"])


def select_device_dtype(config):
    use_cpu = config["distributed"]["use_cpu"]
    if not use_cpu and torch.cuda.is_available():
        local_rank = int(os.environ.get("LOCAL_RANK", 0))
        torch.cuda.set_device(local_rank)
        device = torch.device("cuda", local_rank)
        dtype = torch.bfloat16 if torch.cuda.is_bf16_supported() else torch.float32
    else:
        device, dtype = torch.device("cpu"), torch.float32
    if config["model"].get("dtype") == "float32":
        dtype = torch.float32
    return device, dtype


def init_distributed(config) -> None:
    """``init_process_group`` (env:// rendezvous, 3-minute timeout as ``train.py:94``) + the 4D grid."""
    d = config["distributed"]
    world_size = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    assert world_size == world_size_of(config), "world_size must be equal to tp_size * pp_size * dp_size * cp_size"
    use_cpu = d["use_cpu"] or not torch.cuda.is_available()
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kwargs = {}
        if not use_cpu:
            kwargs["device_id"] = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group(rank=rank, world_size=world_size, backend="gloo" if use_cpu else "nccl",
                                init_method="env://", timeout=datetime.timedelta(minutes=3), **kwargs)
    pgm.setup_process_group_manager(tp_size=d["tp_size"], cp_size=d["cp_size"], pp_size=d["pp_size"], dp_size=d["dp_size"])


def build_model(config, model_config, device, dtype):
    """Meta-device build -> TP -> PP -> materialise -> CP -> dtype/device -> DP wrapper (``train.py:174-193``)."""
    g = pgm.get()
    init = config["model"].get("init", "reference")
    with init_model_with_dematerialized_weights():
        model = Llama(config=model_config, init=init)
        if g.tp_world_size > 1:
            model = apply_tensor_parallel(model)
        if g.pp_world_size > 1:
            from .parallel import pipeline_parallel as _pp
            _pp.LAYER_SPLIT = config["distributed"].get("pp_layer_split", "reference")
            model = PipelineParallel(model, model_config)
    # Every rank draws the full master tensors from the same seed in the same order, so replicas agree
    # without a broadcast and TP shards are slices of the single-GPU initialisation.
    set_all_seed(config["training"]["seed"])
    model = init_model_with_materialized_weights(model, model_config, save_dir="./hf_model_safetensors/",
                                                 load_pretrained=bool(config["model"].get("load_pretrained", False)),
                                                 device="cpu" if device.type == "cpu" else device)
    if g.cp_world_size > 1:
        model = apply_context_parallel(model)
    model.to(dtype).to(device)
    if model_config.tie_word_embeddings:
        from .parallel.tied_embeddings import tie_word_embeddings
        tie_word_embeddings(model)                       # before the gradient buckets and the optimizer see the parameters
    comm = config["distributed"].get("comm", "fused")
    fused_comm = device.type == "cuda" and comm == "fused" and dist.is_initialized() and dist.get_world_size() > 1
    factory = None
    if fused_comm:
        from .comm import fused
        factory = fused.grad_buffer_factory(g.cp_dp_group if g.cp_dp_world_size > 1 else None)
    model = DataParallelBucket(model, bucket_cap_mb=int(config["distributed"].get("bucket_cap_mb", 25)),
                               flat_factory=factory)
    from .parallel import context_parallel as _cpar
    _cpar.FUSED = bool(fused_comm)
    if fused_comm:
        t = config["training"]
        fused.enable_fused_collectives(model, max_tokens=t["micro_batch_size"] * t["seq_length"] // g.cp_world_size,
                                       hidden=model_config.hidden_size)
    model.train()
    return model


def build_trainer(config_or_path, init_dist: bool = True) -> Trainer:
    config = load_config(config_or_path)
    env = config.get("environment", {})
    for k in ("OMP_NUM_THREADS", "TOKENIZERS_PARALLELISM"):
        if env.get(k) is not None:
            os.environ[k] = str(env[k])
    device, dtype = select_device_dtype(config)
    if init_dist:
        init_distributed(config)
    g = pgm.get()
    from .parallel import context_parallel as _cpar
    _cpar.set_layout(config["distributed"].get("cp_layout", "contiguous"))    # read by the loader, the RoPE slice and the ring
    from .parallel import tp_communications as _tpc
    _tpc.SEQUENCE_PARALLEL = bool(config["distributed"].get("sequence_parallel", False))
    set_all_seed(config["training"]["seed"])
    model_config = resolve_model_config(config)
    if device.type == "cuda" and g.global_rank == 0:
        try:                                               # an estimate for the user's benefit: never a reason to stop a run
            from .utils.memory import check_fits
            for warning in check_fits(model_config, config, torch.cuda.get_device_properties(device).total_memory):
                print("[picotron_b200] memory plan: " + warning)
        except Exception as e:  # noqa: BLE001
            print(f"[picotron_b200] memory plan skipped ({type(e).__name__}: {e})")
    t, ds = config["training"], config["dataset"]
    data_loader = MicroBatchDataLoader(
        micro_batch_size=t["micro_batch_size"], seq_length=t["seq_length"], dataset_name=ds["name"],
        tokenizer_name=ds.get("tokenizer") or config["model"]["name"], grad_acc_steps=t["gradient_accumulation_steps"],
        device=device,
        num_workers=ds.get("num_workers", 0), num_proc=ds.get("num_proc", 1), num_samples=t.get("num_samples"),
        subset_name=ds.get("subset_name"), split=ds.get("split", "train"), vocab_size=model_config.vocab_size,
        seed=t["seed"])
    model = build_model(config, model_config, device, dtype)
    optimizer = FusedAdamW(model.parameters(), lr=t["learning_rate"],
                           betas=tuple(t.get("adam_betas", (0.9, 0.999))), eps=float(t.get("adam_eps", 1e-8)),
                           weight_decay=float(t.get("weight_decay", 1e-2)),      # defaults: torch.optim.AdamW's, as the reference
                           master_weights=bool(t.get("master_weights", True)),
                           shard_group=g.cp_dp_group if t.get("zero1") and g.cp_dp_world_size > 1 else None)
    trainer = Trainer(config, model, optimizer, data_loader, model_config, device, dtype)
    if t.get("eval_every"):
        # held-out data: another split of a hub dataset, another file, or (synthetic) another seed
        trainer.eval_loader = MicroBatchDataLoader(
            micro_batch_size=t["micro_batch_size"], seq_length=t["seq_length"], dataset_name=ds.get("eval_name") or ds["name"],
            tokenizer_name=ds.get("tokenizer") or config["model"]["name"], grad_acc_steps=int(t.get("eval_batches", 8)),
            device=device, num_workers=ds.get("num_workers", 0), num_proc=ds.get("num_proc", 1),
            num_samples=t.get("eval_samples"), subset_name=ds.get("subset_name"),
            split=ds.get("eval_split", "train" if ds.get("eval_name") else "validation"),
            vocab_size=model_config.vocab_size, seed=t["seed"] + 1)
    load_path = config["checkpoint"].get("load_path")
    if load_path == "latest":
        load_path = find_latest_checkpoint(config["checkpoint"]["save_dir"])
    if load_path:
        trainer.load(load_path)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
    return trainer
