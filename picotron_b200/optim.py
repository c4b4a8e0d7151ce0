"""Multi-tensor AdamW over the fp32 gradient buckets.

The reference asks ``torch.optim.AdamW`` for ``fused=True`` but never gets it
(``train.py:203-209``: a ``torch.device`` is compared with the string ``'cuda'``), so its optimizer step
is the multi-kernel ``foreach`` path on bf16 parameters and bf16 moments. This optimizer performs the
whole step for all parameters in one kernel launch: it reads the fp32 ``param.main_grad`` (falling back to
``param.grad``), keeps fp32 moments and -- optionally -- an fp32 master copy of each parameter, and
writes the rounded bf16 parameter back. Update rule and defaults are those of ``torch.optim.AdamW``
(betas 0.9/0.999, eps 1e-8, decoupled weight decay 0.01).

It subclasses ``torch.optim.Optimizer`` so ``state_dict()`` / ``load_state_dict()`` keep the usual
format, which is what the per-rank checkpoint files store under ``'optimizer'``.

``shard_group`` (``training.zero1``; not in the reference) shards the optimizer over the data-parallel replicas: every
parameter has one owning rank, which alone keeps its moments and master copy, updates it and broadcasts the new values.
That takes the 12 bytes per parameter of optimizer state down to 12 / dp while gradients and weights stay replicated.
``state_dict()`` reassembles the full state (collectively), so checkpoint files do not depend on the setting.
"""
from __future__ import annotations

from typing import Iterable

import torch
import torch.distributed as dist

from .ops import reference as ref
from .ops import _ext


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params: Iterable, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 1e-2, master_weights: bool = True, state_dtype: torch.dtype = torch.float32,
                 shard_group=None):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.master_weights = master_weights
        self.state_dtype = state_dtype
        self.shard_group = shard_group if shard_group is not None and dist.get_world_size(shard_group) > 1 else None
        self._owner = {}
        if self.shard_group is not None:
            # largest parameters first, each to the least loaded rank: the same assignment on every rank
            n = dist.get_world_size(self.shard_group)
            self._shard_rank = dist.get_rank(self.shard_group)
            load = [0] * n
            ordered = sorted(enumerate(self._all_params()), key=lambda ip: (-ip[1].numel(), ip[0]))
            for _, p in ordered:
                k = min(range(n), key=lambda r: (load[r], r))
                self._owner[p] = k
                load[k] += p.numel()

    def _all_params(self):
        return [p for grp in self.param_groups for p in grp["params"]]

    def _owns(self, p) -> bool:
        return self.shard_group is None or self._owner[p] == self._shard_rank

    def _init_state(self, p):
        st = self.state[p]
        if len(st) == 0:
            st["step"] = 0
            st["exp_avg"] = torch.zeros_like(p, dtype=self.state_dtype)
            st["exp_avg_sq"] = torch.zeros_like(p, dtype=self.state_dtype)
            if self.master_weights and p.dtype != torch.float32:
                st["master"] = p.detach().float().clone()
        return st

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            params, grads, ms, vs, masters = [], [], [], [], []
            step = None
            for p in group["params"]:
                if not self._owns(p):
                    continue
                g = getattr(p, "main_grad", None)
                if g is None:
                    g = p.grad
                if g is None:
                    continue
                st = self._init_state(p)
                st["step"] += 1
                step = st["step"]
                params.append(p.data)
                grads.append(g)
                ms.append(st["exp_avg"])
                vs.append(st["exp_avg_sq"])
                masters.append(st.get("master"))
            if not params:
                continue
            b1, b2 = group["betas"]
            if params[0].is_cuda:
                _ext.load().adamw_multi_(params, grads, ms, vs, masters, int(step), float(group["lr"]), float(b1),
                                         float(b2), float(group["eps"]), float(group["weight_decay"]))
            else:
                ref.adamw_step_(params, grads, ms, vs, masters, step, group["lr"], b1, b2, group["eps"],
                                group["weight_decay"])
        if self.shard_group is not None:
            self._broadcast_updated_parameters()
        return loss

    def _broadcast_updated_parameters(self) -> None:
        """Every owner sends the new values of its parameters to the other replicas, one flat message per owner."""
        params = self._all_params()
        for k in range(dist.get_world_size(self.shard_group)):
            owned = [p for p in params if self._owner[p] == k]
            if not owned:
                continue
            assert len({p.dtype for p in owned}) == 1, "parameters of one optimizer shard must share a dtype"
            if k == self._shard_rank:
                flat = torch.cat([p.data.reshape(-1) for p in owned])
            else:
                flat = torch.empty(sum(p.numel() for p in owned), dtype=owned[0].dtype, device=owned[0].device)
            dist.broadcast(flat, src=dist.get_global_rank(self.shard_group, k), group=self.shard_group)
            if k != self._shard_rank:
                off = 0
                for p in owned:
                    p.data.copy_(flat[off:off + p.numel()].view_as(p.data))
                    off += p.numel()

    def state_dict(self):
        """The usual format. With ``shard_group`` this is a COLLECTIVE over the group: every owner hands its moments and
        master copies to the group's first rank (the rank that writes checkpoints), tensor by tensor, so that the saved
        file is the one an unsharded run would write. Other ranks get their own shard back."""
        sd = super().state_dict()
        if self.shard_group is None:
            return sd
        params = self._all_params()
        dev = params[0].device
        steps = torch.tensor([int(self.state[p]["step"]) if self._owns(p) and len(self.state[p]) else 0 for p in params],
                             dtype=torch.int64, device=dev)
        dist.all_reduce(steps, op=dist.ReduceOp.MAX, group=self.shard_group)
        collector = self._shard_rank == 0
        state = dict(sd["state"]) if not collector else {}
        for i, p in enumerate(params):
            if int(steps[i]) == 0:
                continue                                        # no update has touched this parameter yet
            k = self._owner[p]
            kinds = ["exp_avg", "exp_avg_sq"] + (["master"] if self.master_weights and p.dtype != torch.float32 else [])
            entry = {"step": int(steps[i])}
            for kind in kinds:
                if k == self._shard_rank:
                    buf = self.state[p][kind]
                elif collector:
                    buf = torch.empty(p.shape, dtype=torch.float32 if kind == "master" else self.state_dtype, device=p.device)
                else:
                    continue
                if k != 0:                                      # owner -> collector (both know they take part)
                    if k == self._shard_rank:
                        dist.send(buf, dst=dist.get_global_rank(self.shard_group, 0), group=self.shard_group)
                    else:
                        dist.recv(buf, src=dist.get_global_rank(self.shard_group, k), group=self.shard_group)
                entry[kind] = buf
            if collector:
                state[i] = entry
        return {"state": state, "param_groups": sd["param_groups"]}

    def load_state_dict(self, state_dict):
        """Like the base class, but keeps the stored dtypes (the base class casts state to the parameter dtype,
        which would round the fp32 moments and master weights of bf16 parameters)."""
        saved_ids = [i for grp in state_dict["param_groups"] for i in grp["params"]]
        own = [p for grp in self.param_groups for p in grp["params"]]
        if self.shard_group is not None:                        # a full state comes in; this rank keeps what it owns
            keep = {pid for pid, p in zip(saved_ids, own) if self._owns(p)}
            state_dict = {"state": {pid: s for pid, s in state_dict["state"].items() if pid in keep},
                          "param_groups": state_dict["param_groups"]}
        super().load_state_dict(state_dict)
        for pid, p in zip(saved_ids, own):
            src = state_dict["state"].get(pid)
            if src is None:
                continue
            for k, v in src.items():
                if torch.is_tensor(v) and v.is_floating_point() and k != "step":
                    self.state[p][k] = v.detach().to(device=p.device, dtype=v.dtype).clone()

    def zero_grad(self, set_to_none: bool = True):
        """Clears ``.grad``; the fp32 buckets are cleared by the data-parallel wrapper's ``reset()``."""
        super().zero_grad(set_to_none=set_to_none)


# ----------------------------------------------------------------------------------------------------------------
# Learning-rate schedule and gradient clipping. The reference trains with a constant learning rate and unclipped
# gradients (``train.py:203-209``); both are therefore off unless the config asks for them
# (``training.lr_schedule``, ``training.max_grad_norm``).
# ----------------------------------------------------------------------------------------------------------------
def lr_at(step: int, base_lr: float, schedule) -> float:
    """Learning rate of optimizer step ``step`` (0-based).

    ``schedule`` is None (constant) or a dict: ``warmup_steps`` (linear from ``base_lr / warmup_steps``), ``decay`` in
    {"constant", "linear", "cosine"} over ``total_steps`` after the warm-up, down to ``min_lr_ratio * base_lr``. A pure
    function of the step index, so a resumed run continues the curve without any stored state.
    """
    if not schedule:
        return base_lr
    import math
    warm = int(schedule.get("warmup_steps", 0))
    if step < warm:
        return base_lr * (step + 1) / warm
    decay = schedule.get("decay", "constant")
    if decay == "constant":
        return base_lr
    total = max(int(schedule["total_steps"]), warm + 1)
    floor = float(schedule.get("min_lr_ratio", 0.0)) * base_lr
    frac = min(1.0, (step - warm) / (total - warm))
    if decay == "linear":
        return floor + (base_lr - floor) * (1.0 - frac)
    if decay == "cosine":
        return floor + (base_lr - floor) * 0.5 * (1.0 + math.cos(math.pi * frac))
    raise ValueError(f"unknown lr decay {decay!r}")


def clip_grad_norm_(model, max_norm: float) -> torch.Tensor:
    """Scale the fp32 gradient buckets so that the 2-norm of the WHOLE model's gradient is at most ``max_norm``.

    Call after the step's last backward pass (gradients averaged over the data-parallel group, tied copies and
    sequence-parallel norm gradients already summed). Every distinct parameter of the model counts once: shards are
    summed over the tensor-parallel and pipeline-parallel groups, parameters replicated over a tensor-parallel group
    (the norm weights) count 1/tp on each of its ranks, the last-stage copy of a tied embedding does not count.
    Costs one reduction over the flat gradient buffer, two scalar all-reduces and one scaling pass; no host sync.
    Returns the global norm before clipping (a 0-d tensor on the gradients' device).
    """
    import torch.distributed as dist
    from . import process_group_manager as pgm
    g = pgm.get()
    manager = getattr(model, "bucket_manager", None)
    raw = model
    while hasattr(raw, "module") and hasattr(raw, "require_backward_grad_sync"):
        raw = raw.module
    grads = {n: (getattr(p, "main_grad", None) if getattr(p, "main_grad", None) is not None else p.grad)
             for n, p in raw.named_parameters() if p.requires_grad}
    if manager is not None:
        sq = torch.linalg.vector_norm(manager.flat.float()).double() ** 2          # padding between buckets is zero
    else:
        sq = sum((torch.linalg.vector_norm(x.float()).double() ** 2 for x in grads.values() if x is not None),
                 torch.zeros((), dtype=torch.float64))
    over = torch.zeros_like(sq)
    if g.tp_world_size > 1:
        for n, x in grads.items():
            if x is not None and x.dim() == 1:
                over = over + (1.0 - 1.0 / g.tp_world_size) * torch.linalg.vector_norm(x.float()).double() ** 2
    tied = getattr(raw, "_tied_embedding", None)
    if tied and tied[1] is not None and g.pp_is_last_stage:
        x = getattr(tied[0], "main_grad", None)
        x = x if x is not None else tied[0].grad
        over = over + torch.linalg.vector_norm(x.float()).double() ** 2
    sq = sq - over
    if g.tp_world_size > 1:
        dist.all_reduce(sq, group=g.tp_group)
    if g.pp_world_size > 1:
        dist.all_reduce(sq, group=g.pp_group)
    norm = sq.clamp_min(0).sqrt()
    coef = torch.clamp(max_norm / (norm + 1e-6), max=1.0).float()
    if manager is not None:
        manager.flat.mul_(coef.to(manager.flat.dtype))
    else:
        for x in grads.values():
            if x is not None:
                x.mul_(coef.to(x.dtype))
    return norm.float()
