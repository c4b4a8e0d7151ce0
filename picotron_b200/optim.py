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
"""
from __future__ import annotations

from typing import Iterable

import torch

from .ops import reference as ref
from .ops import _ext


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params: Iterable, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 1e-2, master_weights: bool = True, state_dtype: torch.dtype = torch.float32):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.master_weights = master_weights
        self.state_dtype = state_dtype

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
        return loss

    def load_state_dict(self, state_dict):
        """Like the base class, but keeps the stored dtypes (the base class casts state to the parameter dtype,
        which would round the fp32 moments and master weights of bf16 parameters)."""
        super().load_state_dict(state_dict)
        saved_ids = [i for grp in state_dict["param_groups"] for i in grp["params"]]
        own = [p for grp in self.param_groups for p in grp["params"]]
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
