"""Gradient buckets: flat fp32 buffers that hold ``param.main_grad`` and are all-reduced as a unit.

Semantics of ``data_parallel/bucket.py:6-158`` of the reference: greedy assignment in
``module.parameters()`` order, a parameter larger than the cap gets a private bucket, one flat tensor
per bucket with ``param.main_grad`` a view into it, and an asynchronous all-reduce of
``grad_data / world`` as soon as the last parameter of a bucket is marked ready.

Additions: *atomic groups* (parameters that one GEMM consumes together, e.g. q/k/v, are never split
across buckets and stay adjacent so that a single weight-gradient GEMM can accumulate into their
common region), 256-byte alignment of every parameter's slot (TMA / vector access), and a
``reduce_fn`` hook through which the peer-memory all-reduce kernel replaces NCCL.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist
from torch import nn
from ..utils.tracing import nvtx_range

_ALIGN_ELEMS = 64  # 256 bytes of fp32


class Bucket:
    def __init__(self, params: List[nn.Parameter], grad_data: torch.Tensor, process_group) -> None:
        self.params = set(params)
        self.params_with_grad_ready = set()
        self.grad_data = grad_data
        self.process_group = process_group
        self.process_group_size = dist.get_world_size(group=process_group) if process_group is not None else 1
        self.handle = None
        self.reduce_fn: Optional[Callable[["Bucket"], object]] = None
        self.reset()

    def sync_gradient(self) -> None:
        """Average this bucket over the group (asynchronously)."""
        assert self.handle is None
        if self.process_group_size == 1:
            self.handle = _Done()
            return
        with nvtx_range("bucket_all_reduce"):
            if self.reduce_fn is not None:
                self.handle = self.reduce_fn(self)
                return
            self.grad_data /= self.process_group_size
            self.handle = dist.all_reduce(self.grad_data, group=self.process_group, async_op=True)

    def reset(self) -> None:
        self.handle = None
        self.params_with_grad_ready.clear()
        self.grad_data.zero_()

    def wait(self) -> None:
        assert self.handle is not None, "You should launch an allreduce operation before waiting for it to finish"
        self.handle.wait()

    def mark_param_as_ready(self, param: nn.Parameter) -> None:
        assert param in self.params and param not in self.params_with_grad_ready
        self.params_with_grad_ready.add(param)
        if len(self.params_with_grad_ready) == len(self.params):
            self.sync_gradient()


class _Done:
    def wait(self):
        return None


class BucketManager:
    def __init__(self, params: Sequence[nn.Parameter], process_group, bucket_size: int,
                 grad_type: torch.dtype = torch.float32,
                 atomic_groups: Optional[Sequence[Sequence[nn.Parameter]]] = None,
                 flat_factory: Optional[Callable[[int], Optional[torch.Tensor]]] = None) -> None:
        self.params = list(params)
        self.device = self.params[0].device if self.params[0].is_cuda else torch.device("cpu")
        self.buckets: List[Bucket] = []
        self.process_group = process_group
        self.process_group_size = dist.get_world_size(group=process_group) if process_group is not None else 1
        self.params_to_bucket_location: Dict[nn.Parameter, tuple] = {}
        self.bucket_size = bucket_size
        self.bucket_sizes: Optional[List[int]] = None
        self.grad_data_list: List[torch.Tensor] = []
        self.grad_type = grad_type
        self.flat_factory = flat_factory
        self.symmetric_workspace = None
        self.flat: Optional[torch.Tensor] = None
        self._group_of: Dict[nn.Parameter, List[nn.Parameter]] = {}
        for grp in atomic_groups or []:
            grp = list(grp)
            for p in grp:
                self._group_of[p] = grp
        self._initialize_buckets()

    def _units(self) -> List[List[nn.Parameter]]:
        """Parameters in order, with atomic groups collapsed into one unit at their first member."""
        units, seen = [], set()
        for p in self.params:
            if not p.requires_grad or p in seen:
                continue
            grp = self._group_of.get(p, [p])
            grp = [q for q in grp if q.requires_grad]
            for q in grp:
                seen.add(q)
            units.append(grp)
        return units

    def _initialize_buckets(self) -> None:
        cur_size, cur_idx = 0, 0
        for unit in self._units():
            # inside a unit the slots are packed back to back (no padding) so the unit is one 2-D region
            unit_numel = sum(p.numel() for p in unit)
            if cur_size != 0 and cur_size + unit_numel > self.bucket_size:
                cur_idx += 1
                cur_size = 0
            off = cur_size
            for p in unit:
                self.params_to_bucket_location[p] = (off, off + p.numel(), cur_idx)
                off += p.numel()
            cur_size = (off + _ALIGN_ELEMS - 1) // _ALIGN_ELEMS * _ALIGN_ELEMS

        n_buckets = cur_idx + 1
        sizes = [0] * n_buckets
        members: List[List[nn.Parameter]] = [[] for _ in range(n_buckets)]
        for p, (_, end, idx) in self.params_to_bucket_location.items():
            sizes[idx] = max(sizes[idx], end)
            members[idx].append(p)
        self.bucket_sizes = sizes
        # all buckets are slices of ONE flat buffer (64-element aligned starts): a single memset clears them and,
        # when a factory provides symmetric memory, one mapping serves every bucket's all-reduce
        starts, total = [], 0
        for sz in sizes:
            starts.append(total)
            total += (sz + _ALIGN_ELEMS - 1) // _ALIGN_ELEMS * _ALIGN_ELEMS
        flat = None
        if self.flat_factory is not None and self.grad_type == torch.float32:
            flat = self.flat_factory(total)
            if flat is not None:
                self.symmetric_workspace = getattr(self.flat_factory, "state", {}).get("ws")
        if flat is None:
            flat = torch.zeros(total, dtype=self.grad_type, device=self.device)
        else:
            flat.zero_()
        self.flat = flat
        for i in range(n_buckets):
            self.grad_data_list.append(flat[starts[i]:starts[i] + sizes[i]])
            self.buckets.append(Bucket(members[i], self.grad_data_list[i], self.process_group))
        for p in self.params[::-1]:
            if not p.requires_grad:
                continue
            start, end, idx = self.params_to_bucket_location[p]
            p.main_grad = self.grad_data_list[idx][start:end].view(p.shape)

    def set_reduce_fn(self, fn: Optional[Callable[[Bucket], object]]) -> None:
        for b in self.buckets:
            b.reduce_fn = fn

    def reset(self) -> None:
        self.flat.zero_()
        for b in self.buckets:
            b.handle = None
            b.params_with_grad_ready.clear()

    def wait(self) -> None:
        for b in self.buckets:
            b.wait()

    def mark_param_as_ready(self, param: nn.Parameter) -> None:
        self.buckets[self.params_to_bucket_location[param][2]].mark_param_as_ready(param)
