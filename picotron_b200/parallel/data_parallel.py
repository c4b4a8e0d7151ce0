"""Data parallelism over the flattened CP x DP group.

``DataParallelNaive`` and ``DataParallelBucket`` keep the interface of ``data_parallel.py:10-170`` of the
reference (``require_backward_grad_sync``, ``no_sync()``, ``reset()``, ``backward(...)``, ``.module``,
``param.main_grad``).

How gradients reach the buckets differs. The fused model nodes accumulate weight gradients in the
epilogue of the weight-gradient GEMM directly into ``param.main_grad`` (fp32) and then call
``param._grad_ready_cb()``; parameters whose gradients still arrive through autograd are caught by the
same ``AccumulateGrad`` hook the reference uses (``data_parallel.py:107-144``). Both paths end in
:meth:`DataParallelBucket._on_grad_ready`, which marks the bucket and, for the last parameter of a
bucket, starts its asynchronous all-reduce while the rest of the backward pass runs.

The wrapper is meant to be applied whenever ``cp * dp > 1`` -- and also for a single rank, where it
simply provides fp32 accumulation across micro-batches with no communication.
The optimizer (:class:`picotron_b200.optim.FusedAdamW`) reads ``main_grad`` directly, so the
``p.grad = main_grad.to(p.dtype)`` pass of the reference (``data_parallel.py:153-165``) is only done on
request (``materialize_param_grads=True``, for stock ``torch.optim`` optimizers).
"""
from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist
from torch import nn
from torch.autograd import Variable

from .. import ops
from .. import process_group_manager as pgm
from .bucket import BucketManager


def _sync_group():
    g = pgm.get()
    return g.cp_dp_group if g.cp_dp_world_size > 1 else None


class DataParallelNaive(nn.Module):
    """Blocking all-reduce of every parameter gradient right after it is accumulated."""

    def __init__(self, module):
        super().__init__()
        self.module = module
        self.require_backward_grad_sync = True
        self.register_backward_hook(self._allreduce_grads)

    def forward(self, *inputs, **kwargs):
        return self.module(*inputs, **kwargs)

    def backward(self, input_tensor, output_tensor, output_tensor_grad):
        return self.module.backward(input_tensor, output_tensor, output_tensor_grad)

    def register_backward_hook(self, hook):
        for p in self.module.parameters():
            if p.requires_grad:
                p.register_post_accumulate_grad_hook(hook)

    def _allreduce_grads(self, param):
        group = _sync_group()
        if self.require_backward_grad_sync and group is not None and param.grad is not None:
            dist.all_reduce(param.grad, op=dist.ReduceOp.SUM, group=group)
            param.grad /= dist.get_world_size(group)

    @contextlib.contextmanager
    def no_sync(self):
        self.require_backward_grad_sync = False
        try:
            yield
        finally:
            self.require_backward_grad_sync = True


class DataParallelBucket(nn.Module):
    def __init__(self, module, bucket_cap_mb: int = 25, grad_type: torch.dtype = torch.float32,
                 materialize_param_grads: bool = False, flat_factory=None):
        super().__init__()
        self.module = module
        self.require_backward_grad_sync = True
        self.materialize_param_grads = materialize_param_grads
        grad_size = 2 if grad_type == torch.bfloat16 else 4
        bucket_size = bucket_cap_mb * 1024 * 1024 // grad_size
        groups = module.packed_param_groups() if hasattr(module, "packed_param_groups") else None
        self.bucket_manager = BucketManager(list(module.parameters()), _sync_group(), bucket_size, grad_type,
                                            atomic_groups=groups, flat_factory=flat_factory)
        self._post_backward_callback_set = False
        self.register_backward_hook()

    def forward(self, *inputs, **kwargs):
        return self.module(*inputs, **kwargs)

    def backward(self, input_tensor, output_tensor, output_tensor_grad):
        return self.module.backward(input_tensor, output_tensor, output_tensor_grad)

    def packed_param_groups(self):
        return self.module.packed_param_groups() if hasattr(self.module, "packed_param_groups") else []

    def register_backward_hook(self):
        # Tensor-level post-accumulate hooks (not hooks on long-lived AccumulateGrad nodes as the reference keeps,
        # data_parallel.py:107-117): a node created here would remember the stream of construction time, and the
        # autograd engine would later make a capturing stream wait on that stream, which breaks CUDA-graph capture.
        self._hook_handles = []
        for param in self.module.parameters():
            if not param.requires_grad:
                continue
            param._grad_ready_cb = self._make_ready_cb(param)
            self._hook_handles.append(param.register_post_accumulate_grad_hook(self._make_param_hook(param)))

    def _on_grad_ready(self, param):
        if not self.require_backward_grad_sync:
            return
        if not self._post_backward_callback_set:
            Variable._execution_engine.queue_callback(self._post_backward)
            self._post_backward_callback_set = True
        self.bucket_manager.mark_param_as_ready(param)

    def _make_ready_cb(self, param):
        def cb():
            self._on_grad_ready(param)
        return cb

    def _make_param_hook(self, param):
        def param_hook(*unused):
            if param.requires_grad and param.grad is not None:
                ops.accumulate_(param.main_grad, param.grad.data)
                param.grad = None
                self._on_grad_ready(param)
        return param_hook

    @contextlib.contextmanager
    def no_sync(self):
        self.require_backward_grad_sync = False
        try:
            yield
        finally:
            self.require_backward_grad_sync = True

    def _post_backward(self):
        self.bucket_manager.wait()
        self._post_backward_callback_set = False
        if self.materialize_param_grads:
            for p in self.module.parameters():
                if p.requires_grad:
                    p.grad = p.main_grad.to(p.dtype)

    def reset(self):
        self.bucket_manager.reset()
