"""Tensor-parallel communication primitives.

Autograd functions with the semantics of the reference's ``tp_communications.py:19-101``:
``CopyToModelParallelRegion`` (f: identity forward / all-reduce backward),
``ReduceFromModelParallelRegion`` (g: all-reduce forward / identity backward),
``GatherFromModelParallelRegion`` (all-gather of the last dim forward / local slice backward) and
``LinearWithAsyncAllReduce`` (grad-input all-reduce overlapped with the grad-weight GEMM).

``all_reduce_`` is the single entry the fused model nodes use; on CUDA it routes to the peer-memory
all-reduce kernel of :mod:`picotron_b200.comm` when a symmetric workspace is registered for the group
and the run asked for ``distributed.comm == "fused"``, otherwise to NCCL/Gloo.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .. import process_group_manager as pgm
from .. import ops
from ..utils.tracing import nvtx_range

_OPS = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX}


def all_reduce_(t: torch.Tensor, group, op: str = "sum", async_op: bool = False):
    """In-place all-reduce over ``group`` (no-op for ``None`` or single-rank groups)."""
    if group is None or dist.get_world_size(group) == 1:
        return None
    if t.is_cuda and op == "sum" and not async_op:
        from ..comm import symmetric
        ws = symmetric.workspace_for(group)
        if ws is not None and ws.can_all_reduce(t):
            with nvtx_range("all_reduce/peer_memory"):
                ws.all_reduce_(t)
            return None
    with nvtx_range("all_reduce/nccl"):
        return dist.all_reduce(t, op=_OPS[op], group=group, async_op=async_op)


def stats_workspace(group, like: torch.Tensor, n: int):
    """The group's symmetric workspace when it can exchange the cross-entropy statistics of ``n`` rows, else None."""
    if group is None or not like.is_cuda:
        return None
    from ..comm import symmetric
    ws = symmetric.workspace_for(group)
    return ws if ws is not None and ws.can_exchange_ce_stats(n) else None


def reduce_buffer(shape, dtype, device, group) -> Optional[torch.Tensor]:
    """An output buffer for a GEMM whose result is all-reduced over ``group`` next: a slot of the group's
    symmetric workspace when one is registered (the reduction then runs in place on peer memory), else None."""
    if group is None or device.type != "cuda":
        return None
    from ..comm import symmetric
    ws = symmetric.workspace_for(group)
    return ws.ring_alloc(shape, dtype) if ws is not None else None


def linear_all_reduce(x: torch.Tensor, w: torch.Tensor, group, dgrad: bool = False) -> torch.Tensor:
    """``all_reduce(x @ w^T)`` (row-parallel forward) or ``all_reduce(x @ w)`` (``dgrad``: column-parallel input gradient).

    With a symmetric workspace registered for ``group`` this is ONE kernel: the GEMM writes its tiles into a
    symmetric slot and the tiles are summed across ranks over NVLink while later tiles are still being computed.
    Otherwise: GEMM, then ``all_reduce_``.
    """
    rows = x.shape[0]
    cols = w.shape[1] if dgrad else w.shape[0]
    if group is not None and x.is_cuda and x.dtype == torch.bfloat16 and FUSE_GEMM_ALL_REDUCE != "0":
        from ..comm import symmetric
        ws = symmetric.workspace_for(group)
        if ws is not None and FUSE_GEMM_ALL_REDUCE == "auto" and ws.mc_ptr == 0:
            ws = None
        out = ws.ring_alloc((rows, cols), x.dtype) if ws is not None else None
        if out is not None:
            with nvtx_range("gemm+all_reduce"):
                return ws.gemm_all_reduce(x, w, dgrad, out)
    out = reduce_buffer((rows, cols), x.dtype, x.device, group)
    y = ops.linear_dgrad(x, w, out=out) if dgrad else ops.linear_fwd(x, w, out=out)
    all_reduce_(y, group)
    return y


import os as _os

# One fused kernel (GEMM + tile-wise all-reduce) instead of GEMM followed by an all-reduce kernel: "auto" uses it when the
# workspace reduces through the NVSwitch (multimem, groups of 4+ ranks), where it measured 1.6x faster than GEMM + NCCL;
# between 2 ranks its reducer pulls tiles with peer loads and a 7B-shape step measured 3 % SLOWER than the plain GEMM
# followed by the push all-reduce, which is what "auto" runs there. "1" / "0" force it on / off.
FUSE_GEMM_ALL_REDUCE = _os.environ.get("PICOTRON_FUSE_GEMM_AR", "auto")
# Column-parallel backward: all-reduce the input gradient on a side stream while the weight-gradient GEMM runs. Off by
# default: on a power-capped B200 a 7B-shape tensor-parallel step measured the same with and without it (383.6 vs 381.2 ms).
OVERLAP_DGRAD_ALL_REDUCE = _os.environ.get("PICOTRON_OVERLAP_DGRAD_AR", "0") != "0"
# thread blocks of the side-stream all-reduce: enough loads in flight for the link, few enough to leave the SMs to the GEMM
OVERLAP_ALL_REDUCE_BLOCKS = 32


class _Done:
    def wait(self):
        return None


class _StreamJoin:
    """Handle of work running on a side stream: ``wait()`` orders the current stream behind it."""

    def __init__(self, event):
        self.event = event

    def wait(self):
        torch.cuda.current_stream().wait_event(self.event)


_SIDE_STREAMS = {}


def _side_stream(device) -> "torch.cuda.Stream":
    key = torch.device(device).index
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = torch.cuda.Stream(device=device)
    return _SIDE_STREAMS[key]


def linear_dgrad_all_reduce_async(dy: torch.Tensor, w: torch.Tensor, group):
    """``(dx, handle)`` with ``dx = all_reduce(dy @ w)`` complete once ``handle.wait()`` has been called.

    The column-parallel backward of the reference all-reduces the input gradient and only then computes the weight
    gradient (``tp_communications.py:29-33``; its optional async variant, ``:74-101``, overlaps them with an NCCL
    request). Here the GEMM writes ``dx`` into a symmetric slot, the peer-memory all-reduce kernel runs on a side stream
    with a small grid, and the caller launches the weight-gradient GEMM on the main stream before it waits: the
    NVLink traffic hides behind tensor-core work. Without a workspace the NCCL request plays the same role.
    """
    if group is None or not dy.is_cuda or not OVERLAP_DGRAD_ALL_REDUCE:
        return linear_all_reduce(dy, w, group, dgrad=True), _Done()
    from ..comm import symmetric
    ws = symmetric.workspace_for(group)
    rows, cols = dy.shape[0], w.shape[1]
    out = ws.ring_alloc((rows, cols), dy.dtype) if ws is not None else None
    dx = ops.linear_dgrad(dy, w, out=out)
    if out is None:
        with nvtx_range("all_reduce/nccl_async"):
            return dx, dist.all_reduce(dx, group=group, async_op=True)
    main = torch.cuda.current_stream()
    side = _side_stream(dy.device)
    ready = torch.cuda.Event()
    ready.record(main)
    side.wait_event(ready)
    with torch.cuda.stream(side), nvtx_range("all_reduce/peer_memory_async"):
        ws.all_reduce_(dx, blocks=OVERLAP_ALL_REDUCE_BLOCKS)
        done = torch.cuda.Event()
        done.record(side)
    return dx, _StreamJoin(done)


# ---------------------------------------------------------------------------------------------------------------
# sequence parallelism (optional, ``distributed.sequence_parallel``): between the tensor-parallel regions of a layer
# (RMSNorm, residual adds, the pipeline messages) every rank of the TP group holds 1/tp of the micro-batch's tokens
# instead of a full replica. Column-parallel GEMMs then read ``all_gather(tokens)`` and row-parallel GEMMs end in a
# reduce-scatter instead of an all-reduce: the same bytes on the wire (an all-reduce IS a reduce-scatter followed by an
# all-gather), 1/tp of the activation memory and of the normalisation work. The reference has no such mode (it names
# it as a TODO, ``utils.py:67``). Tokens are split as contiguous rows of the flattened ``[B * S, H]`` activation.
# ---------------------------------------------------------------------------------------------------------------
SEQUENCE_PARALLEL = False


def sequence_parallel_group():
    """The tensor-parallel group when sequence parallelism is on for this grid, else None."""
    if not SEQUENCE_PARALLEL:
        return None
    g = pgm.get()
    return g.tp_group if g.tp_world_size > 1 else None


def gather_tokens(x: torch.Tensor, group) -> torch.Tensor:
    """``[T / n, ...]`` on every rank -> ``[T, ...]``: the ranks' row blocks in rank order."""
    n = dist.get_world_size(group)
    x = x.contiguous()
    out = torch.empty((x.shape[0] * n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    with nvtx_range("sp/all_gather"):
        dist.all_gather_into_tensor(out, x, group=group)
    return out


def reduce_scatter_tokens(x: torch.Tensor, group) -> torch.Tensor:
    """``[T, ...]`` partial sums on every rank -> this rank's ``[T / n, ...]`` row block of their sum."""
    n, r = dist.get_world_size(group), dist.get_rank(group)
    assert x.shape[0] % n == 0, f"{x.shape[0]} tokens do not split over {n} ranks"
    rows = x.shape[0] // n
    x = x.contiguous()
    with nvtx_range("sp/reduce_scatter"):
        if x.is_cuda:
            out = torch.empty((rows,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
            dist.reduce_scatter_tensor(out, x, group=group)
            return out
        dist.all_reduce(x, group=group)                   # Gloo has no reduce-scatter: reduce everything, keep one block
        return x[r * rows:(r + 1) * rows].clone()


class GatherTokens(torch.autograd.Function):
    """All-gather of the token blocks; the gradient arriving at the gathered tensor must already be summed over the
    group (as the LM head's input gradient is), so the backward pass keeps this rank's rows."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return gather_tokens(x, group)

    @staticmethod
    def backward(ctx, grad):
        n, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        rows = grad.shape[0] // n
        return grad[r * rows:(r + 1) * rows].contiguous(), None


class ReduceScatterTokens(torch.autograd.Function):
    """Sum over the group, keep this rank's token block; backward = all-gather of the blocks' gradients."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return reduce_scatter_tokens(x, group)

    @staticmethod
    def backward(ctx, grad):
        return gather_tokens(grad, ctx.group), None


def sync_sequence_parallel_grads(model) -> None:
    """Sum the gradients of the token-wise replicated parameters (the RMSNorm weights) over the tensor-parallel group.

    With sequence parallelism a rank normalises only its own tokens, so its norm-weight gradient is a partial sum. Call
    once per optimizer step after the last backward pass; one small all-reduce (``(2 L + 1) H`` values).
    """
    group = sequence_parallel_group()
    if group is None:
        return
    grads = []
    for name, p in model.named_parameters():
        if p.requires_grad and p.dim() == 1:                # the only vectors of the model are the norm weights
            g_ = getattr(p, "main_grad", None)
            g_ = g_ if g_ is not None else p.grad
            if g_ is not None:
                grads.append(g_)
    if not grads:
        return
    flat = torch.cat([g_.reshape(-1).float() for g_ in grads])
    dist.all_reduce(flat, group=group)
    off = 0
    for g_ in grads:
        g_.copy_(flat[off:off + g_.numel()].view_as(g_))
        off += g_.numel()


def merge_first_two_dims(grad_output: torch.Tensor, input_: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    return (grad_output.contiguous().view(-1, grad_output.shape[-1]),
            input_.contiguous().view(-1, input_.shape[-1]))


def split_tensor_along_last_dim(tensor: torch.Tensor, num_partitions: int):
    last = tensor.dim() - 1
    assert tensor.size(last) % num_partitions == 0, f"{tensor.size(last)} is not divisible by {num_partitions}"
    return torch.split(tensor, tensor.size(last) // num_partitions, dim=last)


def _tp():
    g = pgm.get()
    return (g.tp_group if g.tp_world_size > 1 else None), g.tp_world_size, g.tp_rank


class CopyToModelParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x

    @staticmethod
    def backward(ctx, grad_output):
        group, n, _ = _tp()
        if n == 1:
            return grad_output
        grad_output = grad_output.contiguous()
        all_reduce_(grad_output, group)
        return grad_output


class ReduceFromModelParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        group, n, _ = _tp()
        if n == 1:
            return x
        ctx.mark_dirty(x)
        all_reduce_(x, group)
        return x

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output


class GatherFromModelParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        group, n, rank = _tp()
        if n == 1:
            return x
        x = x.contiguous()
        parts = [torch.empty_like(x) for _ in range(n)]
        dist.all_gather(parts, x, group=group)
        parts[rank] = x
        return torch.cat(parts, dim=-1).contiguous()

    @staticmethod
    def backward(ctx, grad_output):
        group, n, rank = _tp()
        if n == 1:
            return grad_output
        return split_tensor_along_last_dim(grad_output, n)[rank].contiguous()


class LinearWithAllReduce(torch.autograd.Function):
    """Column-parallel linear: ``y_i = x W_i^T`` forward; backward all-reduces grad-input after both GEMMs."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        ctx.use_bias = bias is not None
        y = ops.linear_fwd(x.reshape(-1, x.shape[-1]), weight).view(*x.shape[:-1], weight.shape[0])
        return y + bias if bias is not None else y

    @staticmethod
    def backward(ctx, grad_output):
        x, weight = ctx.saved_tensors
        group, n, _ = _tp()
        go, xi = merge_first_two_dims(grad_output, x)
        grad_input = ops.linear_dgrad(go, weight).view_as(x)
        grad_weight = ops.linear_wgrad(go, xi)
        grad_bias = go.sum(0) if ctx.use_bias else None
        if n > 1:
            all_reduce_(grad_input, group)
        return grad_input, grad_weight, grad_bias


class LinearWithAsyncAllReduce(torch.autograd.Function):
    """Same maths; the grad-input all-reduce is issued before the grad-weight GEMM and waited after it."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        return LinearWithAllReduce.forward(ctx, x, weight, bias)

    @staticmethod
    def backward(ctx, grad_output):
        x, weight = ctx.saved_tensors
        group, n, _ = _tp()
        go, xi = merge_first_two_dims(grad_output, x)
        grad_input = ops.linear_dgrad(go, weight).view_as(x)
        handle = dist.all_reduce(grad_input, group=group, async_op=True) if n > 1 else None
        grad_weight = ops.linear_wgrad(go, xi)
        grad_bias = go.sum(0) if ctx.use_bias else None
        if handle is not None:
            handle.wait()
        return grad_input, grad_weight, grad_bias


def linear_with_all_reduce(x, weight, bias):
    return LinearWithAllReduce.apply(x, weight, bias)


def linear_with_async_all_reduce(x, weight, bias):
    return LinearWithAsyncAllReduce.apply(x, weight, bias)
