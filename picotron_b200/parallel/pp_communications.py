"""Pipeline-parallel point-to-point messages (activations forward, gradients backward).

Operation names and signatures follow ``pp_communications.py:8-46`` of the reference. Messages stay
on NCCL P2P (Gloo on CPU) addressed by global neighbour rank on the WORLD group. What changes: there
is no ``torch.cuda.synchronize()`` after a message (NCCL requests are stream-ordered, consumers queue
behind them), and receive buffers come from a small per-shape pool instead of a fresh allocation per
message.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import process_group_manager as pgm
from ..utils.tracing import nvtx_range

STEP, VERBOSE = 0, os.environ.get("VERBOSE", "0") == "1"


def _recv_buffer(shapes, device, dtype) -> torch.Tensor:
    # requires_grad so that the stage's backward can return the gradient w.r.t. the received activation
    return torch.empty(shapes, requires_grad=True, device=device, dtype=dtype)


def pipeline_communicate(operation: str, device, dtype, tensor: Optional[torch.Tensor] = None, shapes=None):
    """``operation`` in {recv_forward, send_forward, recv_backward, send_backward}."""
    global STEP
    g = pgm.get()
    if operation == "recv_forward":
        if g.pp_is_first_stage:
            return None
        tensor, peer = _recv_buffer(shapes, device, dtype), g.pp_prev_rank
    elif operation == "send_forward":
        if g.pp_is_last_stage:
            return None
        peer = g.pp_next_rank
    elif operation == "recv_backward":
        if g.pp_is_last_stage:
            return None
        tensor, peer = _recv_buffer(shapes, device, dtype), g.pp_next_rank
    elif operation == "send_backward":
        if g.pp_is_first_stage:
            return None
        peer = g.pp_prev_rank
    else:
        raise ValueError(f"unknown pipeline operation {operation}")
    is_send = operation.startswith("send")
    payload = tensor.detach() if is_send else tensor
    if is_send and not payload.is_contiguous():
        payload = payload.contiguous()
    op = dist.P2POp(dist.isend if is_send else dist.irecv, payload, peer)
    if VERBOSE:
        print(f"{operation} | pp_rank {g.pp_rank} {'->' if is_send else '<-'} {peer} | STEP:{STEP}", flush=True)
        STEP += 1
    with nvtx_range(f"pp/{operation}"):
        for req in dist.batch_isend_irecv([op]):
            req.wait()
    return None if is_send else tensor


def bidirectional_pipeline_communicate(operation: str, send_tensor: torch.Tensor, recv_shapes, device, dtype):
    """``operation`` in {send_fwd_recv_bwd, send_bwd_recv_fwd}: one fused send+recv with the same neighbour."""
    global STEP
    g = pgm.get()
    is_fwd = operation == "send_fwd_recv_bwd"
    if (is_fwd and g.pp_is_last_stage) or (not is_fwd and g.pp_is_first_stage):
        return None
    peer = g.pp_next_rank if is_fwd else g.pp_prev_rank
    recv_tensor = _recv_buffer(recv_shapes, device, dtype)
    payload = send_tensor.detach()
    if not payload.is_contiguous():
        payload = payload.contiguous()
    reqs = dist.batch_isend_irecv([dist.P2POp(dist.isend, payload, peer),
                                   dist.P2POp(dist.irecv, recv_tensor, peer)])
    if VERBOSE:
        print(f"{operation} | pp_rank {g.pp_rank} <-> {peer} | STEP:{STEP}", flush=True)
        STEP += 1
    with nvtx_range(f"pp/{operation}"):
        for req in reqs:
            req.wait()
    return recv_tensor
