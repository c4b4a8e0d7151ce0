"""Pipeline-parallel point-to-point messages (activations forward, gradients backward).

The reference (``pp_communications.py:8-46``) sends every message as a one-element ``batch_isend_irecv`` on
the WORLD group, waits for it and then synchronises the whole device, with a fresh receive tensor per
message. Here the messages still travel over NCCL P2P (Gloo on CPU), but the engine is built so that
transfers overlap compute:

* **One communicator per neighbour and direction** (2-rank groups created by the process-group manager).
  A communicator only ever carries one ordered stream of messages (activations of micro-batch 0, 1, ...
  or gradients of micro-batch 0, 1, ...), so a receive can be posted long before its send exists without
  any risk of two ranks posting a send/recv pair in opposite orders, and the forward and backward
  directions never queue behind each other.
* **Receives can be posted ahead** (``POST_AHEAD``): the schedules call ``post_recv_*`` for micro-batch ``k+1`` before
  they launch the compute of micro-batch ``k``, from a dedicated stream that only waits for the event recorded when the
  receive buffer was last released. It is OFF by default: an NCCL receive is a kernel that stays resident and polls
  until its sender arrives, and with a whole micro-batch of compute running beside it that polling cost far more than
  the transfer it hides (a 7B-shape 2-stage step: 879 ms posted ahead, 719 ms posted when needed). By default
  a receive is therefore posted at the point where the schedule needs its data.
* **Sends never stall compute**: ``send_*`` makes the communicator's stream wait for the producer (an
  event on the compute stream) and returns; the compute stream does not wait for the peer. The request
  and the tensor are kept until ``drain()`` / a later send retires them.
* **Receive buffers come from a per-(shape, dtype) pool** and return to it after the backward pass that
  consumed them, together with an event that orders their reuse.

``pipeline_communicate`` / ``bidirectional_pipeline_communicate`` keep the reference's names, arguments and
blocking-on-the-stream semantics on top of the same channels (no device-wide synchronisation).
"""
from __future__ import annotations

import collections
import contextlib
import os
from typing import Deque, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import process_group_manager as pgm
from ..utils.tracing import nvtx_range

STEP, VERBOSE = 0, os.environ.get("VERBOSE", "0") == "1"

# how many finished sends may stay un-retired before the oldest is waited for (bounds the memory they pin)
MAX_PENDING_SENDS = 4
# Post receives one micro-batch ahead (True, PICOTRON_PP_POST_AHEAD=1) or only when their data is needed (False). An NCCL
# receive is a kernel that stays resident and polls until the sender shows up, so a receive posted ahead shares SMs with the
# compute of a whole micro-batch; which of the two costs less is a measurement, not a given.
# Measured on 2 B200s, Llama-2-7B shape, 8 layers per stage, 16 micro-batches: 879 ms per step with receives posted ahead,
# 719 ms with receives posted when needed (the backward of a stage's micro-batch 161 -> 114 ms). Default: not ahead.
POST_AHEAD = os.environ.get("PICOTRON_PP_POST_AHEAD", "0") != "0"


class RecvPool:
    """Free lists of receive buffers keyed by (shape, dtype, device).

    A buffer is handed out as an autograd leaf (``requires_grad=True``) because the stage's backward pass returns the
    gradient with respect to the received activation. ``release`` takes it back together with an event recorded on the
    stream that last read it; ``acquire`` returns that event so the next writer can order itself behind it.
    """

    def __init__(self):
        self._free: Dict[Tuple, List[Tuple[torch.Tensor, Optional[object]]]] = collections.defaultdict(list)
        self.allocated = 0

    @staticmethod
    def _key(shape, dtype, device):
        return (tuple(shape), dtype, str(device))

    def acquire(self, shape, dtype, device):
        free = self._free[self._key(shape, dtype, device)]
        if free:
            return free.pop()
        self.allocated += 1
        return torch.empty(tuple(shape), requires_grad=True, device=device, dtype=dtype), None

    def release(self, tensor: torch.Tensor) -> None:
        tensor.grad = None
        event = None
        if tensor.is_cuda:
            event = torch.cuda.Event()
            event.record(torch.cuda.current_stream(tensor.device))
        self._free[self._key(tensor.shape, tensor.dtype, tensor.device)].append((tensor, event))


class _PostedRecv:
    __slots__ = ("tensor", "work")

    def __init__(self, tensor, work):
        self.tensor, self.work = tensor, work


class PipelineP2P:
    """The four message streams of this pipeline stage (recv/send x forward/backward) with posted-ahead receives."""

    def __init__(self):
        g = pgm.get()
        self.g = g
        self.pool = RecvPool()
        self._posted: Dict[str, Deque[_PostedRecv]] = {"fwd": collections.deque(), "bwd": collections.deque()}
        self._sends: Deque[Tuple[object, torch.Tensor]] = collections.deque()
        self._post_stream = None
        self._connect()

    def _connect(self) -> None:
        """One tiny message on every channel, in the same order on every stage (previous neighbour first).

        NCCL sets a point-to-point connection up on first use, and that set-up blocks the host until the peer issues its
        first operation on the same communicator. Receives that are posted ahead would turn this into a cycle (stage 0
        posting its first gradient receive while stage 1 is still posting its first activation receive), so the
        connections are made here, where every stage walks its channels in an order that resolves stage by stage.
        """
        g = self.g
        if g.pp_world_size == 1 or not (dist.is_available() and dist.is_initialized()):
            return
        on_gpu = dist.get_backend() == "nccl"
        dev = torch.device("cuda", torch.cuda.current_device()) if on_gpu else torch.device("cpu")
        token = torch.zeros(1, dtype=torch.float32, device=dev)
        for kind in ("recv_fwd", "send_bwd", "send_fwd", "recv_bwd"):
            group, peer = self._channel(kind)
            if peer is None:
                continue
            (dist.recv(token, src=peer, group=group) if kind.startswith("recv")
             else dist.send(token, dst=peer, group=group))
        if on_gpu:
            torch.cuda.synchronize()

    # ------------------------------------------------------------------ plumbing
    def _channel(self, kind: str):
        """(process group or None for WORLD, peer global rank) of ``kind`` in {recv_fwd, send_fwd, recv_bwd, send_bwd}."""
        g = self.g
        groups = getattr(g, "pp_channel_groups", None) or {}
        peer = g.pp_prev_rank if kind in ("recv_fwd", "send_bwd") else g.pp_next_rank
        return groups.get(kind), peer

    @contextlib.contextmanager
    def _posting(self, device, after_event):
        """Stream context for posting a receive: a side stream that waits only for the buffer's release event."""
        if torch.device(device).type != "cuda":
            yield
            return
        if self._post_stream is None:
            self._post_stream = torch.cuda.Stream(device=device)
        if after_event is not None:
            self._post_stream.wait_event(after_event)
        else:
            # a buffer fresh from the caching allocator may reuse memory that work already queued on the current stream
            # still reads: order the first write behind everything queued so far
            self._post_stream.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(self._post_stream):
            yield

    def _has(self, direction: str) -> bool:
        g = self.g
        return not (g.pp_is_first_stage if direction == "fwd" else g.pp_is_last_stage)

    # ------------------------------------------------------------------ receives
    def post_recv(self, direction: str, shapes, device, dtype) -> None:
        """Post the receive of the next forward activation / backward gradient (no-op on the edge stage)."""
        if not self._has(direction) or not POST_AHEAD:
            return
        self._post(direction, shapes, device, dtype)

    def _post(self, direction: str, shapes, device, dtype) -> None:
        group, peer = self._channel("recv_" + direction)
        tensor, released = self.pool.acquire(shapes, dtype, device)
        with self._posting(device, released), nvtx_range(f"pp/post_recv_{direction}"):
            work = dist.irecv(tensor, src=peer, group=group)
        self._posted[direction].append(_PostedRecv(tensor, work))
        _log(f"post_recv_{direction}", self.g, peer, "<-")

    def wait_recv(self, direction: str, shapes, device, dtype) -> Optional[torch.Tensor]:
        """The oldest posted receive of ``direction`` (posting one now if none is outstanding); later work on the current
        stream is ordered behind the transfer. Returns None on the edge stage."""
        if not self._has(direction):
            return None
        if not self._posted[direction]:
            self._post(direction, shapes, device, dtype)
        posted = self._posted[direction].popleft()
        with nvtx_range(f"pp/wait_recv_{direction}"):
            posted.work.wait()
        return posted.tensor

    def release(self, *tensors: Optional[torch.Tensor]) -> None:
        """Give receive buffers back once the work that reads them has been enqueued on the current stream."""
        for t in tensors:
            if t is not None:
                self.pool.release(t)

    # ------------------------------------------------------------------ sends
    def send(self, direction: str, tensor: Optional[torch.Tensor]) -> None:
        """Send an activation to the next stage (``fwd``) or a gradient to the previous one (``bwd``) without making the
        current stream wait for the peer. No-op on the edge stage."""
        g = self.g
        if (direction == "fwd" and g.pp_is_last_stage) or (direction == "bwd" and g.pp_is_first_stage):
            return
        group, peer = self._channel("send_" + direction)
        payload = tensor.detach()
        if not payload.is_contiguous():
            payload = payload.contiguous()
        with nvtx_range(f"pp/send_{direction}"):
            work = dist.isend(payload, dst=peer, group=group)
        self._sends.append((work, payload))
        _log(f"send_{direction}", g, peer, "->")
        while len(self._sends) > MAX_PENDING_SENDS:
            self._sends.popleft()[0].wait()

    def drain(self) -> None:
        """Retire every outstanding send (end of a step)."""
        while self._sends:
            self._sends.popleft()[0].wait()
        assert not self._posted["fwd"] and not self._posted["bwd"], "a posted pipeline receive was never consumed"


_P2P: Optional[PipelineP2P] = None


def get_p2p() -> PipelineP2P:
    """The message engine of the active process grid (rebuilt when the grid changes)."""
    global _P2P
    if _P2P is None or _P2P.g is not pgm.get():
        _P2P = PipelineP2P()
    return _P2P


def _log(op, g, peer, arrow):
    global STEP
    if VERBOSE:
        print(f"{op} | pp_rank {g.pp_rank} {arrow} {peer} | STEP:{STEP}", flush=True)
        STEP += 1


# ---------------------------------------------------------------------------------------------------------------
# reference-shaped entry points (one message per call, ordered on the current stream)
# ---------------------------------------------------------------------------------------------------------------
def pipeline_communicate(operation: str, device, dtype, tensor: Optional[torch.Tensor] = None, shapes=None):
    """``operation`` in {recv_forward, send_forward, recv_backward, send_backward}."""
    p2p = get_p2p()
    if operation == "recv_forward":
        return p2p.wait_recv("fwd", shapes, device, dtype)
    if operation == "recv_backward":
        return p2p.wait_recv("bwd", shapes, device, dtype)
    if operation == "send_forward":
        p2p.send("fwd", tensor)
        return None
    if operation == "send_backward":
        p2p.send("bwd", tensor)
        return None
    raise ValueError(f"unknown pipeline operation {operation}")


def bidirectional_pipeline_communicate(operation: str, send_tensor: torch.Tensor, recv_shapes, device, dtype):
    """``operation`` in {send_fwd_recv_bwd, send_bwd_recv_fwd}: a send and the matching receive from the same neighbour."""
    p2p = get_p2p()
    if operation == "send_fwd_recv_bwd":
        if p2p.g.pp_is_last_stage:
            return None
        p2p.send("fwd", send_tensor)
        return p2p.wait_recv("bwd", recv_shapes, device, dtype)
    if operation == "send_bwd_recv_fwd":
        if p2p.g.pp_is_first_stage:
            return None
        p2p.send("bwd", send_tensor)
        return p2p.wait_recv("fwd", recv_shapes, device, dtype)
    raise ValueError(f"unknown pipeline operation {operation}")
