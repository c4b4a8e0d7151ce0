"""Switches the parallel modules from NCCL collectives to the peer-memory kernels of this package.

Data parallel: the fp32 gradient buckets are carved out of one symmetric allocation shared by the CP x DP group;
when the last parameter of a bucket is ready, ONE kernel on a side stream averages the bucket in place across
ranks (``1/n`` scale fused) while the backward pass continues on the main stream.

Tensor parallel: a ring of symmetric slots receives the outputs of row-parallel GEMMs and the input gradients
of column-parallel GEMMs; ``tp_communications.all_reduce_`` reduces them in place.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import process_group_manager as pgm
from . import symmetric
from .workspace import SymmetricWorkspace, try_create


# staging area of the gradient workspace for the push all-reduce (buckets larger than what fits are reduced in pieces)
GRAD_STAGING_BYTES = 64 << 20


# scratch area of the tensor-parallel workspace (two halves of 3 fp32 vectors of one cross-entropy chunk each)
TP_SCRATCH_BYTES = 128 << 10


def share_vocab_parallel_embedding(model, tp_group) -> bool:
    """Move the weight shard of the vocabulary-parallel embedding (first pipeline stage) into symmetric memory, so that the
    lookup can read each token's row from the rank that owns it instead of all-reducing ``[tokens, hidden]`` partial results
    (``tensor_parallel.py:246-270`` of the reference masks, looks up, zeroes and all-reduces). Collective over ``tp_group``."""
    from ..parallel.tensor_parallel import VocabParallelEmbedding
    emb = next((m for m in model.modules() if isinstance(m, VocabParallelEmbedding)), None)
    has = torch.tensor([1 if emb is not None and emb.weight.is_cuda and emb.weight.dtype == torch.bfloat16 else 0],
                       device=torch.device("cuda", torch.cuda.current_device()))
    dist.all_reduce(has, op=dist.ReduceOp.MIN, group=tp_group)       # the ranks of a TP group are on the same stage
    if int(has.item()) == 0:
        return False
    w = emb.weight
    ws = try_create(tp_group, (w.numel() * 2 + 255) // 256 * 256, num_blocks=1)
    if ws is None:
        return False
    shared = ws.view(0, tuple(w.shape), torch.bfloat16)
    with torch.no_grad():
        shared.copy_(w.data)
        w.data = shared                                              # the Parameter object (and its name) stay
    emb.shared_workspace = ws
    return True


class _StreamHandle:
    def __init__(self, event: torch.cuda.Event):
        self.event = event

    def wait(self):
        torch.cuda.current_stream().wait_event(self.event)


class FusedBucketReducer:
    """``Bucket.reduce_fn``: in-place averaging of a bucket that lives in a symmetric workspace."""

    def __init__(self, ws: SymmetricWorkspace):
        self.ws = ws
        self.stream = torch.cuda.Stream()

    def __call__(self, bucket):
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream())
        self.stream.wait_event(ready)
        with torch.cuda.stream(self.stream):
            self.ws.all_reduce_(bucket.grad_data, scale=1.0 / bucket.process_group_size)
            done = torch.cuda.Event()
            done.record(self.stream)
        return _StreamHandle(done)


def grad_buffer_factory(group):
    """Returns ``factory(numel) -> fp32 flat tensor`` placing the gradient buckets in symmetric memory, or None."""
    if group is None or dist.get_world_size(group) == 1:
        return None
    state = {}

    def factory(numel: int) -> Optional[torch.Tensor]:
        ws = try_create(group, numel * 4, num_blocks=48, staging_bytes=GRAD_STAGING_BYTES)
        if ws is None:
            return None
        state["ws"] = ws
        symmetric.register(("grad", id(group)), ws)
        return ws.view(0, (numel,), torch.float32)

    factory.state = state
    return factory


def enable_fused_collectives(model, max_tokens: int = 0, hidden: int = 0) -> bool:
    """Attach workspaces to the groups ``model`` communicates on. Returns True when any fused path is active."""
    g = pgm.get()
    active = False
    bm = getattr(model, "bucket_manager", None)
    if bm is not None and getattr(bm, "symmetric_workspace", None) is not None:
        bm.set_reduce_fn(FusedBucketReducer(bm.symmetric_workspace))
        active = True
    if g.tp_world_size > 1 and max_tokens > 0 and hidden > 0:
        slot = (max_tokens * hidden * 2 + 255) // 256 * 256
        ws = try_create(g.tp_group, 4 * slot + TP_SCRATCH_BYTES, num_blocks=128, staging_bytes=slot)
        if ws is not None:
            ws.configure_ring(4, slot)
            ws.configure_scratch(4 * slot, TP_SCRATCH_BYTES)          # cross-entropy statistics of the vocab-parallel head
            symmetric.register(g.tp_group, ws)
            active = True
            share_vocab_parallel_embedding(model, g.tp_group)
    return active
