"""Weight tying of the token embedding and the LM head (``model.tie_word_embeddings``; off by default).

The reference never ties: it always creates a separate, randomly initialised LM head, also for models whose published
checkpoints share the two matrices such as SmolLM and Llama-3.2-1B (``checkpoint.py:89-102``, ``model.py:271-273``). This
module adds the tied form as an option:

* one pipeline stage (``pp_size == 1``): the head module's ``weight`` IS the embedding's parameter. Under tensor
  parallelism both modules hold the same rows ``[v0, v1)`` of the vocabulary (``VocabParallelEmbedding`` and the
  column-parallel head split the same dimension the same way), so the shards tie rank by rank. Both layers add their
  weight gradient into the same fp32 bucket slice; the data-parallel engine is told that the slice is complete after the
  second contribution (``_grad_uses``).
* several stages: the first stage keeps the embedding and the last stage the head, as two parameters that are made equal
  at start (the last stage receives the first stage's values) and are kept equal by adding their gradients over the
  2-rank group {first stage, last stage} before every optimizer step. Both ranks then apply the same update to the same
  values with the same optimizer state, so the copies never drift.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import process_group_manager as pgm


def _raw(model):
    while hasattr(model, "module") and hasattr(model, "require_backward_grad_sync"):
        model = model.module
    return model


def _weight_of(module) -> Optional[nn.Parameter]:
    return None if isinstance(module, nn.Identity) else module.weight


def tie_word_embeddings(model) -> None:
    """Tie ``model.final_proj.weight`` to ``model.embedding.weight``. Collective when ``pp_size > 1``: every rank calls it.

    Call after the parameters have real storage and before the data-parallel wrapper and the optimizer are built.
    """
    g = pgm.get()
    raw = _raw(model)
    emb, head = _weight_of(raw.embedding), _weight_of(raw.final_proj)
    if g.pp_world_size == 1:
        assert emb.shape == head.shape, f"embedding {tuple(emb.shape)} and LM head {tuple(head.shape)} cannot be tied"
        raw.final_proj.weight = emb                     # nn.Module.__setattr__ re-registers the parameter
        emb._grad_uses = 2
        raw._tied_embedding = (emb, None)
        return
    group = g.pp_ends_group()
    if group is None:                                   # middle stage: took part in creating the groups, holds no copy
        raw._tied_embedding = None
        return
    w = emb if g.pp_is_first_stage else head
    src = g.pp_ends_group_ids[0]
    with torch.no_grad():
        dist.broadcast(w.data, src=src, group=group)
    raw._tied_embedding = (w, group)


def sync_tied_embedding_grads(model) -> None:
    """Add the gradients of the two copies of a tied weight (first and last pipeline stage). Call once per optimizer step,
    after the step's last backward and the data-parallel reduction, before the update. No-op when nothing is tied or
    when one rank holds both uses."""
    tied = getattr(_raw(model), "_tied_embedding", None)
    if not tied or tied[1] is None:
        return
    w, group = tied
    grad = getattr(w, "main_grad", None)
    if grad is None:
        grad = w.grad
    assert grad is not None, "the tied weight has no gradient: was the backward pass run?"
    dist.all_reduce(grad, op=dist.ReduceOp.SUM, group=group)
