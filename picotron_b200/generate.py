"""Greedy decoding with the training model, for checking what a (pre)trained checkpoint says.

The reference has no inference path. This one reuses the training forward pass as it is: the prompt sits at the start
of a fixed ``[B, length]`` buffer, every step runs the whole buffer through the model and reads the logits at the last
filled position. The causal mask makes whatever follows that position irrelevant, so the buffer's tail may hold
anything; shapes never change (the same kernels and tile sizes as in training, CUDA-graph friendly) at the price of
``O(length)`` work per token instead of a key/value cache. Meant for a few hundred tokens of sanity checking, not for
serving. Works under tensor parallelism (the LM head gathers the logits); a pipeline-parallel model is not supported.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import process_group_manager as pgm


@torch.no_grad()
def greedy_generate(model, input_ids: torch.Tensor, max_new_tokens: int, length: Optional[int] = None,
                    eos_token_id: Optional[int] = None, pad_token_id: int = 0) -> torch.Tensor:
    """``input_ids`` ``[B, P]`` -> ``[B, P + n]`` with ``n <= max_new_tokens`` greedily chosen tokens appended.

    ``length`` is the size of the working buffer (default: the model's ``max_position_embeddings``); prompt plus new
    tokens must fit. Sequences that produced ``eos_token_id`` keep emitting ``pad_token_id``; decoding stops early
    once all have.
    """
    assert pgm.get().pp_world_size == 1, "greedy_generate runs the whole model on every rank: no pipeline parallelism"
    raw = model
    while hasattr(raw, "module") and hasattr(raw, "require_backward_grad_sync"):
        raw = raw.module
    B, P = input_ids.shape
    L = int(length or raw.max_position_embeddings)
    assert P >= 1 and P + max_new_tokens <= L <= raw.max_position_embeddings, \
        f"prompt ({P}) + new tokens ({max_new_tokens}) must fit the buffer ({L} <= {raw.max_position_embeddings})"
    buf = torch.full((B, L), pad_token_id, dtype=input_ids.dtype, device=input_ids.device)
    buf[:, :P] = input_ids
    done = torch.zeros(B, dtype=torch.bool, device=input_ids.device)
    end = P
    for t in range(P, P + max_new_tokens):
        logits = model(input_ids=buf)                        # [B, L, V]; position t - 1 sees tokens 0 .. t - 1 only
        nxt = logits[:, t - 1].float().argmax(dim=-1)
        if eos_token_id is not None:
            nxt = torch.where(done, torch.full_like(nxt, pad_token_id), nxt)
            done |= nxt == eos_token_id
        buf[:, t] = nxt
        end = t + 1
        if eos_token_id is not None and bool(done.all()):
            break
    return buf[:, :end]
