"""Pipeline parallelism: stage wrapper plus the AFAB and 1F1B schedules.

Stage construction, layer distribution (contiguous blocks, remainder to the first stages), the
``forward``/``backward`` stage interface and both schedules follow ``pipeline_parallel.py:8-222`` of the
reference, including its rule for data-parallel gradient synchronisation (enabled only for the
stage's truly last backward of the step).

Differences: the last stage computes the loss with the fused LM-head + cross-entropy node (no
``[B,S,V]`` logits), the running loss stays on the device and is read once per step, and the stage-to-stage
messages overlap compute (receives posted one micro-batch ahead, sends that do not stall the compute stream,
pooled receive buffers; :mod:`.pp_communications`) instead of being followed by a device-wide synchronisation. The loss of every micro-batch is divided by the number
of micro-batches before the backward pass (the reference divides only the logged value, so its PP
gradients are ``grad_acc_steps`` times larger than its non-PP gradients); set
``REFERENCE_LOSS_SCALING = True`` to reproduce the reference for oracle comparisons.
"""
from __future__ import annotations

from typing import List

import torch
import torch.nn as nn

from .. import process_group_manager as pgm
from ..models.llama import gather_tokens_for_head, lm_head_loss
from .pp_communications import get_p2p
from ..utils.tracing import nvtx_range, timed_phase

REFERENCE_LOSS_SCALING = False


def balanced_layer_split(config, pp_size: int) -> List[int]:
    """Layers per stage that minimise the slowest stage when the LM head is counted as work of the last stage.

    The reference gives every stage the same number of layers (``pipeline_parallel.py:42-51``), so the last stage, which
    also runs the final norm, the ``[hidden, vocab]`` projection and the loss, sets the pace of the pipeline: with a
    128K vocabulary the head of an 8B model costs about three decoder layers. Cost model: matmul FLOPs per token, a decoder
    layer = its parameters plus the attention term, the head = ``vocab * hidden`` (the embedding lookup is free).
    """
    h, i, v = config.hidden_size, config.intermediate_size, config.vocab_size
    kv = config.num_key_value_heads * (h // config.num_attention_heads)
    layer = 2 * h * h + 2 * h * kv + 3 * h * i + 2 * h * config.max_position_embeddings
    head = v * h
    n = config.num_hidden_layers
    total = n * layer + head
    per = [0] * pp_size
    # fill the stages front to back up to the average; the last stage takes what is left (at least one layer each)
    left = n
    for s in range(pp_size - 1):
        want = round(total / pp_size / layer)
        want = max(1, min(want, left - (pp_size - 1 - s)))
        per[s] = want
        left -= want
    per[-1] = left
    # the greedy fill can leave the last stage over the average: move single layers while that lowers the maximum
    cost = lambda k, s: k * layer + (head if s == pp_size - 1 else 0)
    improved = True
    while improved:
        improved = False
        worst = max(range(pp_size), key=lambda s: cost(per[s], s))
        for s in range(pp_size):
            if s != worst and per[worst] > 1 and max(cost(per[worst] - 1, worst), cost(per[s] + 1, s)) < cost(per[worst], worst):
                per[worst] -= 1
                per[s] += 1
                improved = True
                break
    return per


# "reference": equal split, remainder to the first stages; "balanced": `balanced_layer_split`; or an explicit list of layer
# counts per stage. Set from `distributed.pp_layer_split` by the trainer before the stages are built.
LAYER_SPLIT = "reference"


class PipelineParallel(nn.Module):
    def __init__(self, model, config):
        super().__init__()
        g = pgm.get()
        self.layer_distribution = self.distribute_layers(config.num_hidden_layers, config)
        self.embedding = model.embedding if g.pp_is_first_stage else nn.Identity()
        self.decoder_layers = nn.ModuleDict({str(i): model.decoder_layers[i] for i in self.layer_distribution})
        self.final_norm = model.final_norm if g.pp_is_last_stage else nn.Identity()
        self.final_proj = model.final_proj if g.pp_is_last_stage else nn.Identity()
        self.ce_chunk_tokens = getattr(model, "ce_chunk_tokens", 2048)
        self.init = getattr(model, "init", "reference")
        self.model_config = config
        self.reset_parameters()

    def reset_parameters(self):
        g = pgm.get()
        init = self.init

        def _reset(m):
            try:
                m.reset_parameters(init)
            except TypeError:
                m.reset_parameters()
        if g.pp_is_first_stage:
            _reset(self.embedding)
        for layer in self.decoder_layers.values():
            layer.input_layernorm.reset_parameters()
            layer.attention.reset_parameters(init)
            layer.post_attention_layernorm.reset_parameters()
            layer.mlp.reset_parameters(init)
        if g.pp_is_last_stage:
            self.final_norm.reset_parameters()
            _reset(self.final_proj)

    def packed_param_groups(self):
        return [grp for layer in self.decoder_layers.values() for grp in layer.packed_param_groups()]

    @staticmethod
    def distribute_layers(num_layers: int, config=None) -> List[int]:
        g = pgm.get()
        n, r = g.pp_world_size, g.pp_rank
        if isinstance(LAYER_SPLIT, (list, tuple)):
            per = [int(x) for x in LAYER_SPLIT]
            assert len(per) == n and sum(per) == num_layers and min(per) >= 1, \
                f"pp_layer_split {per} does not distribute {num_layers} layers over {n} stages"
        elif LAYER_SPLIT == "balanced" and config is not None and n > 1:
            per = balanced_layer_split(config, n)
        else:
            per = [num_layers // n + (1 if i < num_layers % n else 0) for i in range(n)]
        start = sum(per[:r])
        return list(range(start, start + per[r]))

    def forward(self, input_ids, position_ids=None, hidden_states=None, target_ids=None, loss_scale: float = 1.0):
        x = hidden_states if hidden_states is not None else input_ids
        x = self.embedding(x)
        for layer in self.decoder_layers.values():
            x = layer(x, position_ids=position_ids)
        x = self.final_norm(x)
        if pgm.get().pp_is_last_stage:
            x = gather_tokens_for_head(x)
        if target_ids is not None and pgm.get().pp_is_last_stage:
            return lm_head_loss(x, self.final_proj, target_ids, loss_scale, self.ce_chunk_tokens)
        return self.final_proj(x)

    def backward(self, input_tensor, output_tensor, output_tensor_grad):
        if input_tensor is not None:
            input_tensor.retain_grad()
        if output_tensor_grad is None:
            output_tensor_grad = torch.ones_like(output_tensor, memory_format=torch.preserve_format)
        torch.autograd.backward(output_tensor, grad_tensors=output_tensor_grad, retain_graph=False, create_graph=False)
        return input_tensor.grad if input_tensor is not None else None


def _stage_forward(model, data_loader, input_tensor, device, loss_acc):
    """One micro-batch forward on this stage; the last stage returns the (scaled) loss tensor."""
    g = pgm.get()
    batch = next(data_loader)
    n_mb = data_loader.grad_acc_steps
    hidden = input_tensor.to(device) if input_tensor is not None else None
    kwargs = {}
    if g.pp_is_last_stage:
        kwargs = dict(target_ids=batch["target_ids"].to(device, non_blocking=True),
                      loss_scale=1.0 if REFERENCE_LOSS_SCALING else 1.0 / n_mb)
    out = model.forward(input_ids=batch["input_ids"].to(device, non_blocking=True),
                        position_ids=batch["position_ids"].to(device, non_blocking=True) if batch.get("position_ids") is not None else None,
                        hidden_states=hidden, **kwargs)
    if g.pp_is_last_stage:
        loss_acc.add_(out.detach() * (1.0 / n_mb if REFERENCE_LOSS_SCALING else 1.0))
    return out


def train_step_pipeline_afab(model, data_loader, tensor_shapes, device, dtype):
    """All-forward-all-backward schedule (``pipeline_parallel.py:77-127``). Returns the mean loss (last stage).

    The receive of micro-batch ``k+1`` is posted before the compute of micro-batch ``k`` is launched and sends do not
    stall the compute stream (see :mod:`.pp_communications`).
    """
    g = pgm.get()
    p2p = get_p2p()
    n_mb = data_loader.grad_acc_steps
    loss_acc = torch.zeros((), dtype=torch.float32, device=device)
    input_tensors, output_tensors = [], []
    requires_grad_sync = g.cp_dp_world_size > 1 or hasattr(model, "require_backward_grad_sync")
    args = dict(shapes=tensor_shapes, device=device, dtype=dtype)

    with nvtx_range("afab/all_forward"):
        p2p.post_recv("fwd", **args)
        for i in range(n_mb):
            input_tensor = p2p.wait_recv("fwd", **args)
            if i + 1 < n_mb:
                p2p.post_recv("fwd", **args)
            output_tensor = _stage_forward(model, data_loader, input_tensor, device, loss_acc)
            p2p.send("fwd", output_tensor)
            input_tensors.append(input_tensor)
            output_tensors.append(output_tensor)

    with nvtx_range("afab/all_backward"):
        p2p.post_recv("bwd", **args)
        for i in range(n_mb):
            if requires_grad_sync:
                model.require_backward_grad_sync = i == n_mb - 1
            output_tensor_grad = p2p.wait_recv("bwd", **args)
            if i + 1 < n_mb:
                p2p.post_recv("bwd", **args)
            input_tensor, output_tensor = input_tensors.pop(0), output_tensors.pop(0)
            input_tensor_grad = model.backward(input_tensor, output_tensor, output_tensor_grad)
            p2p.send("bwd", input_tensor_grad)
            p2p.release(input_tensor, output_tensor_grad)

    p2p.drain()
    return loss_acc.item() if g.pp_is_last_stage else 0.0


@torch.no_grad()
def evaluate_pipeline(model, data_loader, tensor_shapes, device, dtype) -> float:
    """Forward-only pass of ``data_loader.grad_acc_steps`` micro-batches through the stages: each stage receives, computes and
    sends on; nothing is kept for a backward pass and no gradient buffer is touched. Returns the mean loss (last stage)."""
    g = pgm.get()
    p2p = get_p2p()
    n_mb = data_loader.grad_acc_steps
    loss_acc = torch.zeros((), dtype=torch.float32, device=device)
    args = dict(shapes=tensor_shapes, device=device, dtype=dtype)
    for _ in range(n_mb):
        input_tensor = p2p.wait_recv("fwd", **args)
        batch = next(data_loader)
        kwargs = dict(target_ids=batch["target_ids"].to(device, non_blocking=True)) if g.pp_is_last_stage else {}
        out = model.forward(input_ids=batch["input_ids"].to(device, non_blocking=True), position_ids=None,
                            hidden_states=input_tensor, **kwargs)
        if g.pp_is_last_stage:
            loss_acc.add_(out.detach() / n_mb)
        p2p.send("fwd", out)
        p2p.release(input_tensor)
    p2p.drain()
    return loss_acc.item() if g.pp_is_last_stage else 0.0


def train_step_pipeline_1f1b(model, data_loader, tensor_shapes, device, dtype):
    """One-forward-one-backward schedule (``pipeline_parallel.py:129-222``). Returns the mean loss (last stage).

    Order of compute and of messages per stage is the reference's. What differs is when the transfers are issued: the
    activation of micro-batch ``k+1`` and the gradient of micro-batch ``j+1`` are already being received while
    micro-batch ``k`` / ``j`` computes, and a send only orders the communicator behind its producer.
    """
    g = pgm.get()
    p2p = get_p2p()
    n_mb = data_loader.grad_acc_steps
    num_warmup = min(g.pp_world_size - g.pp_rank - 1, n_mb)
    num_remaining = n_mb - num_warmup
    loss_acc = torch.zeros((), dtype=torch.float32, device=device)
    input_tensors, output_tensors = [], []
    requires_grad_sync = g.cp_dp_world_size > 1 or hasattr(model, "require_backward_grad_sync")
    args = dict(shapes=tensor_shapes, device=device, dtype=dtype)
    fwd_posted = bwd_posted = 0           # receives posted so far (n_mb of each in total)

    def next_forward_input():
        nonlocal fwd_posted
        if fwd_posted == 0:
            p2p.post_recv("fwd", **args)
            fwd_posted = 1
        with timed_phase("pp/wait_recv_fwd"):
            t = p2p.wait_recv("fwd", **args)
        if fwd_posted < n_mb:             # the one after it travels while this one computes
            p2p.post_recv("fwd", **args)
            fwd_posted += 1
        return t

    def next_backward_grad():
        nonlocal bwd_posted
        if bwd_posted == 0:
            p2p.post_recv("bwd", **args)
            bwd_posted = 1
        with timed_phase("pp/wait_recv_bwd"):
            t = p2p.wait_recv("bwd", **args)
        if bwd_posted < n_mb:
            p2p.post_recv("bwd", **args)
            bwd_posted += 1
        return t

    with nvtx_range("1f1b/warmup"):
        for _ in range(num_warmup):
            input_tensor = next_forward_input()
            output_tensor = _stage_forward(model, data_loader, input_tensor, device, loss_acc)
            p2p.send("fwd", output_tensor)
            input_tensors.append(input_tensor)
            output_tensors.append(output_tensor)

    if num_remaining > 0:
        input_tensor = next_forward_input()

    if requires_grad_sync:
        model.require_backward_grad_sync = False

    with nvtx_range("1f1b/steady"):
        for i in range(num_remaining):
            is_last = i == num_remaining - 1
            with timed_phase("pp/forward"):
                output_tensor = _stage_forward(model, data_loader, input_tensor, device, loss_acc)
            p2p.send("fwd", output_tensor)
            output_tensor_grad = next_backward_grad()
            input_tensors.append(input_tensor)
            output_tensors.append(output_tensor)
            input_tensor, output_tensor = input_tensors.pop(0), output_tensors.pop(0)
            # the stage without warm-up (the last one) finishes its step here
            if requires_grad_sync and num_warmup == 0 and is_last:
                model.require_backward_grad_sync = True
            with timed_phase("pp/backward"):
                input_tensor_grad = model.backward(input_tensor, output_tensor, output_tensor_grad)
            p2p.send("bwd", input_tensor_grad)
            p2p.release(input_tensor, output_tensor_grad)
            input_tensor = None if is_last else next_forward_input()

    with nvtx_range("1f1b/cooldown"):
        for i in range(num_warmup):
            if requires_grad_sync:
                model.require_backward_grad_sync = i == num_warmup - 1
            input_tensor, output_tensor = input_tensors.pop(0), output_tensors.pop(0)
            output_tensor_grad = next_backward_grad()
            input_tensor_grad = model.backward(input_tensor, output_tensor, output_tensor_grad)
            p2p.send("bwd", input_tensor_grad)
            p2p.release(input_tensor, output_tensor_grad)

    p2p.drain()
    return loss_acc.item() if g.pp_is_last_stage else 0.0
