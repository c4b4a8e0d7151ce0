"""Megatron-style 1-D tensor parallelism.

``apply_tensor_parallel(model)`` performs the module surgery of ``tensor_parallel.py:9-52`` of the
reference: q/k/v/gate/up become :class:`ColumnParallelLinear`, out/down become
:class:`RowParallelLinear`, the embedding becomes :class:`VocabParallelEmbedding` and the LM head a
column-parallel linear with gathered output. Shards are cut from a full master weight generated
identically on every rank (same seed), so a TP run starts from the same values as a single-GPU run.

The fused decoder-layer node reads the shard ``.weight`` of whichever module sits in the tree and puts
the all-reduces where these modules would; the modules' own ``forward`` stays available for
stand-alone use and for the parity tests.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import process_group_manager as pgm
from ..models.llama import embedding_lookup_2d
from .tp_communications import (GatherFromModelParallelRegion, ReduceFromModelParallelRegion,
                                linear_with_all_reduce, linear_with_async_all_reduce)
from ..models import llama as _llama


def apply_tensor_parallel(model):
    def _replace(module, name, style, gather_output=False):
        old = getattr(module, name)
        if style == "column":
            new = ColumnParallelLinear(old.in_features, old.out_features, bias=old.bias is not None,
                                       gather_output=gather_output)
        elif style == "row":
            new = RowParallelLinear(old.in_features, old.out_features, bias=old.bias is not None)
        else:
            new = VocabParallelEmbedding(old.num_embeddings, old.embedding_dim)
        new.init = getattr(model, "init", "reference")
        if old.weight.device.type != "meta":
            new.reset_parameters()
        setattr(module, name, new)

    plan = [("attention", "q_proj", "column"), ("attention", "k_proj", "column"),
            ("attention", "v_proj", "column"), ("attention", "out_proj", "row"),
            ("mlp", "gate_proj", "column"), ("mlp", "up_proj", "column"), ("mlp", "down_proj", "row")]
    for layer in model.decoder_layers:
        for sub, name, style in plan:
            _replace(getattr(layer, sub), name, style)
        layer._qkv_flat = layer._gu_flat = None
    _replace(model, "embedding", "vocab")
    _replace(model, "final_proj", "column", gather_output=True)
    return model


def _master_uniform(out_features: int, in_features: int, like: torch.Tensor, init: str) -> torch.Tensor:
    master = torch.empty(out_features, in_features, dtype=like.dtype, device=like.device)
    _llama.init_linear_weight_(master, init)
    return master


class ColumnParallelLinear(nn.Module):
    """``Y_i = X W_i^T`` with ``W`` split along its output dimension (``tensor_parallel.py:54-123``)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, gather_output: bool = False,
                 async_all_reduce: bool = False) -> None:
        super().__init__()
        g = pgm.get()
        self.tp_world_size, self.tp_rank = g.tp_world_size, g.tp_rank
        self.in_features, self.out_features = in_features, out_features
        assert out_features % self.tp_world_size == 0, "Hidden dimension must be divisible by the tensor parallel world size"
        self.output_size_per_partition = out_features // self.tp_world_size
        self.gather_output = gather_output
        self.async_all_reduce = async_all_reduce
        self.init = "reference"
        self.weight = nn.Parameter(torch.empty(self.output_size_per_partition, in_features))
        if bias:
            self.bias = nn.Parameter(torch.zeros(self.output_size_per_partition))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self, init: Optional[str] = None):
        if self.weight.device.type == "meta":
            return
        master = _master_uniform(self.out_features, self.in_features, self.weight, init or self.init)
        shard = torch.split(master, self.output_size_per_partition, dim=0)[self.tp_rank]
        with torch.no_grad():
            self.weight.copy_(shard)

    def ce_partition(self):
        """(tp group, first vocab id of this shard) when this layer is the vocab-parallel LM head."""
        g = pgm.get()
        if self.tp_world_size == 1:
            return None, 0
        return g.tp_group, self.tp_rank * self.output_size_per_partition

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        fn = linear_with_async_all_reduce if self.async_all_reduce else linear_with_all_reduce
        out = fn(x, self.weight, self.bias)
        if self.gather_output:
            out = GatherFromModelParallelRegion.apply(out)
        return out


class RowParallelLinear(nn.Module):
    """``Y = sum_i X_i W_i^T`` with ``W`` split along its input dimension (``tensor_parallel.py:125-189``)."""

    def __init__(self, in_features: int, out_features: int, bias: bool):
        super().__init__()
        g = pgm.get()
        self.tp_world_size, self.tp_rank = g.tp_world_size, g.tp_rank
        self.in_features, self.out_features = in_features, out_features
        assert in_features % self.tp_world_size == 0, "Hidden dimension must be divisible by the tensor parallel world size"
        self.input_size_per_partition = in_features // self.tp_world_size
        self.init = "reference"
        self.weight = nn.Parameter(torch.empty(out_features, self.input_size_per_partition))
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self, init: Optional[str] = None):
        if self.weight.device.type == "meta":
            return
        master = _master_uniform(self.out_features, self.in_features, self.weight, init or self.init)
        shard = torch.split(master, self.input_size_per_partition, dim=1)[self.tp_rank]
        with torch.no_grad():
            self.weight.copy_(shard)

    def forward(self, x):
        out = ReduceFromModelParallelRegion.apply(_llama.linear_2d(x.reshape(-1, x.shape[-1]), self.weight))
        out = out.view(*x.shape[:-1], self.out_features)
        return out if self.bias is None else out + self.bias


class VocabParallelEmbedding(nn.Module):
    """Embedding split along the vocabulary; out-of-shard ids give zero rows, then all-reduce
    (``tensor_parallel.py:191-270``). The lookup kernel does the range test, shift and zeroing itself."""

    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx: Optional[int] = None,
                 max_norm: Optional[float] = None, norm_type: float = 2.0, scale_grad_by_freq: bool = False,
                 sparse: bool = False):
        super().__init__()
        g = pgm.get()
        self.tp_world_size, self.tp_rank = g.tp_world_size, g.tp_rank
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.padding_idx, self.max_norm, self.norm_type = padding_idx, max_norm, norm_type
        self.scale_grad_by_freq, self.sparse = scale_grad_by_freq, sparse
        self.vocab_start_index, self.vocab_end_index = self._vocab_range_from_global_vocab_size(
            num_embeddings, self.tp_rank, self.tp_world_size)
        self.num_embeddings_per_partition = self.vocab_end_index - self.vocab_start_index
        self.init = "reference"
        self.weight = nn.Parameter(torch.empty(self.num_embeddings_per_partition, embedding_dim))
        self.reset_parameters()

    @staticmethod
    def _vocab_range_from_global_vocab_size(global_vocab_size: int, rank: int, world_size: int):
        assert global_vocab_size % world_size == 0, f"{global_vocab_size} is not divisible by {world_size}"
        per = global_vocab_size // world_size
        return rank * per, (rank + 1) * per

    def reset_parameters(self, init: Optional[str] = None):
        if self.weight.device.type == "meta":
            return
        init = init or self.init
        master = torch.empty(self.num_embeddings, self.embedding_dim, dtype=self.weight.dtype,
                             device=self.weight.device)
        with torch.no_grad():
            master.normal_(0.0, 0.02 if init == "normal" else 1.0)
            self.weight.copy_(torch.split(master, self.num_embeddings_per_partition, dim=0)[self.tp_rank])

    def forward(self, x):
        from . import tp_communications as tpc
        sp_group = tpc.sequence_parallel_group()
        if sp_group is not None:
            # sequence parallelism: the partial lookups are summed and each rank keeps its 1/tp of the tokens
            assert x.shape[-1] % self.tp_world_size == 0, "sequence parallelism needs seq_length divisible by tp_size"
            out = tpc.ReduceScatterTokens.apply(embedding_lookup_2d(x, self.weight, self.vocab_start_index), sp_group)
            return out.view(*x.shape[:-1], x.shape[-1] // self.tp_world_size, self.embedding_dim)
        ws = getattr(self, "shared_workspace", None)
        if ws is not None and x.is_cuda and self.weight.data_ptr() == ws.data.data_ptr():
            # shards in symmetric memory: read every row from its owner, no reduction
            out = _SharedEmbeddingFn.apply(x, self.weight, self)
        else:
            out = ReduceFromModelParallelRegion.apply(embedding_lookup_2d(x, self.weight, self.vocab_start_index))
        return out.view(*x.shape, self.embedding_dim)


class _SharedEmbeddingFn(torch.autograd.Function):
    """Lookup across the tensor-parallel group's weight shards (peer loads); backward = the local scatter-add of this
    rank's own rows, as for the masked lookup (the reference's all-reduce has an identity backward)."""

    @staticmethod
    def forward(ctx, ids, weight, module):
        from ..ops import _ext
        ws = module.shared_workspace
        flat = ids.reshape(-1).contiguous()
        ws.barrier()                 # every rank finished its last optimizer step: the shards hold this step's weights
        out = _ext.load().embedding_gather_peers(flat, ws.buf_ptrs, module.num_embeddings_per_partition, module.embedding_dim,
                                                 weight)
        ctx.save_for_backward(flat)
        ctx.weight, ctx.vocab_start = weight, module.vocab_start_index
        return out

    @staticmethod
    def backward(ctx, dy):
        from .. import ops
        from ..models.llama import notify_grad_ready
        (flat,) = ctx.saved_tensors
        w = ctx.weight
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        mg = getattr(w, "main_grad", None)
        if mg is not None:
            ops.embedding_bwd(flat, dy2, mg, ctx.vocab_start)
            notify_grad_ready(w)
            return None, None, None
        dw = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        ops.embedding_bwd(flat, dy2, dw, ctx.vocab_start)
        return None, dw.to(w.dtype), None
