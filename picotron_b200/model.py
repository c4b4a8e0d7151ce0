"""Flat-module alias of :mod:`picotron_b200.models.llama` (the reference exposes ``picotron.model``)."""
from .models.llama import *  # noqa: F401,F403
from .models.llama import Llama, DecoderLayer, Attention, MLP, RMSNorm, Embedding, FinalProjection  # noqa: F401
from .ops import rope_tables


def get_cos_sin(seq_length, head_dim, base=500000.0):
    """fp32 ``(cos, sin)`` tables of shape ``[seq_length, head_dim]`` (halves repeated, ``model.py:21-31``)."""
    cos, sin = rope_tables(seq_length, head_dim, base)
    return cos.repeat(1, 2), sin.repeat(1, 2)


def apply_rotary_pos_emb(x, cos, sin):
    """Eager NeoX-layout RoPE on ``[B, heads, S, d]`` with ``[S, d]`` tables (``model.py:12-19``)."""
    import torch
    half = x.shape[-1] // 2
    rot = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * cos + rot * sin
