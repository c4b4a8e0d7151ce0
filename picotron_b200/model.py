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


class TritonRMSNorm(RMSNorm):
    """Name of the reference's fused RMSNorm (``model.py:39-65``): same module as :class:`RMSNorm` here (fp32 statistics,
    weight applied before the single rounding), backed by this package's kernels on the GPU."""


class LlamaRMSNorm(RMSNorm):
    """The reference's eager RMSNorm (``model.py:67-86``): identical except that it rounds the normalised activation to the
    input dtype BEFORE multiplying by the weight. ``forward`` follows that order; it is a plain PyTorch module meant for
    parity checks, not a hot path."""

    def forward(self, x):
        import torch
        xf = x.float()
        normed = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype)
        return self.weight * normed


def flash_attention(q, k, v, causal=True):
    """``[B, heads, S, d]`` in, ``[B, S, heads, d]`` out, as the reference's wrapper of ``flash_attn_func``
    (``model.py:33-37``); K/V may have fewer heads than Q (grouped-query attention is native here)."""
    from . import ops
    out, _ = ops.attention_fwd(q.permute(0, 2, 1, 3).contiguous(), k.permute(0, 2, 1, 3).contiguous(),
                               v.permute(0, 2, 1, 3).contiguous(), bool(causal))
    return out
