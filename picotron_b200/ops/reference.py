"""Plain PyTorch restatements of every op of :mod:`picotron_b200.ops`.

They serve three purposes: (1) the CPU/Gloo execution path (the framework imports and trains with no
CUDA present), (2) the fp32 oracle the GPU numerics tests compare the sm_100a kernels against, and
(3) an executable definition of each op's contract (shapes, dtypes, rounding points).

All statistics and reductions are computed in fp32 and cast once at the end, which is the rounding
order of the fused kernels (the reference's fused RMSNorm, ``flash_attn/ops/triton/layer_norm.py``,
does the same; its eager ``LlamaRMSNorm`` casts before the weight multiply, ``model.py:83-86``).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


# ----------------------------------------------------------------------------- RMSNorm
def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
    y = (xf * rstd.unsqueeze(-1) * w.float()).to(x.dtype)
    return y, rstd


def add_rmsnorm_fwd(x: torch.Tensor, delta: torch.Tensor, w: torch.Tensor, eps: float):
    x_new = (x.float() + delta.float()).to(x.dtype)
    y, rstd = rmsnorm_fwd(x_new, w, eps)
    return x_new, y, rstd


def rmsnorm_bwd(dy: torch.Tensor, x: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor,
                dres: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """dx = rstd * (w*dy - xhat * mean(xhat * w*dy)) (+ dres);  dw = sum_t dy * xhat  (fp32)."""
    xf, dyf, wf = x.float(), dy.float(), w.float()
    xhat = xf * rstd.unsqueeze(-1)
    wdy = dyf * wf
    c = (xhat * wdy).mean(-1, keepdim=True)
    dx = (wdy - xhat * c) * rstd.unsqueeze(-1)
    if dres is not None:
        dx = dx + dres.float()
    dw = (dyf * xhat).sum(0)
    return dx.to(x.dtype), dw


# ----------------------------------------------------------------------------- RoPE
def scaled_rope_frequencies(inv_freq: torch.Tensor, scaling: dict) -> torch.Tensor:
    """Frequency rescaling of long-context checkpoints (``rope_scaling`` of a Hugging Face config).

    ``linear``: every frequency divided by ``factor`` (position interpolation). ``llama3`` (Llama 3.1 / 3.2): wavelengths
    longer than ``original_max_position_embeddings / low_freq_factor`` are divided by ``factor``, those shorter than
    ``original_max_position_embeddings / high_freq_factor`` are kept, the band between is blended linearly in
    ``original_max_position_embeddings / wavelength``. The reference ignores the field (``model.py:21-31``), which
    is exact for training from scratch but changes what a pretrained Llama-3.2 checkpoint computes.
    """
    import math
    kind = scaling.get("rope_type", scaling.get("type"))
    factor = float(scaling["factor"])
    if kind == "linear":
        return inv_freq / factor
    if kind != "llama3":
        raise ValueError(f"unsupported rope scaling {kind!r} (supported: linear, llama3)")
    low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    old_len = float(scaling["original_max_position_embeddings"])
    wavelen = 2 * math.pi / inv_freq
    scaled = torch.where(wavelen > old_len / low, inv_freq / factor, inv_freq)
    smooth = (old_len / wavelen - low) / (high - low)
    blended = (1 - smooth) * inv_freq / factor + smooth * inv_freq
    medium = ~(wavelen < old_len / high) & ~(wavelen > old_len / low)
    return torch.where(medium, blended, scaled)


def rope_tables(seq_length: int, head_dim: int, base: float, device=None,
                scaling: Optional[dict] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 cos/sin tables ``[S, head_dim/2]``; frequencies ``base**(-2i/d)`` as ``model.py:21-31``, optionally rescaled
    (:func:`scaled_rope_frequencies`)."""
    assert head_dim % 2 == 0
    theta = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    if scaling:
        theta = scaled_rope_frequencies(theta, scaling)
    pos = torch.arange(seq_length, dtype=torch.float32).unsqueeze(1)
    ang = pos * theta.unsqueeze(0)
    cos, sin = torch.cos(ang), torch.sin(ang)
    if device is not None:
        cos, sin = cos.to(device), sin.to(device)
    return cos.contiguous(), sin.contiguous()


def rope_(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_rot_heads: int, head_dim: int,
          seq_len: int, inverse: bool = False) -> torch.Tensor:
    """Rotate, in place, the first ``n_rot_heads`` heads of every row of ``qkv`` ``[T, n_heads*head_dim]``.

    Row ``t`` is at position ``t % seq_len``. NeoX (half-split) layout, fp32 math:
    ``out[:d/2] = x1*cos - x2*sin``, ``out[d/2:] = x2*cos + x1*sin`` (``model.py:12-19``); ``inverse``
    flips the sign of ``sin`` (this is the backward pass).
    """
    T = qkv.shape[0]
    half = head_dim // 2
    x = qkv[:, : n_rot_heads * head_dim].reshape(T, n_rot_heads, head_dim).float()
    pos = torch.arange(T, device=qkv.device) % seq_len
    c = cos[pos].unsqueeze(1).float()
    s = sin[pos].unsqueeze(1).float()
    if inverse:
        s = -s
    x1, x2 = x[..., :half], x[..., half:]
    out = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
    qkv[:, : n_rot_heads * head_dim] = out.reshape(T, n_rot_heads * head_dim).to(qkv.dtype)
    return qkv


# ----------------------------------------------------------------------------- SwiGLU
def swiglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    inter = gu.shape[-1] // 2
    g, u = gu[..., :inter].float(), gu[..., inter:].float()
    return (g * torch.sigmoid(g) * u).to(gu.dtype)


def swiglu_bwd(gu: torch.Tensor, da: torch.Tensor) -> torch.Tensor:
    inter = gu.shape[-1] // 2
    g, u, d = gu[..., :inter].float(), gu[..., inter:].float(), da.float()
    sig = torch.sigmoid(g)
    silu = g * sig
    dg = d * u * (sig * (1.0 + g * (1.0 - sig)))
    du = d * silu
    return torch.cat([dg, du], dim=-1).to(gu.dtype)


# ----------------------------------------------------------------------------- GEMMs
def linear_fwd(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return x @ w.t()


def linear_dgrad(dy: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return dy @ w


def linear_wgrad(dy: torch.Tensor, x: torch.Tensor, out: Optional[torch.Tensor] = None):
    """``dy^T @ x``; with ``out`` (fp32) the product is accumulated into it and ``None`` is returned."""
    if out is None:
        return dy.t() @ x
    out.add_((dy.t().float() @ x.float()).to(out.dtype) if out.dtype != dy.dtype else dy.t() @ x)
    return None


# ----------------------------------------------------------------------------- attention
def _expand_kv(k: torch.Tensor, hq: int) -> torch.Tensor:
    hkv = k.shape[2]
    return k if hkv == hq else k.repeat_interleave(hq // hkv, dim=2)


def attention_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool, scale: float):
    """q ``[B,Sq,hq,d]``, k/v ``[B,Sk,hkv,d]`` -> o ``[B,Sq,hq,d]``, lse ``[B,hq,Sq]`` (fp32, natural log).

    ``causal`` masks ``j > i`` (query i, key j, both counted from the start of their block: the
    diagonal-block convention of ring attention, ``context_parallel.py:112-128``).
    """
    B, Sq, hq, d = q.shape
    Sk = k.shape[1]
    qf = q.float().permute(0, 2, 1, 3)
    kf = _expand_kv(k, hq).float().permute(0, 2, 1, 3)
    vf = _expand_kv(v, hq).float().permute(0, 2, 1, 3)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(Sq, Sk, dtype=torch.bool, device=q.device).triu(1)
        s = s.masked_fill(mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    o = torch.matmul(p, vf).permute(0, 2, 1, 3).contiguous().to(q.dtype)
    return o, lse


def attention_bwd(do: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor,
                  lse: torch.Tensor, causal: bool, scale: float, delta: Optional[torch.Tensor] = None):
    """FlashAttention-2 backward formulae from a (possibly global) ``lse``; returns fp32 dq, dk, dv.

    ``delta = rowsum(do * o)`` may be passed in (ring attention computes it once from the merged output).
    dk/dv are reduced over the query heads of each KV group (native GQA).
    """
    B, Sq, hq, d = q.shape
    Sk, hkv = k.shape[1], k.shape[2]
    g = hq // hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = _expand_kv(k, hq).float().permute(0, 2, 1, 3)
    vf = _expand_kv(v, hq).float().permute(0, 2, 1, 3)
    dof = do.float().permute(0, 2, 1, 3)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(Sq, Sk, dtype=torch.bool, device=q.device).triu(1)
        s = s.masked_fill(mask, float("-inf"))
    p = torch.exp(s - lse.unsqueeze(-1))
    if delta is None:
        delta = (dof * o.float().permute(0, 2, 1, 3)).sum(-1)
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    ds = p * (dp - delta.unsqueeze(-1))
    dq = torch.matmul(ds, kf) * scale
    dk = torch.matmul(ds.transpose(-1, -2), qf) * scale
    dq = dq.permute(0, 2, 1, 3).contiguous()
    dk = dk.view(B, hkv, g, Sk, d).sum(2).permute(0, 2, 1, 3).contiguous()
    dv = dv.view(B, hkv, g, Sk, d).sum(2).permute(0, 2, 1, 3).contiguous()
    return dq, dk, dv


# ----------------------------------------------------------------------------- embedding
def embedding_fwd(ids: torch.Tensor, w: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    """Rows of ``w`` for ``ids - vocab_start``; ids outside ``[vocab_start, vocab_start+rows)`` give zeros."""
    flat = ids.reshape(-1) - vocab_start
    ok = (flat >= 0) & (flat < w.shape[0])
    out = w[flat.clamp(0, w.shape[0] - 1)]
    return out * ok.unsqueeze(-1).to(out.dtype)


def embedding_bwd(ids: torch.Tensor, dy: torch.Tensor, dw: torch.Tensor, vocab_start: int = 0) -> None:
    flat = ids.reshape(-1) - vocab_start
    ok = (flat >= 0) & (flat < dw.shape[0])
    dw.index_add_(0, flat[ok], dy.reshape(-1, dy.shape[-1])[ok].to(dw.dtype))


# ----------------------------------------------------------------------------- cross entropy
def ce_stats(logits: torch.Tensor, targets: torch.Tensor, vocab_start: int = 0):
    """Per-row (max, sum exp(l - max), target logit or 0 when the target is not in this vocab shard)."""
    lf = logits.float()
    rowmax = lf.max(-1).values
    sumexp = torch.exp(lf - rowmax.unsqueeze(-1)).sum(-1)
    local = targets - vocab_start
    ok = (local >= 0) & (local < logits.shape[-1])
    tgt = lf.gather(-1, local.clamp(0, logits.shape[-1] - 1).unsqueeze(-1)).squeeze(-1) * ok.float()
    return rowmax, sumexp, tgt


def ce_grad_(logits: torch.Tensor, targets: torch.Tensor, lse: torch.Tensor, scale: float,
             vocab_start: int = 0) -> torch.Tensor:
    """In place: ``logits <- (exp(logits - lse) - onehot(target)) * scale``."""
    p = torch.exp(logits.float() - lse.unsqueeze(-1))
    local = targets - vocab_start
    ok = (local >= 0) & (local < logits.shape[-1])
    rows = torch.nonzero(ok).squeeze(-1)
    p[rows, local[rows]] -= 1.0
    logits.copy_((p * scale).to(logits.dtype))
    return logits


# ----------------------------------------------------------------------------- gradient buckets / optimizer
def accumulate_(main_grad: torch.Tensor, grad: torch.Tensor) -> None:
    main_grad.add_(grad.to(main_grad.dtype))


def adamw_step_(params, grads, exp_avgs, exp_avg_sqs, masters, step: int, lr: float, beta1: float,
                beta2: float, eps: float, weight_decay: float, grad_scale: float = 1.0) -> None:
    """Decoupled-weight-decay Adam, the update of ``torch.optim.AdamW`` (used at ``train.py:209``).

    ``masters[i]`` (fp32) is the tensor that is updated when present; ``params[i]`` then receives the
    rounded copy. Moments may be fp32 or the parameter dtype.
    """
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    for p, g, m, v, mw in zip(params, grads, exp_avgs, exp_avg_sqs, masters):
        gf = g.float() * grad_scale
        w = mw if mw is not None else p.float()
        w = w * (1.0 - lr * weight_decay)
        mf = m.float() * beta1 + gf * (1.0 - beta1)
        vf = v.float() * beta2 + gf * gf * (1.0 - beta2)
        denom = (vf.sqrt() / math.sqrt(bc2)) + eps
        w = w - (lr / bc1) * (mf / denom)
        m.copy_(mf.to(m.dtype))
        v.copy_(vf.to(v.dtype))
        if mw is not None:
            mw.copy_(w)
        p.copy_(w.to(p.dtype))


# ----------------------------------------------------------------------------- ring-attention merge
def merge_attention_(out: torch.Tensor, lse: torch.Tensor, block_out: torch.Tensor, block_lse: torch.Tensor):
    """Online merge of two partial attention results (fp32 ``out [B,S,h,d]``, ``lse [B,h,S]``), in place.

    Same algebra as ``context_parallel.py:157-187`` (sigmoid / logsigmoid form).
    """
    bl = block_lse.transpose(1, 2).unsqueeze(-1)  # [B,S,h,1]
    cl = lse.transpose(1, 2).unsqueeze(-1)
    out.sub_(torch.sigmoid(bl - cl) * (out - block_out.float()))
    lse.sub_(torch.nn.functional.logsigmoid(lse - block_lse))
    return out, lse
