"""Independent plain-PyTorch Llama (autograd does the backward) used as the numerical oracle.

Written from the architecture description (pre-norm residual blocks, NeoX RoPE, GQA by head
repetition, SwiGLU, untied head), not from the framework's ops, so that a shared bug cannot hide.
"""
import math

import torch
import torch.nn.functional as F


def rmsnorm(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def rope(x, theta, positions):
    # x: [B, S, h, d]
    d = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, d, 2).float() / d))
    ang = positions.float()[:, None] * inv[None, :]
    cos, sin = torch.cos(ang)[None, :, None, :], torch.sin(ang)[None, :, None, :]
    x1, x2 = x[..., : d // 2].float(), x[..., d // 2:].float()
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).to(x.dtype)


def llama_forward(params, cfg, input_ids, positions=None):
    """params: dict name -> tensor with the framework's state-dict names. Returns logits [B,S,V]."""
    B, S = input_ids.shape
    if positions is None:
        positions = torch.arange(S)
    hq, hkv = cfg.num_attention_heads, cfg.num_key_value_heads
    d = cfg.hidden_size // hq
    x = params["embedding.weight"][input_ids]
    for i in range(cfg.num_hidden_layers):
        p = lambda n: params[f"decoder_layers.{i}.{n}.weight"]
        h = rmsnorm(x, p("input_layernorm"), cfg.rms_norm_eps)
        q = (h @ p("attention.q_proj").t()).view(B, S, hq, d)
        k = (h @ p("attention.k_proj").t()).view(B, S, hkv, d)
        v = (h @ p("attention.v_proj").t()).view(B, S, hkv, d)
        q, k = rope(q, cfg.rope_theta, positions), rope(k, cfg.rope_theta, positions)
        k = k.repeat_interleave(hq // hkv, dim=2)
        v = v.repeat_interleave(hq // hkv, dim=2)
        s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) / math.sqrt(d)
        mask = torch.ones(S, S, dtype=torch.bool).triu(1)
        s = s.masked_fill(mask, float("-inf"))
        o = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), v.float()).to(x.dtype).reshape(B, S, hq * d)
        x = x + o @ p("attention.out_proj").t()
        h = rmsnorm(x, p("post_attention_layernorm"), cfg.rms_norm_eps)
        x = x + (F.silu(h @ p("mlp.gate_proj").t()) * (h @ p("mlp.up_proj").t())) @ p("mlp.down_proj").t()
    x = rmsnorm(x, params["final_norm.weight"], cfg.rms_norm_eps)
    return x @ params["final_proj.weight"].t()


def loss_and_grads(params, cfg, input_ids, target_ids):
    ps = {k: v.detach().clone().requires_grad_(True) for k, v in params.items()}
    logits = llama_forward(ps, cfg, input_ids)
    loss = F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), target_ids.reshape(-1))
    loss.backward()
    return loss.detach(), {k: v.grad for k, v in ps.items()}
