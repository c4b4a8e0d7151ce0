"""Llama decoder built from fused ops with hand-derived backward passes.

Module tree and parameter names follow the reference model (``picotron/model.py:88-298``) so that
state dicts and the per-rank checkpoint layout are interchangeable:
``embedding``, ``decoder_layers.{i}.{input_layernorm,post_attention_layernorm}``,
``decoder_layers.{i}.attention.{q,k,v,out}_proj``, ``decoder_layers.{i}.mlp.{gate,up,down}_proj``,
``final_norm``, ``final_proj`` (never tied in the reference, ``checkpoint.py:89-102``; tying is an option here,
``parallel/tied_embeddings.py``).

What differs is how a layer executes. A decoder layer is ONE autograd node
(:class:`DecoderLayerFn`): its forward launches the kernels of the layer back to back
(RMSNorm -> packed QKV GEMM -> in-place RoPE -> flash attention -> out-proj GEMM -> residual+RMSNorm ->
packed gate/up GEMM -> SwiGLU -> down GEMM) and its backward is written out by hand, so autograd
bookkeeping costs one node per layer instead of ~25, K/V are never expanded for GQA
(``model.py:142-143`` expands them), and weight gradients are accumulated by the GEMM epilogue straight
into the fp32 gradient buckets of the data-parallel engine (``param.main_grad``) when those exist.

Tensor parallelism (column-parallel q/k/v/gate/up, row-parallel out/down, ``tensor_parallel.py:9-52``)
and context parallelism (ring attention, ``context_parallel.py:14-110``) are handled inside the node:
the all-reduces sit exactly where the reference's ``f``/``g`` functions put them.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from .. import process_group_manager as pgm
from ..parallel import tp_communications as tpc
from ..utils.tracing import nvtx_range


# ----------------------------------------------------------------------------------------------
# helpers shared by the fused nodes
# ----------------------------------------------------------------------------------------------
def pack_parameters(params: Sequence[nn.Parameter]) -> torch.Tensor:
    """Return one ``[sum(rows), cols]`` tensor whose row blocks alias ``params`` (re-homing them if needed).

    q/k/v (and gate/up) are separate parameters for state-dict compatibility but are consumed by a
    single GEMM. The parameters are moved (``param.data`` re-pointed, the Parameter objects stay) into
    one flat allocation the first time, or again after ``module.to(...)`` gave them new storage.
    """
    p0 = params[0]
    cols = p0.shape[1]
    esize = p0.element_size()
    adjacent = all(p.is_contiguous() and p.shape[1] == cols and p.dtype == p0.dtype and p.device == p0.device
                   for p in params)
    if adjacent:
        for a, b in zip(params[:-1], params[1:]):
            if a.data_ptr() + a.numel() * esize != b.data_ptr() or \
                    a.untyped_storage().data_ptr() != b.untyped_storage().data_ptr():
                adjacent = False
                break
    rows = sum(p.shape[0] for p in params)
    if not adjacent:
        flat = torch.empty(rows, cols, dtype=p0.dtype, device=p0.device)
        r = 0
        with torch.no_grad():
            for p in params:
                flat[r:r + p.shape[0]].copy_(p.data)
                p.data = flat[r:r + p.shape[0]]
                r += p.shape[0]
        return flat
    return torch.empty(0, dtype=p0.dtype, device=p0.device).set_(
        p0.untyped_storage(), p0.storage_offset(), (rows, cols), (cols, 1))


def packed_main_grad(params: Sequence[nn.Parameter]) -> Optional[torch.Tensor]:
    """The fp32 gradient-bucket region covering ``params`` as one ``[rows, cols]`` tensor, or None."""
    mgs = [getattr(p, "main_grad", None) for p in params]
    if any(m is None for m in mgs):
        return None
    m0 = mgs[0]
    for a, b in zip(mgs[:-1], mgs[1:]):
        if a.data_ptr() + a.numel() * a.element_size() != b.data_ptr():
            return None
    rows = sum(m.shape[0] for m in mgs)
    if len(mgs) == 1:
        return m0
    return torch.empty(0, dtype=m0.dtype, device=m0.device).set_(
        m0.untyped_storage(), m0.storage_offset(), (rows, m0.shape[1]), (m0.shape[1], 1))


def notify_grad_ready(p: nn.Parameter) -> None:
    """Tell the data-parallel engine that ``p.main_grad`` received this backward's contribution."""
    cb = getattr(p, "_grad_ready_cb", None)
    if cb is None:
        return
    uses = getattr(p, "_grad_uses", 1)
    if uses > 1:
        # a weight used by several layers of this rank (tied embedding / LM head) is ready after its LAST contribution
        seen = getattr(p, "_grad_seen", 0) + 1
        p._grad_seen = seen % uses
        if seen < uses:
            return
    cb()


def weight_grad(dy: torch.Tensor, x: torch.Tensor, params: Sequence[nn.Parameter]) -> List[Optional[torch.Tensor]]:
    """``dy^T @ x`` for a (packed) weight: fused fp32 accumulation into the buckets, else autograd grads."""
    mg = packed_main_grad(params)
    if mg is not None:
        ops.linear_wgrad(dy, x, out=mg)
        for p in params:
            notify_grad_ready(p)
        return [None] * len(params)
    dw = ops.linear_wgrad(dy, x)
    out, r = [], 0
    for p in params:
        out.append(dw[r:r + p.shape[0]])
        r += p.shape[0]
    return out


def vector_grad(dw32: torch.Tensor, p: nn.Parameter) -> Optional[torch.Tensor]:
    mg = getattr(p, "main_grad", None)
    if mg is not None:
        mg.add_(dw32)
        notify_grad_ready(p)
        return None
    return dw32.to(p.dtype)


def rmsnorm_backward(dy, x, p: nn.Parameter, rstd, dres=None):
    """RMSNorm backward whose weight gradient goes straight into the fp32 bucket slice of ``p`` when it has one.

    Returns ``(dx, grad)``; ``grad`` is None when the bucket received the gradient, else a tensor for autograd.
    """
    mg = getattr(p, "main_grad", None)
    if mg is not None and mg.is_contiguous():
        dx, _ = ops.rmsnorm_bwd(dy, x, p, rstd, dres, dw_acc=mg)
        notify_grad_ready(p)
        return dx, None
    dx, dw = ops.rmsnorm_bwd(dy, x, p, rstd, dres)
    return dx, vector_grad(dw, p)


# ----------------------------------------------------------------------------------------------
# basic modules (usable on their own; the decoder layer bypasses their forward)
# ----------------------------------------------------------------------------------------------
class _LinearFn(torch.autograd.Function):
    """2-D in, 2-D out (no views are created inside the node, so callers may reduce the result in place)."""

    @staticmethod
    def forward(ctx, x2, weight):
        ctx.save_for_backward(x2, weight)
        return ops.linear_fwd(x2, weight)

    @staticmethod
    def backward(ctx, dy2):
        x2, weight = ctx.saved_tensors
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = ops.linear_dgrad(dy2, weight) if ctx.needs_input_grad[0] else None
        dw = ops.linear_wgrad(dy2, x2) if ctx.needs_input_grad[1] else None
        return dx, dw


def linear_2d(x2: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    return _LinearFn.apply(x2 if x2.is_contiguous() else x2.contiguous(), weight)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = linear_2d(x.reshape(-1, x.shape[-1]), weight).view(*x.shape[:-1], weight.shape[0])
    return y if bias is None else y + bias


class Linear(nn.Module):
    """``y = x W^T`` (+ b) on the framework's GEMM; init U(+-1/sqrt(in)) as ``model.py:112-120``."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        self.reset_parameters()

    def reset_parameters(self, init: str = "reference"):
        init_linear_weight_(self.weight, init)
        if self.bias is not None:
            with torch.no_grad():
                self.bias.zero_()

    def forward(self, x):
        return linear(x, self.weight, self.bias)


def init_linear_weight_(w: torch.Tensor, init: str = "reference") -> None:
    if w.device.type == "meta":
        return
    with torch.no_grad():
        if init == "normal":
            w.normal_(0.0, 0.02)
        else:
            bound = math.sqrt(1.0 / w.shape[1])
            w.uniform_(-bound, bound)


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        x2 = x.reshape(-1, x.shape[-1])
        y, rstd = ops.rmsnorm_fwd(x2, weight, eps)
        ctx.save_for_backward(x2, rstd)
        ctx.weight = weight
        return y.view_as(x)

    @staticmethod
    def backward(ctx, dy):
        x2, rstd = ctx.saved_tensors
        weight = ctx.weight
        dx, g_w = rmsnorm_backward(dy.reshape(-1, dy.shape[-1]).contiguous(), x2, weight, rstd)
        # with gradient buckets the weight gradient is accumulated in place (no AccumulateGrad node runs)
        return dx.view_as(dy), g_w, None


class RMSNorm(nn.Module):
    """fp32-statistics RMSNorm, weight initialised to ones (``model.py:39-86``)."""

    def __init__(self, hidden_size: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(hidden_size))
        self.eps = eps
        self.variance_epsilon = eps
        self.reset_parameters()

    def reset_parameters(self, init: str = "reference"):
        if self.weight.device.type != "meta":
            with torch.no_grad():
                self.weight.fill_(1.0)

    def forward(self, x):
        return _RMSNormFn.apply(x, self.weight, self.eps)


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, vocab_start):
        ctx.save_for_backward(ids)
        ctx.weight = weight
        ctx.vocab_start = vocab_start
        return ops.embedding_fwd(ids, weight, vocab_start)          # [T, H]

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        w = ctx.weight
        dy2 = dy.reshape(-1, dy.shape[-1])
        mg = getattr(w, "main_grad", None)
        if mg is not None:
            ops.embedding_bwd(ids, dy2, mg, ctx.vocab_start)
            notify_grad_ready(w)
            return None, None, None
        dw = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        ops.embedding_bwd(ids, dy2, dw, ctx.vocab_start)
        return None, dw.to(w.dtype), None


def embedding_lookup_2d(ids: torch.Tensor, weight: nn.Parameter, vocab_start: int = 0) -> torch.Tensor:
    """``[T, H]`` rows for the flattened ids (zeros for ids outside this vocab shard)."""
    return _EmbeddingFn.apply(ids, weight, vocab_start)


def embedding_lookup(ids: torch.Tensor, weight: nn.Parameter, vocab_start: int = 0) -> torch.Tensor:
    return embedding_lookup_2d(ids, weight, vocab_start).view(*ids.shape, weight.shape[1])


class Embedding(nn.Module):
    """Token embedding, N(0,1) init (``model.py:237-251``)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx=None):
        super().__init__()
        self.num_embeddings, self.embedding_dim, self.padding_idx = num_embeddings, embedding_dim, padding_idx
        self.weight = nn.Parameter(torch.empty(num_embeddings, embedding_dim))
        self.reset_parameters()

    def reset_parameters(self, init: str = "reference"):
        if self.weight.device.type == "meta":
            return
        with torch.no_grad():
            self.weight.normal_(0.0, 0.02 if init == "normal" else 1.0)

    def forward(self, x):
        return embedding_lookup(x, self.weight)


class FinalProjection(Linear):
    """LM head ``[vocab, hidden]`` (``model.py:188-212``)."""

    def __init__(self, hidden_size: int, vocab_size: int, bias: bool = False):
        super().__init__(hidden_size, vocab_size, bias=bias)


class Attention(nn.Module):
    """Holder of the attention projections; heads are split across TP ranks (``model.py:95-98``)."""

    def __init__(self, config, layer_idx: int):
        super().__init__()
        g = pgm.get()
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.num_key_values = config.num_key_value_heads
        self.head_dim = self.hidden_size // self.num_heads
        assert self.num_heads % g.tp_world_size == 0, "num_attention_heads should be divisible by tp world size"
        assert self.num_key_values % g.tp_world_size == 0, "num_key_value_heads should be divisible by tp world size"
        self.num_local_heads = self.num_heads // g.tp_world_size
        self.num_local_kv_heads = self.num_key_values // g.tp_world_size
        self.q_proj = Linear(config.hidden_size, self.num_heads * self.head_dim)
        self.k_proj = Linear(config.hidden_size, self.num_key_values * self.head_dim)
        self.v_proj = Linear(config.hidden_size, self.num_key_values * self.head_dim)
        self.out_proj = Linear(config.hidden_size, config.hidden_size)
        self.layer_idx = layer_idx
        self.cp_enabled = False  # set by parallel.context_parallel.apply_context_parallel

    def reset_parameters(self, init: str = "reference"):
        for m in (self.q_proj, self.k_proj, self.v_proj, self.out_proj):
            m.reset_parameters(init) if isinstance(m, Linear) else m.reset_parameters()


class MLP(nn.Module):
    """SwiGLU MLP ``down(silu(gate(x)) * up(x))`` (``model.py:164-186``)."""

    def __init__(self, config):
        super().__init__()
        self.gate_proj = Linear(config.hidden_size, config.intermediate_size)
        self.up_proj = Linear(config.hidden_size, config.intermediate_size)
        self.down_proj = Linear(config.intermediate_size, config.hidden_size)

    def reset_parameters(self, init: str = "reference"):
        for m in (self.gate_proj, self.up_proj, self.down_proj):
            m.reset_parameters(init) if isinstance(m, Linear) else m.reset_parameters()


# ----------------------------------------------------------------------------------------------
# the decoder layer as one autograd node
# ----------------------------------------------------------------------------------------------
class DecoderLayerFn(torch.autograd.Function):
    """x -> x + Attn(RMSNorm(x)); -> + MLP(RMSNorm(.)) with a hand-written backward.

    Saved per layer: the layer input, both rstd vectors, the normed inputs of the two column-parallel
    GEMMs, the post-RoPE packed qkv, the attention output and its LSE, the mid residual, the packed
    gate/up pre-activations and the SwiGLU output.
    """

    @staticmethod
    def forward(ctx, x, ln1_w, ln2_w, wq, wk, wv, wo, wg, wu, wd, layer):
        B, S_in, H = x.shape
        att = layer.attention
        hq, hkv, d = att.num_local_heads, att.num_local_kv_heads, att.head_dim
        tp_group = layer.tp_group
        # sequence parallelism: x holds this rank's 1/tp of the micro-batch's tokens (rows of the flattened [B*S, H]);
        # the norms and residual adds work on those rows, the GEMMs and the attention on all of them
        sp_group = tpc.sequence_parallel_group()
        S = S_in * (dist.get_world_size(sp_group) if sp_group is not None else 1)
        T = B * S
        x2 = x.reshape(B * S_in, H)

        w_qkv = layer.packed_qkv()
        w_gu = layer.packed_gu()

        h1, rstd1 = ops.rmsnorm_fwd(x2, ln1_w, layer.eps)
        h1_all = tpc.gather_tokens(h1, sp_group) if sp_group is not None else h1
        cos, sin = layer.rope(x.device)
        qkv = ops.linear_rope_fwd(h1_all, w_qkv, cos, sin, hq + hkv, d, S)  # [T, (hq+2hkv)d], q and k heads rotated
        del h1_all
        q, k, v = layer.split_qkv(qkv, B, S)
        if att.cp_enabled:
            from ..parallel import context_parallel as cpar
            o, lse = cpar.ring_attention_forward_blocks(q, k, v, layer.sm_scale, True)
        else:
            o, lse = ops.attention_fwd(q, k, v, True, layer.sm_scale)      # o [B,S,hq,d]
        o2 = o.reshape(T, hq * d)
        if sp_group is not None:
            attn_out = tpc.reduce_scatter_tokens(ops.linear_fwd(o2, wo), sp_group)     # row-parallel GEMM + reduce-scatter
        else:
            attn_out = tpc.linear_all_reduce(o2, wo, tp_group)              # row-parallel GEMM + `g`
        x_mid, h2, rstd2 = ops.add_rmsnorm_fwd(x2, attn_out, ln2_w, layer.eps)
        h2_all = tpc.gather_tokens(h2, sp_group) if sp_group is not None else h2
        gu, a = ops.linear_swiglu_fwd(h2_all, w_gu)                         # [T, 2I] pre-activations, [T, I] silu(g)*u
        del h2_all
        if tp_group is None:
            out = ops.linear_add_fwd(a, wd, x_mid)                          # down projection + residual in one kernel
        elif sp_group is not None:
            out = ops.add(x_mid, tpc.reduce_scatter_tokens(ops.linear_fwd(a, wd), sp_group))
        else:
            out = ops.add(x_mid, tpc.linear_all_reduce(a, wd, tp_group))

        # h1 and h2 are kept as this rank's rows under sequence parallelism and gathered again in the backward pass
        ctx.save_for_backward(x2, rstd1, h1, qkv, o2, lse, x_mid, rstd2, h2, gu, a)
        ctx.layer = layer
        ctx.dims = (B, S, H, S_in)
        ctx.sp_group = sp_group
        return out.view(B, S_in, H)

    @staticmethod
    def backward(ctx, dout):
        with nvtx_range(f"layer{ctx.layer.layer_idx}/bwd"):
            return DecoderLayerFn._backward(ctx, dout)

    @staticmethod
    def _backward(ctx, dout):
        x2, rstd1, h1, qkv, o2, lse, x_mid, rstd2, h2, gu, a = ctx.saved_tensors
        layer = ctx.layer
        B, S, H, S_in = ctx.dims
        sp_group = ctx.sp_group
        att, mlp = layer.attention, layer.mlp
        hq, hkv, d = att.num_local_heads, att.num_local_kv_heads, att.head_dim
        tp_group = layer.tp_group
        ln1, ln2 = layer.input_layernorm, layer.post_attention_layernorm
        w_qkv, w_gu = layer.packed_qkv(), layer.packed_gu()
        wo, wd = att.out_proj.weight, mlp.down_proj.weight
        dout2 = dout.reshape(B * S_in, H)
        if not dout2.is_contiguous():
            dout2 = dout2.contiguous()
        sp = sp_group is not None
        dout_all = tpc.gather_tokens(dout2, sp_group) if sp else dout2      # backward of the forward's reduce-scatter

        # ---- MLP
        dgu = ops.linear_dgrad_swiglu_bwd(dout_all, wd, gu)                 # dgrad GEMM + SwiGLU backward in its epilogue
        g_wd = weight_grad(dout_all, a, [wd])
        del dout_all
        if sp:
            dh2 = tpc.reduce_scatter_tokens(ops.linear_dgrad(dgu, w_gu), sp_group)   # backward of the forward's all-gather
            h2, reduced = tpc.gather_tokens(h2, sp_group), tpc._Done()
        else:
            dh2, reduced = tpc.linear_dgrad_all_reduce_async(dgu, w_gu, tp_group)   # column-parallel `f` backward ...
        g_wg, g_wu = weight_grad(dgu, h2, [mlp.gate_proj.weight, mlp.up_proj.weight])
        reduced.wait()                                                          # ... overlapped with the weight gradient
        del dgu, h2
        dx_mid, g_ln2 = rmsnorm_backward(dh2, x_mid, ln2.weight, rstd2, dout2)

        # ---- attention
        dx_mid_all = tpc.gather_tokens(dx_mid, sp_group) if sp else dx_mid
        do2 = ops.linear_dgrad(dx_mid_all, wo)
        g_wo = weight_grad(dx_mid_all, o2, [wo])
        del dx_mid_all
        q, k, v = layer.split_qkv(qkv, B, S)
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = layer.split_qkv(dqkv, B, S)
        do4, o4 = do2.view(B, S, hq, d), o2.view(B, S, hq, d)
        if att.cp_enabled:
            from ..parallel import context_parallel as cpar
            rq, rk, rv = cpar.ring_attention_backward_blocks(do4, q, k, v, o4, lse, layer.sm_scale, True)
            dq.copy_(rq), dk.copy_(rk), dv.copy_(rv)
            ops.rope_(dqkv, *layer.rope(dout.device), hq + hkv, d, S, True)
        elif ops.attention_bwd_fuses_rope(q):
            # the kernel un-rotates dq (while converting its fp32 accumulator) and dk (in its epilogue)
            ops.attention_bwd(do4, q, k, v, o4, lse, True, layer.sm_scale, outs=(dq, dk, dv), rope=layer.rope(dout.device))
        else:
            ops.attention_bwd(do4, q, k, v, o4, lse, True, layer.sm_scale, outs=(dq, dk, dv))
            ops.rope_(dqkv, *layer.rope(dout.device), hq + hkv, d, S, True)
        if sp:
            dh1 = tpc.reduce_scatter_tokens(ops.linear_dgrad(dqkv, w_qkv), sp_group)
            h1, reduced = tpc.gather_tokens(h1, sp_group), tpc._Done()
        else:
            dh1, reduced = tpc.linear_dgrad_all_reduce_async(dqkv, w_qkv, tp_group)
        g_wq, g_wk, g_wv = weight_grad(dqkv, h1, [att.q_proj.weight, att.k_proj.weight, att.v_proj.weight])
        reduced.wait()
        dx, g_ln1 = rmsnorm_backward(dh1, x2, ln1.weight, rstd1, dx_mid)
        return dx.view(B, S_in, H), g_ln1, g_ln2, g_wq, g_wk, g_wv, g_wo[0], g_wg, g_wu, g_wd[0], None


class DecoderLayer(nn.Module):
    """Pre-norm residual block (``model.py:214-235``) executed as :class:`DecoderLayerFn`."""

    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.input_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.attention = Attention(config, layer_idx=layer_idx)
        self.mlp = MLP(config)
        self.layer_idx = layer_idx
        self.eps = config.rms_norm_eps
        self.head_dim = config.hidden_size // config.num_attention_heads
        self.sm_scale = 1.0 / math.sqrt(self.head_dim)
        self.rope_theta = config.rope_theta
        self.rope_scaling = getattr(config, "rope_scaling", None)      # None: plain frequencies, as the reference
        self.max_position_embeddings = config.max_position_embeddings
        self._rope_cache = {}
        self._nvtx_name = f"layer{layer_idx}/fwd"
        self._qkv_flat = None
        self._gu_flat = None

    # --- topology -------------------------------------------------------------------------
    @property
    def tp_group(self):
        g = pgm.get()
        return g.tp_group if g.tp_world_size > 1 else None

    # --- rope tables: fp32, built once per device, sliced for this CP rank ----------------
    def rope(self, device):
        key = str(device)
        if key not in self._rope_cache:
            cos, sin = ops.rope_tables(self.max_position_embeddings, self.head_dim, self.rope_theta,
                                       scaling=self.rope_scaling)
            from ..parallel.context_parallel import update_rope_for_context_parallel
            cos, sin = update_rope_for_context_parallel(cos, sin)
            self._rope_cache[key] = (cos.contiguous().to(device), sin.contiguous().to(device))
        return self._rope_cache[key]

    @property
    def cos(self):
        return self.rope(self.input_layernorm.weight.device)[0]

    @property
    def sin(self):
        return self.rope(self.input_layernorm.weight.device)[1]

    # --- packed weights -----------------------------------------------------------------------
    def packed_qkv(self) -> torch.Tensor:
        a = self.attention
        ps = [a.q_proj.weight, a.k_proj.weight, a.v_proj.weight]
        f = self._qkv_flat
        if f is None or f.data_ptr() != ps[0].data_ptr() or f.dtype != ps[0].dtype or \
                ps[1].data_ptr() != ps[0].data_ptr() + ps[0].numel() * ps[0].element_size() or \
                ps[2].data_ptr() != ps[1].data_ptr() + ps[1].numel() * ps[1].element_size():
            f = self._qkv_flat = pack_parameters(ps)
        return f

    def packed_gu(self) -> torch.Tensor:
        m = self.mlp
        ps = [m.gate_proj.weight, m.up_proj.weight]
        f = self._gu_flat
        if f is None or f.data_ptr() != ps[0].data_ptr() or f.dtype != ps[0].dtype or \
                ps[1].data_ptr() != ps[0].data_ptr() + ps[0].numel() * ps[0].element_size():
            f = self._gu_flat = pack_parameters(ps)
        return f

    def packed_param_groups(self) -> List[List[nn.Parameter]]:
        """Parameters that one GEMM consumes together; gradient buckets keep each group contiguous."""
        a, m = self.attention, self.mlp
        return [[a.q_proj.weight, a.k_proj.weight, a.v_proj.weight], [m.gate_proj.weight, m.up_proj.weight]]

    def split_qkv(self, qkv: torch.Tensor, B: int, S: int):
        a = self.attention
        hq, hkv, d = a.num_local_heads, a.num_local_kv_heads, a.head_dim
        q = qkv[:, : hq * d].view(B, S, hq, d)
        k = qkv[:, hq * d: (hq + hkv) * d].view(B, S, hkv, d)
        v = qkv[:, (hq + hkv) * d:].view(B, S, hkv, d)
        return q, k, v

    def forward(self, x, attention_mask=None, position_ids=None):
        a, m = self.attention, self.mlp
        with nvtx_range(self._nvtx_name):
            return DecoderLayerFn.apply(
                x, self.input_layernorm.weight, self.post_attention_layernorm.weight,
                a.q_proj.weight, a.k_proj.weight, a.v_proj.weight, a.out_proj.weight,
                m.gate_proj.weight, m.up_proj.weight, m.down_proj.weight, self)


# ----------------------------------------------------------------------------------------------
# fused LM head + cross entropy
# ----------------------------------------------------------------------------------------------
class LinearCrossEntropyFn(torch.autograd.Function):
    """mean-over-tokens cross entropy of ``h @ W^T`` without ever holding the ``[T, V]`` logits.

    Tokens are processed in chunks: chunk logits (GEMM whose epilogue also yields the row statistics) -> (TP: all-reduce of the
    ``[chunk]``-sized max / sum-exp / target-logit, which replaces the reference's logits all-gather,
    ``tp_communications.py:51-72``) -> in-place gradient of the chunk -> ``dh`` and ``dW`` GEMMs. The
    gradients are therefore produced during the forward pass, scaled by ``loss_scale / T``; the
    returned loss is ``loss_scale * mean CE``.

    ``need_grad=False`` (evaluation, ``torch.no_grad()``, frozen inputs) computes the loss only and
    touches no gradient buffer. In the backward pass ``dh`` is multiplied by the incoming gradient; the
    weight gradient was already accumulated (into ``weight.main_grad`` when the parameter has one) with
    the scale given at forward time and cannot be rescaled afterwards, so scale the loss through
    ``loss_scale`` rather than by multiplying the returned tensor.
    """

    @staticmethod
    def forward(ctx, h, weight, targets, head, loss_scale, chunk_tokens, need_grad=True):
        T = h.shape[0]
        tp_group, vocab_start = head.ce_partition()
        ctx.need_grad = need_grad
        dh = dw = acc = None
        if need_grad:
            dh = torch.empty_like(h)
            mg = getattr(weight, "main_grad", None)
            dw = None if mg is not None else torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
            acc = mg if mg is not None else dw
        loss_sum = torch.zeros((), dtype=torch.float32, device=h.device)
        scale = float(loss_scale) / T
        for s in range(0, T, chunk_tokens):
            e = min(T, s + chunk_tokens)
            hc, tc = h[s:e], targets[s:e]
            logits, rowmax, sumexp, tgt = ops.linear_ce_stats(hc, weight, tc, vocab_start)   # statistics from the GEMM epilogue
            ws = tpc.stats_workspace(tp_group, hc, rowmax.numel())
            if ws is not None:
                lse, tgt = ws.ce_stats_exchange(rowmax, sumexp, tgt)          # [chunk]-sized triples through peer memory
            else:
                if tp_group is not None:
                    gmax = rowmax.clone()
                    tpc.all_reduce_(gmax, tp_group, op="max")
                    sumexp = sumexp * torch.exp(rowmax - gmax)
                    packed = torch.stack([sumexp, tgt])
                    tpc.all_reduce_(packed, tp_group)
                    sumexp, tgt, rowmax = packed[0], packed[1], gmax
                lse = rowmax + torch.log(sumexp)
            loss_sum += (lse - tgt).sum()
            if need_grad:
                ops.ce_grad_(logits, tc, lse, scale, vocab_start)
                ops.linear_dgrad(logits, weight, out=dh[s:e])
                ops.linear_wgrad(logits, hc, out=acc)
            del logits
        if need_grad:
            if tp_group is not None:
                tpc.all_reduce_(dh, tp_group)
            ctx.save_for_backward(dh)
        ctx.dw = dw
        ctx.weight = weight
        return loss_sum * (float(loss_scale) / T)

    @staticmethod
    def backward(ctx, grad_out):
        if not ctx.need_grad:
            raise RuntimeError("LinearCrossEntropyFn: backward through a loss that was computed with need_grad=False")
        (dh,) = ctx.saved_tensors
        w = ctx.weight
        dh = dh * grad_out.to(dh.dtype)
        if ctx.dw is None:
            notify_grad_ready(w)
            return dh, None, None, None, None, None, None
        return dh, ctx.dw.to(w.dtype), None, None, None, None, None


# ----------------------------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------------------------
class Llama(nn.Module):
    def __init__(self, config, init: str = "reference") -> None:
        super().__init__()
        assert config.hidden_size % config.num_attention_heads == 0
        assert config.num_attention_heads % config.num_key_value_heads == 0
        self.vocab_size = config.vocab_size
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.num_key_values = config.num_key_value_heads
        self.head_dim = self.hidden_size // self.num_heads
        self.max_position_embeddings = config.max_position_embeddings
        self.num_layers = config.num_hidden_layers
        self.model_config = config
        self.init = init
        self.ce_chunk_tokens = 2048

        self.embedding = Embedding(self.vocab_size, self.hidden_size)
        self.decoder_layers = nn.ModuleList([DecoderLayer(config, layer_idx=i) for i in range(self.num_layers)])
        self.final_proj = FinalProjection(self.hidden_size, self.vocab_size, bias=False)
        self.final_norm = RMSNorm(self.hidden_size, eps=config.rms_norm_eps)
        self.reset_parameters()

    def reset_parameters(self):
        init = self.init
        self.embedding.reset_parameters(init) if isinstance(self.embedding, Embedding) else self.embedding.reset_parameters()
        for layer in self.decoder_layers:
            layer.input_layernorm.reset_parameters()
            layer.attention.reset_parameters(init)
            layer.post_attention_layernorm.reset_parameters()
            layer.mlp.reset_parameters(init)
        self.final_norm.reset_parameters()
        self.final_proj.reset_parameters(init) if isinstance(self.final_proj, Linear) else self.final_proj.reset_parameters()

    def packed_param_groups(self):
        return [g for layer in self.decoder_layers for g in layer.packed_param_groups()]

    def forward(self, input_ids, attention_mask=None, position_ids=None, target_ids=None, loss_scale: float = 1.0):
        """Logits ``[B,S,V]`` (reference signature, ``model.py:291-298``), or the fused loss when ``target_ids`` is given."""
        x = self.embedding(input_ids)
        for layer in self.decoder_layers:
            x = layer(x)
        x = gather_tokens_for_head(self.final_norm(x))
        if target_ids is None:
            return self.final_proj(x)
        return lm_head_loss(x, self.final_proj, target_ids, loss_scale, self.ce_chunk_tokens)


def gather_tokens_for_head(x: torch.Tensor) -> torch.Tensor:
    """Under sequence parallelism ``[B, S / tp, H]`` (this rank's tokens) -> ``[B, S, H]`` for the vocabulary-parallel head,
    whose input gradient comes back summed over the group, so the backward pass keeps this rank's rows. Else identity."""
    sp_group = tpc.sequence_parallel_group()
    if sp_group is None:
        return x
    B, S_in, H = x.shape
    full = tpc.GatherTokens.apply(x.reshape(B * S_in, H), sp_group)
    return full.view(B, S_in * dist.get_world_size(sp_group), H)


def head_ce_partition(head):
    """(tp group or None, first vocab id of this rank's shard) of an LM-head module."""
    if hasattr(head, "ce_partition"):
        return head.ce_partition()
    return None, 0


def lm_head_loss(x: torch.Tensor, head: nn.Module, target_ids: torch.Tensor, loss_scale: float = 1.0,
                 chunk_tokens: int = 2048) -> torch.Tensor:
    """``loss_scale * mean CE`` of the LM head applied to ``x`` ``[B,S,H]`` (fused, chunked)."""
    h = x.reshape(-1, x.shape[-1])
    need_grad = torch.is_grad_enabled() and (h.requires_grad or head.weight.requires_grad)
    return LinearCrossEntropyFn.apply(h, head.weight, target_ids.reshape(-1), _HeadView(head), loss_scale,
                                      chunk_tokens, need_grad)


class _HeadView:
    def __init__(self, head):
        self.head = head

    def ce_partition(self):
        return head_ce_partition(self.head)
