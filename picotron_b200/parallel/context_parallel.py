"""Context parallelism: ring attention over contiguous sequence chunks.

Behaviour of the reference (``context_parallel.py:14-195``): the sequence is cut into ``cp`` contiguous
chunks; attention rotates K/V around the CP ring, attends block by block and merges the partial
results with their log-sum-exp; causality is handled by skipping blocks that come from later ranks
(``step <= rank``) and masking only the diagonal block; the backward pass rotates K/V again while a
second ring carries the fp32 dK/dV accumulators home.

Differences: blocks are computed by the flash-attention op (no ``s x s`` score matrix is
materialised), K and V travel as one packed message in their ``hkv`` heads (the reference expands GQA
heads first, ``model.py:142-143``, which quadruples the traffic for 32q/8kv), ``delta = rowsum(dO*O)``
is computed once, and no host/device synchronisation happens per ring step.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import ops
from .. import process_group_manager as pgm
from .cp_communications import ContextCommunicate
from ..utils.tracing import nvtx_range


# Set by the trainer when ``distributed.comm == "fused"``: ring attention then runs as one kernel per rank that reads the
# peers' K/V out of symmetric memory (picotron_b200/comm/ring.py) instead of the host-driven send/recv ring below.
FUSED = False


def _fused_workspace(q, k):
    if not (FUSED and q.is_cuda and q.dtype == torch.bfloat16):
        return None
    g = pgm.get()
    if g.cp_world_size == 1 or g.cp_world_size > 8:
        return None
    from ..comm.ring import ring_workspace
    B, s, hkv, d = k.shape
    return ring_workspace(g.cp_group, B, s, hkv, d)


def apply_context_parallel(model):
    """Switch the attention of every decoder layer to ring attention when ``cp_world_size > 1``."""
    on = pgm.get().cp_world_size > 1
    for m in model.modules():
        if hasattr(m, "cp_enabled"):
            m.cp_enabled = on
    return model


def update_rope_for_context_parallel(cos: torch.Tensor, sin: torch.Tensor):
    """Slice the RoPE tables to this CP rank's contiguous positions (``context_parallel.py:189-195``)."""
    g = pgm.get()
    seq_len = cos.shape[0]
    assert seq_len % g.cp_world_size == 0, (
        f"Input sequence length ({seq_len}) must be divisible by cp_world_size ({g.cp_world_size})")
    per = seq_len // g.cp_world_size
    return cos[g.cp_rank * per:(g.cp_rank + 1) * per], sin[g.cp_rank * per:(g.cp_rank + 1) * per]


# ------------------------------------------------------------------------------------------
# block-level ring on [B, S, heads, d] tensors with native GQA (what the fused layer calls)
# ------------------------------------------------------------------------------------------
def ring_attention_forward_blocks(q, k, v, sm_scale: float, is_causal: bool):
    """Returns ``(o [B,S,hq,d] in q.dtype, lse [B,hq,S] fp32)`` of attention over the whole CP sequence."""
    rw = _fused_workspace(q, k)
    if rw is not None:
        with nvtx_range("ring_attention/fwd"):
            return rw.forward(q, k, v, sm_scale, is_causal)
    comm = ContextCommunicate("fwd_kv")
    n, rank = comm.world_size, comm.rank
    kv = torch.stack([k, v]).contiguous()                 # [2,B,S,hkv,d], one message per step
    out = lse = None
    for step in range(n):
        nxt = None
        if step + 1 != n:
            nxt = comm.send_recv(kv)
            comm.commit()
        if not is_causal or step <= rank:
            bo, bl = ops.attention_fwd(q, kv[0], kv[1], is_causal and step == 0, sm_scale)
            if out is None:
                out, lse = bo.float(), bl
            else:
                ops.merge_attention_(out, lse, bo, bl)
        if nxt is not None:
            comm.wait()
            kv = nxt
    return out.to(q.dtype), lse


def ring_attention_backward_blocks(do, q, k, v, o, lse, sm_scale: float, is_causal: bool):
    """Returns ``dq`` and the ``dk``, ``dv`` of this rank's own K/V chunk (fp32 on the host-driven ring)."""
    rw = _fused_workspace(q, k)
    if rw is not None:
        with nvtx_range("ring_attention/bwd"):
            return rw.backward(do.contiguous(), q, k, v, o.contiguous(), lse, sm_scale, is_causal)
    kv_comm = ContextCommunicate("bwd_kv")
    dkv_comm = ContextCommunicate("bwd_dkv")
    n, rank = kv_comm.world_size, kv_comm.rank
    kv = torch.stack([k, v]).contiguous()
    delta = (do.float() * o.float()).sum(-1).permute(0, 2, 1).contiguous()      # [B,hq,S]
    dq = None
    dkv = None          # accumulator that travels with the K/V block it belongs to
    nxt_dkv = None
    for step in range(n):
        nxt = None
        if step + 1 != n:
            nxt = kv_comm.send_recv(kv)
            kv_comm.commit()
        if not is_causal or step <= rank:
            bq, bk, bv = ops.attention_bwd(do, q, kv[0], kv[1], o, lse, is_causal and step == 0, sm_scale, delta)
            dq = bq.float() if dq is None else dq.add_(bq)
            blk = torch.stack([bk.float(), bv.float()])
            if step == 0:
                dkv = blk
            else:
                dkv_comm.wait()
                dkv = blk.add_(nxt_dkv)
        elif step != 0:
            dkv_comm.wait()
            dkv = nxt_dkv
        if nxt is not None:
            kv_comm.wait()
            kv = nxt
        nxt_dkv = dkv_comm.send_recv(dkv)
        dkv_comm.commit()
    dkv_comm.wait()
    return dq, nxt_dkv[0], nxt_dkv[1]


# ------------------------------------------------------------------------------------------
# reference-shaped public API: [B, H, s, d] tensors, autograd function
# ------------------------------------------------------------------------------------------
class RingAttentionFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, sm_scale, is_causal):
        qb, kb, vb = (t.transpose(1, 2).contiguous() for t in (q, k, v))       # -> [B,S,h,d]
        o, lse = ring_attention_forward_blocks(qb, kb, vb, sm_scale, is_causal)
        ctx.save_for_backward(qb, kb, vb, o, lse)
        ctx.sm_scale, ctx.is_causal = sm_scale, is_causal
        return o.transpose(1, 2)

    @staticmethod
    def backward(ctx, dout):
        qb, kb, vb, o, lse = ctx.saved_tensors
        dob = dout.transpose(1, 2).contiguous()
        dq, dk, dv = ring_attention_backward_blocks(dob, qb, kb, vb, o, lse, ctx.sm_scale, ctx.is_causal)
        return (dq.transpose(1, 2).to(qb.dtype), dk.transpose(1, 2).to(kb.dtype),
                dv.transpose(1, 2).to(vb.dtype), None, None)


def ring_attention(q, k, v, sm_scale, is_causal):
    """Ring attention on ``[B, H, s, d]`` tensors (K/V may have fewer heads than Q: native GQA)."""
    return RingAttentionFunc.apply(q, k, v, sm_scale, is_causal)


def ring_attention_forward(q, k, v, sm_scale, is_causal):
    """One attention block on ``[B,H,s,d]`` tensors -> ``(O, LSE [B,H,s])`` (``context_parallel.py:112-128``)."""
    o, lse = ops.attention_fwd(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal, sm_scale)
    return o.transpose(1, 2), lse


def ring_attention_backward(dO, Q, K, V, O, softmax_lse, sm_scale, is_causal):
    """Block backward from a global LSE on ``[B,H,s,d]`` tensors (``context_parallel.py:130-155``)."""
    t = lambda x: x.transpose(1, 2)
    dq, dk, dv = ops.attention_bwd(t(dO), t(Q), t(K), t(V), t(O), softmax_lse, is_causal, sm_scale)
    return t(dq), t(dk), t(dv)


def update_out_and_lse(out: Optional[torch.Tensor], lse: Optional[torch.Tensor], block_out: torch.Tensor,
                       block_lse: torch.Tensor, slice_=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Merge a block result into the running ``(out [B,H,s,d] fp32, lse [B,H,s,1])`` (``context_parallel.py:157-187``)."""
    block_out = block_out.to(torch.float32)
    block_lse = block_lse.unsqueeze(-1)
    if out is None:
        if slice_ is not None:
            raise RuntimeError("first update_out_and_lse should not pass slice_ args")
        return block_out, block_lse
    sl = slice_ if slice_ is not None else slice(None)
    o, l = out[sl], lse[sl]
    bo, bl = (block_out, block_lse) if slice_ is None else (block_out, block_lse)
    new_o = o - torch.sigmoid(bl - l) * (o - bo)
    new_l = l - torch.nn.functional.logsigmoid(l - bl)
    if slice_ is not None:
        out[sl], lse[sl] = new_o, new_l
        return out, lse
    return new_o, new_l
