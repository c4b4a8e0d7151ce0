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


# Sequence layout over the CP ranks (``distributed.cp_layout``). "contiguous": rank r holds tokens [r s, (r+1) s) as the
# reference does (``data.py:105-108``), so under a causal mask rank r attends to r + 1 chunks and the last rank sets the
# pace. "zigzag": the sequence is cut into 2 cp chunks and rank r holds chunks r and 2 cp - 1 - r, which gives every rank
# the same amount of causal attention work (the load balancing the reference leaves as a TODO, ``tests/test_dataloader.py:136``).
LAYOUT = "contiguous"


def set_layout(layout: str) -> None:
    global LAYOUT
    assert layout in ("contiguous", "zigzag"), f"unknown context-parallel layout {layout!r}"
    LAYOUT = layout


def local_token_positions(seq_len: int, cp_rank: int, cp_size: int, layout: Optional[str] = None) -> torch.Tensor:
    """Global positions of the tokens CP rank ``cp_rank`` holds, in the order it holds them."""
    layout = layout or LAYOUT
    if layout == "zigzag" and cp_size > 1:
        assert seq_len % (2 * cp_size) == 0, f"zigzag layout needs seq_length ({seq_len}) divisible by 2 * cp_size"
        h = seq_len // (2 * cp_size)
        lo, hi = cp_rank, 2 * cp_size - 1 - cp_rank
        return torch.cat([torch.arange(lo * h, (lo + 1) * h), torch.arange(hi * h, (hi + 1) * h)])
    per = seq_len // cp_size
    return torch.arange(cp_rank * per, (cp_rank + 1) * per)


# Set by the trainer when ``distributed.comm == "fused"``: ring attention then runs as one kernel per rank that reads the
# peers' K/V out of symmetric memory (picotron_b200/comm/ring.py) instead of the host-driven send/recv ring below.
FUSED = False


def _fused_workspace(q, k):
    if not (FUSED and q.is_cuda and q.dtype == torch.bfloat16) or LAYOUT != "contiguous":
        return None          # (the one-kernel ring walks whole chunks in sequence order; zigzag runs the block-wise ring below)
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
    if LAYOUT == "zigzag" and g.cp_world_size > 1:
        pos = local_token_positions(seq_len, g.cp_rank, g.cp_world_size).to(cos.device)
        return cos[pos], sin[pos]
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
    if LAYOUT == "zigzag" and is_causal and pgm.get().cp_world_size > 1:
        return _zigzag_forward(q, k, v, sm_scale)
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
    if LAYOUT == "zigzag" and is_causal and pgm.get().cp_world_size > 1:
        return _zigzag_backward(do, q, k, v, o, lse, sm_scale)
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
# zigzag layout: every rank holds an early half-chunk ("lo", index r) and a late one ("hi", index 2 cp - 1 - r)
# ------------------------------------------------------------------------------------------
def _zigzag_pairs(rank: int, src: int):
    """(query half, key half, diagonal?) pairs that are visible when the K/V of rank ``src`` is at rank ``rank``.

    lo chunks are the first cp chunks of the sequence, hi chunks the last cp in reverse rank order, so: a hi query sees every
    lo key; a lo query sees the lo keys of lower ranks; a hi query sees the hi keys of HIGHER ranks; equal ranks meet on the
    diagonal. Every rank gets 2 cp + 1 half-blocks in total (the contiguous layout gives rank r 4 (r + 1) - 2 of them)."""
    pairs = [("hi", "lo", False)]
    if src < rank:
        pairs.append(("lo", "lo", False))
    elif src > rank:
        pairs.append(("hi", "hi", False))
    else:
        pairs = [("lo", "lo", True), ("hi", "lo", False), ("hi", "hi", True)]
    return pairs


def _halves(t: torch.Tensor, dim: int = 1):
    h = t.shape[dim] // 2
    return {"lo": t.narrow(dim, 0, h).contiguous(), "hi": t.narrow(dim, h, h).contiguous()}


def _zigzag_forward(q, k, v, sm_scale: float):
    comm = ContextCommunicate("fwd_kv_zigzag")
    n, rank = comm.world_size, comm.rank
    kv = torch.stack([k, v]).contiguous()
    qh = _halves(q)
    out = {"lo": None, "hi": None}
    lse = {"lo": None, "hi": None}
    for step in range(n):
        src = (rank - step) % n
        nxt = None
        if step + 1 != n:
            nxt = comm.send_recv(kv)
            comm.commit()
        kh, vh = _halves(kv[0]), _halves(kv[1])
        for qs, ks, diag in _zigzag_pairs(rank, src):
            bo, bl = ops.attention_fwd(qh[qs], kh[ks], vh[ks], diag, sm_scale)
            if out[qs] is None:
                out[qs], lse[qs] = bo.float(), bl
            else:
                ops.merge_attention_(out[qs], lse[qs], bo, bl)
        if nxt is not None:
            comm.wait()
            kv = nxt
    o = torch.cat([out["lo"], out["hi"]], dim=1).to(q.dtype)
    return o, torch.cat([lse["lo"], lse["hi"]], dim=2).contiguous()


def _zigzag_backward(do, q, k, v, o, lse, sm_scale: float):
    kv_comm = ContextCommunicate("bwd_kv_zigzag")
    dkv_comm = ContextCommunicate("bwd_dkv_zigzag")
    n, rank = kv_comm.world_size, kv_comm.rank
    kv = torch.stack([k, v]).contiguous()
    h = q.shape[1] // 2
    qh, doh, oh = _halves(q), _halves(do), _halves(o)
    lseh = _halves(lse, dim=2)
    delta = (do.float() * o.float()).sum(-1).permute(0, 2, 1).contiguous()      # [B,hq,S]
    deltah = _halves(delta, dim=2)
    dq = {"lo": None, "hi": None}
    nxt_dkv = None
    off = {"lo": 0, "hi": h}
    for step in range(n):
        src = (rank - step) % n
        nxt = None
        if step + 1 != n:
            nxt = kv_comm.send_recv(kv)
            kv_comm.commit()
        kh, vh = _halves(kv[0]), _halves(kv[1])
        blk = torch.zeros(kv.shape, dtype=torch.float32, device=kv.device)     # gradient of the K/V block we hold now
        for qs, ks, diag in _zigzag_pairs(rank, src):
            bq, bk, bv = ops.attention_bwd(doh[qs], qh[qs], kh[ks], vh[ks], oh[qs], lseh[qs], diag, sm_scale, deltah[qs])
            dq[qs] = bq.float() if dq[qs] is None else dq[qs].add_(bq)
            blk[0].narrow(1, off[ks], h).add_(bk)
            blk[1].narrow(1, off[ks], h).add_(bv)
        if step != 0:
            dkv_comm.wait()
            blk.add_(nxt_dkv)                                                   # the accumulator travels with its K/V block
        if nxt is not None:
            kv_comm.wait()
            kv = nxt
        nxt_dkv = dkv_comm.send_recv(blk)
        dkv_comm.commit()
    dkv_comm.wait()
    return torch.cat([dq["lo"], dq["hi"]], dim=1), nxt_dkv[0], nxt_dkv[1]


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
