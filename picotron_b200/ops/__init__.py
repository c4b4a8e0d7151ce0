"""Hot ops of the framework.

Every function takes token-major 2-D activations (``[T, features]``) unless stated otherwise and
dispatches on the device of its first tensor argument: CUDA tensors go to the hand-written sm_100a
kernels of ``picotron_b200._C`` (mandatory there, see :mod:`._ext`), CPU tensors go to the PyTorch
restatements of :mod:`.reference`. The contracts are documented on the reference functions.
"""
from __future__ import annotations

import os

import math
from typing import Optional

import torch

from . import reference as ref
from . import _ext

rope_tables = ref.rope_tables


def _c():
    return _ext.load()


# ------------------------------------------------------------------ norms
def rmsnorm_fwd(x, w, eps):
    if x.is_cuda:
        return _c().rmsnorm_fwd(x, w, float(eps))
    return ref.rmsnorm_fwd(x, w, eps)


def add_rmsnorm_fwd(x, delta, w, eps):
    if x.is_cuda:
        return _c().add_rmsnorm_fwd(x, delta, w, float(eps))
    return ref.add_rmsnorm_fwd(x, delta, w, eps)


def rmsnorm_bwd(dy, x, w, rstd, dres=None, dw_acc=None):
    """Returns (dx, dw fp32). With ``dw_acc`` (fp32 [H]) the weight gradient is added to it in place and returned."""
    if x.is_cuda:
        return _c().rmsnorm_bwd(dy, x, w, rstd, dres, dw_acc)
    dx, dw = ref.rmsnorm_bwd(dy, x, w, rstd, dres)
    if dw_acc is not None:
        dw_acc.add_(dw)
        return dx, dw_acc
    return dx, dw


# ------------------------------------------------------------------ rope / swiglu
def rope_(qkv, cos, sin, n_rot_heads, head_dim, seq_len, inverse=False):
    if qkv.is_cuda:
        _c().rope_(qkv, cos, sin, int(n_rot_heads), int(head_dim), int(seq_len), bool(inverse))
        return qkv
    return ref.rope_(qkv, cos, sin, n_rot_heads, head_dim, seq_len, inverse)


def swiglu_fwd(gu):
    if gu.is_cuda:
        return _c().swiglu_fwd(gu)
    return ref.swiglu_fwd(gu)


def swiglu_bwd(gu, da):
    if gu.is_cuda:
        return _c().swiglu_bwd(gu, da)
    return ref.swiglu_bwd(gu, da)


# ------------------------------------------------------------------ GEMMs
# SwiGLU / RoPE in the epilogue of the gate-up / qkv GEMM (env PICOTRON_FUSE_EPILOGUE=0 keeps the separate kernels)
FUSE_GEMM_EPILOGUES = os.environ.get("PICOTRON_FUSE_EPILOGUE", "1") != "0"

def _use_tc(*ts) -> bool:
    """True for CUDA operands (which must then be bf16: the kernels have no other precision), False for CPU operands."""
    if not ts[0].is_cuda:
        return False
    for t in ts:
        if t.dtype != torch.bfloat16:
            raise TypeError(f"picotron_b200 CUDA kernels take bf16 operands, got {t.dtype}; run fp32 models on the CPU "
                            "path (distributed.use_cpu) or cast to bf16")
    return True


def linear_swiglu_fwd(x, w_gu):
    """``gu = x @ w_gu^T`` ([T, 2I], gate | up) and ``h = silu(gate) * up`` ([T, I]).

    On the GPU one GEMM whose epilogue also produces ``h`` (when the kernel covers the shape), else GEMM + activation.
    """
    if _use_tc(x, w_gu) and FUSE_GEMM_EPILOGUES:
        r = _c().gemm_swiglu(x, w_gu)
        if r:
            return r[0], r[1]
    gu = linear_fwd(x, w_gu)
    return gu, swiglu_fwd(gu)


def linear_rope_fwd(x, w_qkv, cos, sin, n_rot_heads, head_dim, seq_len):
    """Packed ``qkv = x @ w_qkv^T`` with RoPE applied to the first ``n_rot_heads`` heads (q and k)."""
    if _use_tc(x, w_qkv) and FUSE_GEMM_EPILOGUES:
        r = _c().gemm_rope(x, w_qkv, cos, sin, int(n_rot_heads), int(head_dim), int(seq_len))
        if r is not None:
            return r
    qkv = linear_fwd(x, w_qkv)
    return rope_(qkv, cos, sin, n_rot_heads, head_dim, seq_len, False)


def linear_add_fwd(x, w, res):
    """``x @ w^T + res`` (a projection followed by the residual add); on the GPU one GEMM with the add in its epilogue."""
    if _use_tc(x, w, res) and FUSE_GEMM_EPILOGUES:
        y = _c().gemm_add(x, w, res)
        if y is not None:
            return y
    return add(res, linear_fwd(x, w))


def linear_dgrad_swiglu_bwd(dy, w_down, gu):
    """Gradient of the packed SwiGLU pre-activations ``gu`` ([T, 2I]) given ``dy`` ([T, H]) behind the down projection
    ``w_down`` ([H, I]): ``swiglu_bwd(gu, dy @ w_down)``. On the GPU the activation backward runs in the epilogue of the
    dgrad GEMM (``dy @ w_down`` is never written)."""
    if _use_tc(dy, w_down, gu) and FUSE_GEMM_EPILOGUES:
        dgu = _c().gemm_dgrad_swiglu_bwd(dy, w_down, gu)
        if dgu is not None:
            return dgu
    return swiglu_bwd(gu, linear_dgrad(dy, w_down))


def linear_fwd(x, w, out: Optional[torch.Tensor] = None):
    """``x[T,K] @ w[N,K]^T`` -> ``[T,N]`` (written into ``out`` when given)."""
    if _use_tc(x, w):
        return _c().gemm(x, w, False, False, out, False)
    y = ref.linear_fwd(x, w)
    return y if out is None else out.copy_(y)


def linear_dgrad(dy, w, out: Optional[torch.Tensor] = None):
    """``dy[T,N] @ w[N,K]`` -> ``[T,K]`` (written into ``out`` when given)."""
    if _use_tc(dy, w):
        return _c().gemm(dy, w, False, True, out, False)
    y = ref.linear_dgrad(dy, w)
    return y if out is None else out.copy_(y)


def linear_wgrad(dy, x, out: Optional[torch.Tensor] = None):
    """``dy[T,N]^T @ x[T,K]`` -> ``[N,K]``; accumulated into ``out`` (fp32) when given."""
    if _use_tc(dy, x):
        if out is None:
            return _c().gemm(dy, x, True, True, None, False)
        _c().gemm(dy, x, True, True, out, True)
        return None
    return ref.linear_wgrad(dy, x, out)


# ------------------------------------------------------------------ attention
def attention_fwd(q, k, v, causal: bool, scale: Optional[float] = None):
    scale = float(scale if scale is not None else 1.0 / math.sqrt(q.shape[-1]))
    if _use_tc(q, k, v):
        return _c().attention_fwd(q, k, v, bool(causal), scale)
    return ref.attention_fwd(q, k, v, causal, scale)


def attention_bwd_fuses_rope(q) -> bool:
    """True when :func:`attention_bwd` can undo RoPE on dq / dk itself (``rope=(cos, sin)``)."""
    return bool(q.is_cuda and q.dtype == torch.bfloat16 and FUSE_GEMM_EPILOGUES)


def attention_bwd(do, q, k, v, o, lse, causal: bool, scale: Optional[float] = None, delta=None, outs=None, rope=None):
    """Returns ``(dq, dk, dv)``; with ``outs=(dq, dk, dv)`` the results are written into those (strided) views.

    ``rope=(cos, sin)`` (only where :func:`attention_bwd_fuses_rope`) applies the inverse rotary rotation to dq and dk.
    """
    scale = float(scale if scale is not None else 1.0 / math.sqrt(q.shape[-1]))
    if _use_tc(q, k, v, do):
        cos, sin = rope if rope is not None else (None, None)
        return _c().attention_bwd(do, q, k, v, o, lse, bool(causal), scale, delta,
                                  list(outs) if outs is not None else None, cos, sin)
    assert rope is None, "rope fusion is only available on the GPU"
    res = ref.attention_bwd(do, q, k, v, o, lse, causal, scale, delta)
    if outs is not None:
        for dst, src in zip(outs, res):
            dst.copy_(src)
        return tuple(outs)
    return res


# ------------------------------------------------------------------ embedding
def embedding_fwd(ids, w, vocab_start: int = 0):
    if w.is_cuda:
        return _c().embedding_fwd(ids.reshape(-1), w, int(vocab_start))
    return ref.embedding_fwd(ids, w, vocab_start)


def embedding_bwd(ids, dy, dw, vocab_start: int = 0):
    if dw.is_cuda:
        _c().embedding_bwd(ids.reshape(-1), dy, dw, int(vocab_start))
        return
    ref.embedding_bwd(ids, dy, dw, vocab_start)


# ------------------------------------------------------------------ cross entropy
def ce_stats(logits, targets, vocab_start: int = 0):
    if logits.is_cuda:
        return _c().ce_stats(logits, targets, int(vocab_start))
    return ref.ce_stats(logits, targets, vocab_start)


def linear_ce_stats(x, w, targets, vocab_start: int = 0):
    """``logits = x @ w^T`` and the row statistics of :func:`ce_stats` -> ``(logits, rowmax, sumexp, target_logit)``.

    On the GPU the statistics come out of the GEMM's epilogue (per 256-column tile, merged by a small kernel), so the
    logits are not read again before the gradient pass."""
    if _use_tc(x, w) and FUSE_GEMM_EPILOGUES:
        r = _c().gemm_ce_stats(x, w, targets, int(vocab_start))
        if r:
            return r[0], r[1], r[2], r[3]
    logits = linear_fwd(x, w)
    return (logits,) + tuple(ce_stats(logits, targets, vocab_start))


def ce_grad_(logits, targets, lse, scale: float, vocab_start: int = 0):
    if logits.is_cuda:
        _c().ce_grad_(logits, targets, lse, float(scale), int(vocab_start))
        return logits
    return ref.ce_grad_(logits, targets, lse, scale, vocab_start)


def add(a, b):
    """``a + b`` (residual add)."""
    if a.is_cuda and a.dtype == torch.bfloat16:
        return _c().add(a, b)
    return a + b


# ------------------------------------------------------------------ grads / optimizer / merge
def accumulate_(main_grad, grad):
    if main_grad.is_cuda:
        _c().accumulate_(main_grad, grad)
        return
    ref.accumulate_(main_grad, grad)


def merge_attention_(out, lse, block_out, block_lse):
    if out.is_cuda:
        _c().merge_attention_(out, lse, block_out, block_lse)
        return out, lse
    return ref.merge_attention_(out, lse, block_out, block_lse)


# ------------------------------------------------------------------ checked mode
_CHECKED_OPS = ("rmsnorm_fwd", "add_rmsnorm_fwd", "rmsnorm_bwd", "rope_", "swiglu_fwd", "swiglu_bwd", "linear_swiglu_fwd",
                "linear_rope_fwd", "linear_add_fwd", "linear_dgrad_swiglu_bwd", "linear_fwd", "linear_dgrad", "linear_wgrad", "attention_fwd", "attention_bwd",
                "embedding_fwd", "embedding_bwd", "ce_stats", "linear_ce_stats", "ce_grad_", "add", "accumulate_", "merge_attention_")
_UNCHECKED = {}


def _tensors_of(x):
    if torch.is_tensor(x):
        yield x
    elif isinstance(x, (list, tuple)):
        for y in x:
            yield from _tensors_of(y)


def enable_checked_mode(on: bool = True, check_finite: bool = True) -> None:
    """Debug aid (``PICOTRON_CHECKED_OPS=1``): every op of this module is followed by a device synchronisation, a read of
    the kernel status word (a bounded wait that gave up inside a kernel) and, optionally, a finiteness check of its
    floating-point results, and raises naming the op. It replaces what a sanitizer run would give on a machine where
    none is available: the first op that misbehaves is reported instead of a corrupted loss thousands of launches later.
    Slow (one host synchronisation per op); never enable it for timing runs or under CUDA-graph capture.
    """
    g = globals()
    if not on:
        for name, fn in _UNCHECKED.items():
            g[name] = fn
        _UNCHECKED.clear()
        return
    if _UNCHECKED:
        return

    def wrap(name, fn):
        def checked(*args, **kwargs):
            out = fn(*args, **kwargs)
            on_gpu = any(t.is_cuda for t in _tensors_of(list(args) + list(kwargs.values())))
            if on_gpu:
                torch.cuda.synchronize()
                status = _c().kernel_status()
                if status:
                    raise RuntimeError(f"ops.{name}: a kernel gave up a bounded wait (status {status:#x}: kernel id "
                                       f"{status >> 24}, site {(status >> 16) & 0xff}, block {status & 0xffff})")
            if check_finite:
                for t in _tensors_of(out):
                    if t.is_floating_point() and t.numel() and not bool(torch.isfinite(t).all()):
                        raise FloatingPointError(f"ops.{name}: non-finite values in a result of shape {tuple(t.shape)}")
            return out
        checked.__name__, checked.__doc__ = fn.__name__, fn.__doc__
        return checked

    for name in _CHECKED_OPS:
        _UNCHECKED[name] = g[name]
        g[name] = wrap(name, g[name])


if os.environ.get("PICOTRON_CHECKED_OPS", "0") == "1":
    enable_checked_mode(True)
