"""Ring attention with the K/V exchange inside the attention kernel.

The reference rotates K/V around the context-parallel ring with NCCL send/recv, computes one materialised
attention block per step and merges the partial results (``context_parallel.py:20-110``). Here every rank
publishes its K/V chunk in a symmetric buffer once, and ONE flash-attention kernel per rank walks over the
chunks of all ranks it may attend to: the TMA loads of that kernel read the remote chunks straight out of the
peers' memory over NVLink while the tensor cores work on the previous tile, and the online softmax of the
kernel makes the merge of partial results implicit. NVSwitch gives every pair of GPUs full bandwidth, so
pulling each chunk from its owner replaces the hop-by-hop ring without a bandwidth penalty.

Backward: the same multi-segment walk produces dQ locally and fp32 dK/dV partials for every chunk the rank
attended to; after a barrier each owner sums the partials of its chunk from the ranks that hold one.

Synchronisation: one cross-rank barrier kernel (bounded wait) after publishing K/V, one before the owner-side
reduction. K/V slots alternate between two buffers so that a rank may publish the next call's K/V while slower
peers still read the previous one.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _ext
from .workspace import SymmetricWorkspace, try_create


class RingWorkspace:
    def __init__(self, group, B: int, s: int, hkv: int, d: int):
        self.B, self.s, self.hkv, self.d = B, s, hkv, d
        self.cp = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.per = B * s * hkv * d                       # elements of one of K / V (and of dK / dV)
        self.kv_slot_bytes = 2 * self.per * 2            # K and V, bf16
        self.part_bytes = self.cp * 2 * self.per * 4     # per segment: dK and dV partials, fp32
        kv_total = (2 * self.kv_slot_bytes + 255) // 256 * 256
        self.ws: Optional[SymmetricWorkspace] = try_create(group, kv_total + self.part_bytes, num_blocks=1)
        self.part_off = kv_total
        self.calls = 0

    @property
    def ok(self) -> bool:
        return self.ws is not None

    def close(self) -> None:
        """Drop the symmetric allocation (after the work queued on it has finished)."""
        if self.ws is not None:
            torch.cuda.synchronize()
            self.ws.storage = self.ws.data = self.ws.handle = None
            self.ws = None

    def matches(self, B, s, hkv, d) -> bool:
        return (B, s, hkv, d) == (self.B, self.s, self.hkv, self.d)

    def _barrier(self):
        self.ws.barrier()

    def _publish(self, k: torch.Tensor, v: torch.Tensor):
        """Copy this rank's K/V into the next slot, barrier, return (k_ptrs, v_ptrs) of all ranks' slots."""
        ws = self.ws
        off = (self.calls % 2) * self.kv_slot_bytes
        self.calls += 1
        kv = ws.view(off, (2, self.B, self.s, self.hkv, self.d), torch.bfloat16)
        kv[0].copy_(k)
        kv[1].copy_(v)
        self._barrier()
        k_ptrs = [p + off for p in ws.buf_ptrs]
        v_ptrs = [p + off + self.per * 2 for p in ws.buf_ptrs]
        return k_ptrs, v_ptrs

    def forward(self, q, k, v, scale: float, causal: bool):
        C = _ext.load()
        k_ptrs, v_ptrs = self._publish(k, v)
        n = self.rank + 1 if causal else self.cp
        return C.attention_fwd_segs(q, k_ptrs[:n], v_ptrs[:n], self.s, self.hkv, self.hkv * self.d, causal, scale)

    def backward(self, do, q, k, v, o, lse, scale: float, causal: bool):
        C = _ext.load()
        ws = self.ws
        k_ptrs, v_ptrs = self._publish(k, v)
        n = self.rank + 1 if causal else self.cp
        seg_stride = 2 * self.per
        part_ptr = ws.data.data_ptr() + self.part_off
        dq = C.attention_bwd_segs(do, q, k_ptrs[:n], v_ptrs[:n], self.s, self.hkv, self.hkv * self.d, o, lse, None,
                                  part_ptr, seg_stride, causal, scale)
        self._barrier()                                   # every rank's partials are in place
        dk = torch.empty(self.B, self.s, self.hkv, self.d, dtype=torch.bfloat16, device=q.device)
        dv = torch.empty_like(dk)
        first = self.rank if causal else 0                # ranks first..cp-1 hold a partial for this rank's chunk
        C.reduce_dkv_symm([p + self.part_off for p in ws.buf_ptrs], self.rank * seg_stride, first, self.cp, dk, dv)
        return dq, dk, dv


# Ring workspaces per (group, shape). A run normally has one shape; evaluation with another batch or sequence length adds a
# second. Beyond MAX_CACHED shapes the least recently used workspace is closed: its references to the symmetric
# allocation are dropped so the memory returns to the driver instead of piling up with every shape change.
MAX_CACHED = 2
_CACHE: "dict[tuple, RingWorkspace]" = {}


def ring_workspace(group, B: int, s: int, hkv: int, d: int) -> Optional[RingWorkspace]:
    """The (lazily created) ring workspace of ``group`` for this problem shape, or None when unavailable.

    Creation is collective over ``group`` (every rank asks for the same shapes in the same order)."""
    key = (id(group), B, s, hkv, d)
    rw = _CACHE.pop(key, None)
    if rw is None:
        while len(_CACHE) >= MAX_CACHED:
            _CACHE.pop(next(iter(_CACHE))).close()
        rw = RingWorkspace(group, B, s, hkv, d)
    _CACHE[key] = rw                                  # most recently used last
    return rw if rw.ok else None
