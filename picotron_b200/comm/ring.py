"""Ring attention with the K/V exchange inside the attention kernel.

The reference rotates K/V around the context-parallel ring with NCCL send/recv, computes one materialised
attention block per step and merges the partial results (``context_parallel.py:20-110``). Here every rank
publishes its K/V chunk in a symmetric buffer once, and ONE flash-attention kernel per rank walks over the
chunks of all ranks it may attend to: the TMA loads of that kernel read the remote chunks straight out of the
peers' memory over NVLink while the tensor cores work on the previous tile, and the online softmax of the
kernel makes the merge of partial results implicit. NVSwitch gives every pair of GPUs full bandwidth, so
pulling each chunk from its owner replaces the hop-by-hop ring without a bandwidth penalty.

How the remote chunks reach the attention kernel is a choice (``GATHER``). The kernel can read them in place: its TMA
loads then pull every K/V tile from the owner each time a CTA needs it, and since one CTA serves one (query block,
head), a remote tile crosses NVLink once per CTA that attends to it (hundreds of times at 32K tokens). Or -- the
default -- one small copy kernel (``csrc/comm.cu: gather_peer_kernel``, plain peer loads) first brings the chunks of the
ranks this rank attends to into a local buffer, every remote byte crossing NVLink exactly once (56 MiB per layer for
cp = 8, 32K tokens, 8 KV heads: ~75 us at link speed against milliseconds of attention), and the kernel reads local
memory, where the 126 MB L2 absorbs the re-reads.

Backward: the same multi-segment walk produces dQ locally and fp32 dK/dV partials for every chunk the rank
attended to; after a barrier each owner sums the partials of its chunk from the ranks that hold one.

Synchronisation: one cross-rank barrier kernel (bounded wait) after publishing K/V, one before the owner-side
reduction. K/V slots alternate between two buffers so that a rank may publish the next call's K/V while slower
peers still read the previous one.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _ext
from .workspace import SymmetricWorkspace, try_create


# True: copy the remote K/V chunks into local memory once per call; False: the attention kernel reads them in place
import os as _os
GATHER = _os.environ.get("PICOTRON_RING_GATHER", "1") != "0"


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
        self._gathered = None                             # local copies of the other ranks' K/V chunks (lazily allocated)

    @property
    def ok(self) -> bool:
        return self.ws is not None

    def close(self) -> None:
        """Drop the symmetric allocation (after the work queued on it has finished)."""
        if self.ws is not None:
            torch.cuda.synchronize()
            self.ws.storage = self.ws.data = self.ws.handle = None
            self.ws = None
            self._gathered = None

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

    def _localize(self, k_ptrs, v_ptrs, n: int):
        """Pointers to the first ``n`` chunks with every remote one replaced by a local copy (one gather kernel)."""
        if not GATHER:
            return k_ptrs[:n], v_ptrs[:n]
        remote = [i for i in range(n) if i != self.rank]
        if not remote:
            return k_ptrs[:n], v_ptrs[:n]
        if self._gathered is None:
            self._gathered = torch.empty((self.cp - 1) * self.kv_slot_bytes, dtype=torch.uint8, device=self.ws.data.device)
        # a chunk is K followed by V in its owner's slot: one block of kv_slot_bytes per remote rank
        _ext.load().gather_peer(self._gathered, [k_ptrs[i] for i in remote], self.kv_slot_bytes)
        base = self._gathered.data_ptr()
        k_loc, v_loc = list(k_ptrs[:n]), list(v_ptrs[:n])
        for j, i in enumerate(remote):
            k_loc[i] = base + j * self.kv_slot_bytes
            v_loc[i] = base + j * self.kv_slot_bytes + self.per * 2
        return k_loc, v_loc

    def forward(self, q, k, v, scale: float, causal: bool):
        C = _ext.load()
        k_ptrs, v_ptrs = self._publish(k, v)
        n = self.rank + 1 if causal else self.cp
        k_loc, v_loc = self._localize(k_ptrs, v_ptrs, n)
        return C.attention_fwd_segs(q, k_loc, v_loc, self.s, self.hkv, self.hkv * self.d, causal, scale)

    def backward(self, do, q, k, v, o, lse, scale: float, causal: bool):
        C = _ext.load()
        ws = self.ws
        k_ptrs, v_ptrs = self._publish(k, v)
        n = self.rank + 1 if causal else self.cp
        seg_stride = 2 * self.per
        part_ptr = ws.data.data_ptr() + self.part_off
        k_loc, v_loc = self._localize(k_ptrs, v_ptrs, n)
        dq = C.attention_bwd_segs(do, q, k_loc, v_loc, self.s, self.hkv, self.hkv * self.d, o, lse, None,
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
