"""Symmetric-memory workspaces: one allocation mapped at every rank of a process group.

A workspace owns a flag region (cross-rank barriers of the collective kernels) and a data region. The data
region is either handed out whole (the fp32 gradient buckets of the data-parallel engine live in it) or as a
small ring of slots (row-parallel GEMM outputs and column-parallel input gradients of the tensor-parallel
layers are written straight into a slot by the GEMM and all-reduced there in place).

Allocation and the exchange of peer mappings use ``torch.distributed._symmetric_memory`` (CUDA virtual memory
management with an NVSwitch multicast mapping when the fabric supports it); the collectives themselves are
this package's kernels (``csrc/comm.cu``), launched on the caller's stream. The epoch that tells one call's flags from
the previous call's is a counter in the workspace's own device memory, advanced by the kernels themselves: nothing about
a launch changes from call to call, so the collectives can be captured in CUDA graphs and replayed. The price is a
rule: all launches on one workspace are issued on one stream (or otherwise ordered), and every rank issues the same
sequence of them. If symmetric memory cannot be set up the callers keep using NCCL.
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _ext

FLAG_BYTES = 2 * 8 * 128 * 4          # barrier flags [phase][rank][block] uint32, see csrc/comm.cu
CTRL_OFFSET = FLAG_BYTES              # two uint32 control words behind them: the workspace's call counter and a CTA arrival count
# 16 KiB of barrier flags and control words, then the per-tile flags of the fused GEMM+all-reduce kernel
# (csrc/gemm_allreduce_tcgen05.cu: 1024 tiles x 2 halves x (8 start words + 1 done word)), padded to 128 KiB
FLAG_REGION = 131072
# Guard words: the last CANARY_BYTES of the flag region (padding no kernel uses) and CANARY_BYTES appended behind the data
# region are filled with a pattern at creation; `check_canaries()` verifies them from the host. A peer or a local
# kernel that writes past the end of the flags or of the data region (an off-by-one tile, a wrong element offset)
# shows up there instead of silently corrupting a neighbour allocation.
CANARY_BYTES = 256
CANARY_VALUE = 0xA5


class SymmetricWorkspace:
    def __init__(self, group, data_bytes: int, num_blocks: int = 32, use_multicast: Optional[bool] = None,
                 staging_bytes: int = 0):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.num_blocks = num_blocks
        self.data_bytes = int(data_bytes)
        # staging area of the push all-reduce (csrc/comm.cu), behind the data region: peers store their contributions to
        # this rank's slice here. Unused (and best left at 0) when the multicast path is taken.
        self.staging_bytes = (int(staging_bytes) + 255) // 256 * 256
        self.staging_off = (self.data_bytes + 255) // 256 * 256
        dev = torch.device("cuda", torch.cuda.current_device())
        body = self.staging_off + self.staging_bytes if self.staging_bytes else self.data_bytes
        self._body_bytes = body
        total = FLAG_REGION + body + CANARY_BYTES
        try:
            symm_mem.enable_symm_mem_for_group(group.group_name)
        except Exception:  # noqa: BLE001  (newer releases enable every group implicitly)
            pass
        self.storage = symm_mem.empty(total, dtype=torch.uint8, device=dev)
        self.storage.zero_()
        self.storage[FLAG_REGION - CANARY_BYTES:FLAG_REGION].fill_(CANARY_VALUE)
        self.storage[FLAG_REGION + body:].fill_(CANARY_VALUE)
        self.handle = symm_mem.rendezvous(self.storage, group.group_name)
        base_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.flag_ptrs: List[int] = base_ptrs
        self.buf_ptrs: List[int] = [p + FLAG_REGION for p in base_ptrs]
        if use_multicast is None:
            # measured: with 2 ranks plain peer loads/stores beat the switch reduction, which pays off from 4 ranks up
            env = os.environ.get("PICOTRON_MULTIMEM")
            use_multicast = (env != "0") if env is not None else self.world > 2
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.mc_ptr = (mc + FLAG_REGION) if (use_multicast and mc != 0) else 0
        self.data = self.storage[FLAG_REGION:FLAG_REGION + self.data_bytes]
        self._gemm_clusters = None
        self._ring_slot_bytes = 0
        self._ring_slots = 0
        self._ring_next = 0
        torch.cuda.synchronize()
        dist.barrier(group=group)              # every rank zeroed its flags before anyone signals

    # ------------------------------------------------------------------ guard words
    def check_canaries(self) -> None:
        """Raise if a guard word behind the flag or data region of THIS rank's buffer was overwritten (host read, syncs)."""
        lo = self.storage[FLAG_REGION - CANARY_BYTES:FLAG_REGION]
        hi = self.storage[FLAG_REGION + self._body_bytes:FLAG_REGION + self._body_bytes + CANARY_BYTES]
        bad = [name for name, t in (("flag region", lo), ("data region", hi)) if not bool((t == CANARY_VALUE).all().item())]
        if bad:
            raise RuntimeError(f"symmetric workspace of rank {self.rank}: guard words behind the {' and the '.join(bad)} "
                               "were overwritten (an out-of-bounds write by a collective kernel or a peer)")

    # ------------------------------------------------------------------ views
    def view(self, offset_bytes: int, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        assert offset_bytes % 16 == 0 and offset_bytes + nbytes <= self.data_bytes
        return self.data[offset_bytes:offset_bytes + nbytes].view(dtype).view(*shape)

    def configure_ring(self, slots: int, slot_bytes: int) -> None:
        assert slots * slot_bytes <= self.data_bytes
        self._ring_slots, self._ring_slot_bytes, self._ring_next = slots, slot_bytes, 0

    def ring_alloc(self, shape, dtype) -> Optional[torch.Tensor]:
        """Next slot of the ring as a tensor, or None when the request does not fit a slot."""
        n = 1
        for s in shape:
            n *= s
        if self._ring_slots == 0 or n * torch.empty(0, dtype=dtype).element_size() > self._ring_slot_bytes:
            return None
        off = self._ring_next * self._ring_slot_bytes
        self._ring_next = (self._ring_next + 1) % self._ring_slots
        return self.view(off, shape, dtype)

    def configure_scratch(self, offset_bytes: int, nbytes: int) -> None:
        """Reserve ``nbytes`` of the data region (two halves used alternately) for small per-call exchanges."""
        assert offset_bytes % 256 == 0 and offset_bytes + nbytes <= self.data_bytes
        self._scratch_off, self._scratch_half, self._scratch_calls = offset_bytes, nbytes // 2 // 256 * 256, 0

    def can_exchange_ce_stats(self, n: int) -> bool:
        return getattr(self, "_scratch_half", 0) >= 3 * n * 4

    def ce_stats_exchange(self, rowmax: torch.Tensor, sumexp: torch.Tensor, tgt: torch.Tensor):
        """Vocabulary-parallel cross entropy: ``(lse, target_logit)`` over the whole vocabulary from this shard's row
        statistics. Every rank stores its triple in its own half of the scratch area, a barrier makes them visible, and each
        rank combines all triples with peer loads (``csrc/comm.cu``). The halves alternate, so the next call's stores cannot
        overtake a slow peer that still reads this call's (it has to pass the next barrier first)."""
        n = rowmax.numel()
        off = self._scratch_off + (self._scratch_calls % 2) * self._scratch_half
        self._scratch_calls += 1
        st = self.view(off, (3, n), torch.float32)
        st[0].copy_(rowmax)
        st[1].copy_(sumexp)
        st[2].copy_(tgt)
        self.barrier()
        lse, t = _ext.load().ce_stats_combine_peers(self.buf_ptrs, off, n, st)
        # close the call with a second barrier: eager calls alternate the halves, but a captured sequence replays with the
        # half it was captured with, and no rank may store the next triple while a peer still reads this one
        self.barrier()
        return lse, t

    # ------------------------------------------------------------------ collectives
    def barrier(self) -> None:
        """Every rank of the group reached this point of its stream (one small kernel, bounded wait)."""
        _ext.load().symm_barrier(self.flag_ptrs, self.rank, self.world)

    def calls(self) -> int:
        """Number of collective calls completed on this workspace (reads the device counter: synchronises)."""
        return int(self.storage[CTRL_OFFSET:CTRL_OFFSET + 4].view(torch.int32).item()) & 0xFFFFFFFF

    def contains(self, t: torch.Tensor) -> bool:
        lo = self.data.data_ptr()
        return t.is_cuda and t.is_contiguous() and lo <= t.data_ptr() and \
            t.data_ptr() + t.numel() * t.element_size() <= lo + self.data_bytes

    def can_all_reduce(self, t: torch.Tensor) -> bool:
        return self.contains(t) and t.dtype in (torch.bfloat16, torch.float32) and \
            (t.data_ptr() - self.data.data_ptr()) % 16 == 0

    def gemm_all_reduce(self, a: torch.Tensor, b: torch.Tensor, trans_b: bool, out: torch.Tensor) -> torch.Tensor:
        """``out = sum over ranks of a @ op(b)`` in one kernel (GEMM tiles reduced over NVLink while later tiles compute).

        ``out`` must be a 2-D bf16 tensor inside this workspace; ``b`` is ``[N,K]`` (``trans_b=False``) or ``[K,N]``.
        """
        assert self.contains(out) and out.dtype == torch.bfloat16 and out.dim() == 2
        if self._gemm_clusters is None:
            # tile ownership depends on the grid: agree on the smallest CTA-pair capacity of the group once
            n = torch.tensor([_ext.load().gemm_allreduce_max_clusters()], dtype=torch.int64, device=out.device)
            dist.all_reduce(n, op=dist.ReduceOp.MIN, group=self.group)
            self._gemm_clusters = int(n.item())
            assert self._gemm_clusters > 0, "CTA pairs cannot be scheduled on this device"
        off = (out.data_ptr() - self.data.data_ptr()) // 2
        _ext.load().gemm_allreduce(a, b, False, bool(trans_b), out, self.buf_ptrs, self.flag_ptrs, self.mc_ptr, off, self.rank,
                                   self.world, self._gemm_clusters)
        return out

    def all_reduce_(self, t: torch.Tensor, scale: float = 1.0, blocks: Optional[int] = None) -> torch.Tensor:
        """In-place sum over the group (times ``scale`` for fp32) of a tensor that lives in this workspace.

        ``blocks`` caps the grid (a call that overlaps a GEMM leaves most SMs to it); every rank must pass the same value."""
        assert self.can_all_reduce(t)
        esize = t.element_size()
        off = (t.data_ptr() - self.data.data_ptr()) // esize
        cap = self.num_blocks if blocks is None else min(blocks, 128)
        C = _ext.load()
        is_bf16 = t.dtype == torch.bfloat16
        nbytes = t.numel() * esize
        if self.mc_ptr == 0 and self.staging_bytes and self.world > 1 and nbytes % 16 == 0:
            # push variant: pieces whose (world - 1) staged slices fit the staging area
            piece = self.staging_bytes // (self.world - 1) // 16 * 16 * self.world
            done = 0
            while done < nbytes:
                cur = min(piece, nbytes - done)
                grid = max(1, min(cap, (cur // self.world + 65535) // 65536))
                C.allreduce_symm(self.buf_ptrs, self.flag_ptrs, 0, off + done // esize, cur // esize, is_bf16, float(scale),
                                 self.rank, self.world, grid, self.staging_off)
                done += cur
            return t
        # one block moves 64 KiB per sweep (512 threads x 16 B x 8 in flight); cap at this workspace's block budget
        per_rank_bytes = nbytes // self.world
        grid = max(1, min(cap, (per_rank_bytes + 65535) // 65536))
        C.allreduce_symm(self.buf_ptrs, self.flag_ptrs, self.mc_ptr, off, t.numel(), is_bf16, float(scale), self.rank,
                         self.world, grid, 0)
        return t


def group_is_on_one_node(group) -> bool:
    """True when every rank of ``group`` runs on this host (peer memory only reaches GPUs of the same NVLink domain; a
    group that spans hosts keeps its collectives on NCCL). Collective over the group; if the exchange itself fails the
    answer is True and the symmetric-memory rendezvous decides."""
    import socket
    try:
        hosts = [None] * dist.get_world_size(group)
        dist.all_gather_object(hosts, socket.gethostname(), group=group)
        return len(set(hosts)) == 1
    except Exception:  # noqa: BLE001
        return True


def try_create(group, data_bytes: int, **kw) -> Optional[SymmetricWorkspace]:
    """A workspace, or None (with one warning on rank 0) when symmetric memory is unavailable or the group spans hosts."""
    if not group_is_on_one_node(group):
        if dist.get_rank() == 0:
            print("[picotron_b200] a process group spans several hosts: its collectives use NCCL")
        return None
    try:
        return SymmetricWorkspace(group, data_bytes, **kw)
    except Exception as e:  # noqa: BLE001
        if dist.get_rank() == 0:
            print(f"[picotron_b200] symmetric memory unavailable ({type(e).__name__}: {e}); using NCCL collectives")
        return None
