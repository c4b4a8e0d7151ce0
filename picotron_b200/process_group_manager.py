"""The 4D process grid (data x pipeline x context x tensor) and its communicators.

Same attribute surface as the reference's ``picotron/process_group_manager.py:5-68``:
ranks are laid out as ``arange(world).view(dp, pp, cp, tp)`` (TP fastest, DP slowest), six families of
sub-groups are created collectively on every rank (tp, cp, pp, dp, cp_dp, pp_dp) and the neighbour
ranks of the CP ring and of the pipeline are derived from the grid.

Differences: the grid arithmetic lives in :class:`GridTopology`, a pure-Python object that needs no
``torch.distributed`` (so that the topology is unit-testable and usable by launch tooling), and every
group additionally carries the list of its global ranks so that the symmetric-memory runtime can build
peer tables for it.
"""
from __future__ import annotations

import contextlib
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class GridTopology:
    """Pure index arithmetic of the dp x pp x cp x tp grid (no communication)."""

    tp_size: int
    cp_size: int
    pp_size: int
    dp_size: int

    @property
    def world_size(self) -> int:
        return self.tp_size * self.cp_size * self.pp_size * self.dp_size

    def coords(self, rank: int) -> Tuple[int, int, int, int]:
        """Global rank -> (dp, pp, cp, tp)."""
        tp = rank % self.tp_size
        rank //= self.tp_size
        cp = rank % self.cp_size
        rank //= self.cp_size
        pp = rank % self.pp_size
        dp = rank // self.pp_size
        return dp, pp, cp, tp

    def rank(self, dp: int, pp: int, cp: int, tp: int) -> int:
        return ((dp * self.pp_size + pp) * self.cp_size + cp) * self.tp_size + tp

    # Each *_groups() returns the full enumeration (every rank must create every group).
    def tp_groups(self) -> List[List[int]]:
        return [[self.rank(d, p, c, t) for t in range(self.tp_size)]
                for d in range(self.dp_size) for p in range(self.pp_size) for c in range(self.cp_size)]

    def cp_groups(self) -> List[List[int]]:
        return [[self.rank(d, p, c, t) for c in range(self.cp_size)]
                for d in range(self.dp_size) for p in range(self.pp_size) for t in range(self.tp_size)]

    def pp_groups(self) -> List[List[int]]:
        return [[self.rank(d, p, c, t) for p in range(self.pp_size)]
                for d in range(self.dp_size) for c in range(self.cp_size) for t in range(self.tp_size)]

    def dp_groups(self) -> List[List[int]]:
        return [[self.rank(d, p, c, t) for d in range(self.dp_size)]
                for p in range(self.pp_size) for c in range(self.cp_size) for t in range(self.tp_size)]

    def cp_dp_groups(self) -> List[List[int]]:
        return [[self.rank(d, p, c, t) for d in range(self.dp_size) for c in range(self.cp_size)]
                for p in range(self.pp_size) for t in range(self.tp_size)]

    def pp_dp_groups(self) -> List[List[int]]:
        return [[self.rank(d, p, c, t) for d in range(self.dp_size) for p in range(self.pp_size)]
                for c in range(self.cp_size) for t in range(self.tp_size)]

    def pp_end_groups(self) -> List[List[int]]:
        """[first stage, last stage] of every pipeline: the two ranks that hold the copies of a tied embedding / LM head."""
        return [[self.rank(d, 0, c, t), self.rank(d, self.pp_size - 1, c, t)]
                for d in range(self.dp_size) for c in range(self.cp_size) for t in range(self.tp_size)]


def _new_groups(enumeration: List[List[int]], my_rank: int):
    """Create every group of ``enumeration`` (collective) and return (my group, my group's ranks)."""
    mine, mine_ids = None, None
    for ranks in enumeration:
        g = dist.new_group(ranks=ranks)
        if my_rank in ranks:
            mine, mine_ids = g, list(ranks)
    return mine, mine_ids


class ProcessGroupManager:
    def __init__(self, tp_size: int, cp_size: int, pp_size: int, dp_size: int):
        self.global_rank = dist.get_rank()
        self.world_size = dist.get_world_size()
        self.local_rank = int(os.environ.get("LOCAL_RANK", self.global_rank % max(1, self.world_size)))
        self.topology = GridTopology(tp_size, cp_size, pp_size, dp_size)
        assert self.world_size == self.topology.world_size, (
            f"World size ({self.world_size}) != TP ({tp_size}) * CP ({cp_size}) * PP ({pp_size}) * DP ({dp_size})")
        topo = self.topology
        self.grid = torch.arange(self.world_size).view(dp_size, pp_size, cp_size, tp_size)
        self.dp_rank, self.pp_rank, self.cp_rank, self.tp_rank = topo.coords(self.global_rank)

        r = self.global_rank
        self.tp_group, self.tp_group_ids = _new_groups(topo.tp_groups(), r)
        self.cp_group, self.cp_group_ids = _new_groups(topo.cp_groups(), r)
        self.pp_group, self.pp_group_ids = _new_groups(topo.pp_groups(), r)
        self.dp_group, self.dp_group_ids = _new_groups(topo.dp_groups(), r)
        self.cp_dp_group, self.cp_dp_group_ids = _new_groups(topo.cp_dp_groups(), r)
        self.pp_dp_group, self.pp_dp_group_ids = _new_groups(topo.pp_dp_groups(), r)
        self.world_group = dist.group.WORLD

        self.tp_world_size = tp_size
        self.tp_first_rank, self.tp_last_rank = self.tp_group_ids[0], self.tp_group_ids[-1]

        self.cp_world_size = cp_size
        self.cp_first_rank, self.cp_last_rank = self.cp_group_ids[0], self.cp_group_ids[-1]
        self.cp_send_rank = self.cp_group_ids[(self.cp_rank + 1) % cp_size]
        self.cp_recv_rank = self.cp_group_ids[(self.cp_rank - 1) % cp_size]

        self.pp_world_size = pp_size
        self.pp_first_rank, self.pp_last_rank = self.pp_group_ids[0], self.pp_group_ids[-1]
        self.pp_is_first_stage = self.pp_rank == 0
        self.pp_is_last_stage = self.pp_rank == pp_size - 1
        self.pp_next_rank: Optional[int] = None if self.pp_is_last_stage else topo.rank(
            self.dp_rank, self.pp_rank + 1, self.cp_rank, self.tp_rank)
        self.pp_prev_rank: Optional[int] = None if self.pp_is_first_stage else topo.rank(
            self.dp_rank, self.pp_rank - 1, self.cp_rank, self.tp_rank)

        # One 2-rank communicator per stage boundary and direction (created collectively, like the groups above): the
        # pipeline engine posts receives ahead of time, which is only safe when a communicator carries a single ordered
        # stream of messages. Keys: recv_fwd / send_bwd (with the previous stage), send_fwd / recv_bwd (with the next).
        self.pp_channel_groups: Dict[str, object] = {}
        if pp_size > 1:
            for ranks in topo.pp_groups():
                for a, b in zip(ranks[:-1], ranks[1:]):
                    g_fwd = dist.new_group(ranks=[a, b])
                    g_bwd = dist.new_group(ranks=[a, b])
                    if r == a:
                        self.pp_channel_groups.update(send_fwd=g_fwd, recv_bwd=g_bwd)
                    if r == b:
                        self.pp_channel_groups.update(recv_fwd=g_fwd, send_bwd=g_bwd)

        self.dp_world_size = dp_size
        self.dp_first_rank, self.dp_last_rank = self.dp_group_ids[0], self.dp_group_ids[-1]

        self.cp_dp_world_size = cp_size * dp_size

    def pp_ends_group(self):
        """The 2-rank group {first stage, last stage} of this rank's pipeline, or None on a middle stage.

        Created on first use, and collectively: EVERY rank of the job has to make this call (the first time) even if it
        sits on a middle stage, because creating a group is a collective over the world. Needs ``pp_size >= 2``.
        """
        assert self.pp_world_size > 1, "first and last stage are the same rank"
        if not hasattr(self, "_pp_ends_group"):
            self._pp_ends_group, self.pp_ends_group_ids = _new_groups(self.topology.pp_end_groups(), self.global_rank)
        return self._pp_ends_group

    def group_ranks(self, name: str) -> List[int]:
        """Global ranks of this rank's group ``name`` in {tp, cp, pp, dp, cp_dp, pp_dp}."""
        return list(getattr(self, f"{name}_group_ids"))

    def __str__(self) -> str:
        return (f"TP({self.tp_world_size})-CP({self.cp_world_size})-PP({self.pp_world_size})-"
                f"DP({self.dp_world_size})-Rank({self.global_rank})")


process_group_manager: Optional[ProcessGroupManager] = None


def setup_process_group_manager(tp_size: int, cp_size: int, pp_size: int, dp_size: int) -> ProcessGroupManager:
    global process_group_manager
    process_group_manager = ProcessGroupManager(tp_size, cp_size, pp_size, dp_size)
    return process_group_manager


class _SingleProcessGrid:
    """Stand-in used when no process group exists (single-process library use, unit tests).

    Every axis has size 1, every group is ``None`` (``torch.distributed`` is never called).
    """

    def __init__(self):
        self.global_rank = self.local_rank = 0
        self.world_size = 1
        self.topology = GridTopology(1, 1, 1, 1)
        self.grid = torch.zeros(1, 1, 1, 1, dtype=torch.long)
        for axis in ("tp", "cp", "pp", "dp"):
            setattr(self, f"{axis}_rank", 0)
            setattr(self, f"{axis}_world_size", 1)
            setattr(self, f"{axis}_group", None)
            setattr(self, f"{axis}_group_ids", [0])
            setattr(self, f"{axis}_first_rank", 0)
            setattr(self, f"{axis}_last_rank", 0)
        self.cp_dp_group = self.pp_dp_group = self.world_group = None
        self.cp_dp_group_ids = self.pp_dp_group_ids = [0]
        self.cp_dp_world_size = 1
        self.cp_send_rank = self.cp_recv_rank = 0
        self.pp_is_first_stage = self.pp_is_last_stage = True
        self.pp_next_rank = self.pp_prev_rank = None
        self.pp_channel_groups = {}

    def group_ranks(self, name: str) -> List[int]:
        return [0]

    def __str__(self) -> str:
        return "TP(1)-CP(1)-PP(1)-DP(1)-Rank(0)"


class LayoutGrid(_SingleProcessGrid):
    """Coordinates of ONE rank of a tp x pp grid without any communicator: enough to construct that rank's modules on
    the meta device and read off its parameter names and shard shapes (offline tools such as checkpoint resharding)."""

    def __init__(self, tp_rank: int, tp_size: int, pp_rank: int, pp_size: int):
        super().__init__()
        self.topology = GridTopology(tp_size, 1, pp_size, 1)
        self.world_size = tp_size * pp_size
        self.tp_rank, self.tp_world_size = tp_rank, tp_size
        self.pp_rank, self.pp_world_size = pp_rank, pp_size
        self.pp_is_first_stage, self.pp_is_last_stage = pp_rank == 0, pp_rank == pp_size - 1
        self.global_rank = self.topology.rank(0, pp_rank, 0, tp_rank)


@contextlib.contextmanager
def layout_grid(tp_rank: int, tp_size: int, pp_rank: int, pp_size: int):
    """Temporarily make :class:`LayoutGrid` the active grid (restores the previous one on exit)."""
    global process_group_manager
    previous = process_group_manager
    process_group_manager = LayoutGrid(tp_rank, tp_size, pp_rank, pp_size)
    try:
        yield process_group_manager
    finally:
        process_group_manager = previous


def get() -> "ProcessGroupManager":
    """The active grid; a size-1 stand-in when ``setup_process_group_manager`` was never called."""
    global process_group_manager
    if process_group_manager is None:
        return _SingleProcessGrid()  # type: ignore[return-value]
    return process_group_manager


def reset() -> None:
    """Forget the active grid (tests that build several grids in one process)."""
    global process_group_manager
    process_group_manager = None
