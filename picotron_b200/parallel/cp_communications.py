"""Ring send/recv helper for context parallelism.

Same surface as the reference's ``ContextCommunicate`` (``cp_communications.py:10-54``):
``send_recv`` queues an isend to the next CP rank and an irecv from the previous one, ``commit`` issues
the batch, ``wait`` completes it. Unlike the reference, ``wait`` does not synchronise the device: NCCL
requests are stream-ordered, so the consumer kernels simply queue behind the transfer.
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import process_group_manager as pgm

VERBOSE = os.environ.get("VERBOSE", "0") == "1"


class ContextCommunicate:
    def __init__(self, msg: str = ""):
        g = pgm.get()
        self._pending: List[dist.P2POp] = []
        self._active = None
        self.msg = msg
        self.rank = g.cp_rank
        self.world_size = g.cp_world_size
        self.send_rank = g.cp_send_rank
        self.recv_rank = g.cp_recv_rank
        self.group = g.cp_group
        if VERBOSE:
            print(f"RingComm ({msg}) | init | rank {self.rank}/{self.world_size} | send->{self.send_rank} | "
                  f"recv<-{self.recv_rank}", flush=True)

    def send_recv(self, tensor_to_send: torch.Tensor, recv_tensor: Optional[torch.Tensor] = None) -> torch.Tensor:
        result = torch.empty_like(tensor_to_send) if recv_tensor is None else recv_tensor
        self._pending.append(dist.P2POp(dist.isend, tensor_to_send, self.send_rank, group=self.group))
        self._pending.append(dist.P2POp(dist.irecv, result, self.recv_rank, group=self.group))
        return result

    def commit(self) -> None:
        if self._active is not None:
            raise RuntimeError("Commit called twice")
        self._active = dist.batch_isend_irecv(self._pending)

    def wait(self) -> None:
        if self._active is None:
            raise RuntimeError("Wait called before commit")
        for req in self._active:
            req.wait()
        self._active = None
        self._pending = []
