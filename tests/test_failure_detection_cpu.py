"""Failure detection on the host: a rank that never joins a collective makes the others raise, not hang."""
import datetime
import os
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dist_utils import free_port


def _rank(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    t = torch.ones(4)
    dist.all_reduce(t)                       # everyone takes part in the first step
    if rank == world - 1:
        q.put((rank, "left"))                # this rank leaves between steps and never joins the next collective
        time.sleep(8)
        return
    t0 = time.time()
    try:
        dist.all_reduce(t)
        q.put((rank, "no error"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, f"raised after {time.time() - t0:.1f}s: {type(e).__name__}"))


def test_missing_rank_turns_into_an_exception_within_the_timeout():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    world = 3
    procs = [ctx.Process(target=_rank, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    msgs = dict(q.get(timeout=60) for _ in range(world))
    for p in procs:
        p.join(timeout=20)
        if p.is_alive():
            p.kill()
    assert msgs[world - 1] == "left"
    for r in range(world - 1):
        assert msgs[r].startswith("raised"), msgs
