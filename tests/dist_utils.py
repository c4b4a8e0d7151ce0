"""Spawn helpers for multi-process CPU (Gloo) tests."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _to_numpy(x):
    """Tensors cross the process boundary by value (shared-memory handles die with the child)."""
    if torch.is_tensor(x):
        x = x.detach().cpu()
        return ("__tensor__", (x.float() if x.dtype in (torch.bfloat16, torch.float16) else x).numpy())
    if isinstance(x, dict):
        return {k: _to_numpy(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_to_numpy(v) for v in x)
    return x


def _to_torch(x):
    if isinstance(x, tuple) and len(x) == 2 and isinstance(x[0], str) and x[0] == "__tensor__":
        return torch.from_numpy(x[1])
    if isinstance(x, dict):
        return {k: _to_torch(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_to_torch(v) for v in x)
    return x


def _entry(rank, world_size, port, fn_ref, pickled_args, queue, backend, env):
    # CPU ranks are forked from a server process that has imported torch once (not the package under test): its
    # environment is the one of the moment it started, so the parent's current environment is applied here, BEFORE the
    # package and the test module are imported (they read environment switches at import time).
    os.environ.clear()
    os.environ.update(env)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world_size),
                      LOCAL_RANK=str(rank), OMP_NUM_THREADS="1")
    torch.set_num_threads(1)
    try:
        import importlib
        import pickle
        module, qualname = fn_ref
        fn = importlib.import_module(module)
        for part in qualname.split("."):
            fn = getattr(fn, part)
        args = pickle.loads(pickled_args)
        if backend == "nccl":
            torch.cuda.set_device(rank)
        import datetime
        dist.init_process_group(backend=backend, rank=rank, world_size=world_size, init_method="env://",
                                timeout=datetime.timedelta(seconds=120))
        out = fn(rank, world_size, *args)
        queue.put((rank, "ok", _to_numpy(out)))
    except Exception:  # noqa: BLE001
        queue.put((rank, "error", traceback.format_exc()))
    finally:
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:  # noqa: BLE001
                pass


def run_distributed(fn, world_size, *args, backend="gloo", timeout=120, start_method=None):
    """Run ``fn(rank, world_size, *args)`` on ``world_size`` processes; return the per-rank results."""
    import pickle
    if (start_method or ("forkserver" if backend == "gloo" else "spawn")) == "forkserver":
        ctx = mp.get_context("forkserver")               # a child costs a fork, not a fresh interpreter + `import torch`
        ctx.set_forkserver_preload(["torch", "torch._dynamo"])  # the optimizer base class pulls dynamo in (3-4 s) on first use
    else:
        ctx = mp.get_context("spawn")                    # CUDA ranks start from a clean interpreter
    queue = ctx.Queue()
    port = free_port()
    fn_ref = (fn.__module__, fn.__qualname__)
    payload, env = pickle.dumps(args), dict(os.environ)
    procs = [ctx.Process(target=_entry, args=(r, world_size, port, fn_ref, payload, queue, backend, env))
             for r in range(world_size)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world_size):
            rank, status, payload = queue.get(timeout=timeout)
            if status != "ok":
                raise AssertionError(f"rank {rank} failed:\n{payload}")
            results[rank] = _to_torch(payload)
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    return [results[r] for r in range(world_size)]
