"""Failure detection on the host: a rank that never joins a collective makes the others raise, not hang."""
import datetime
import os
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dist_utils import free_port, run_distributed


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


def test_resume_skips_a_truncated_checkpoint_and_half_written_files(tmp_path):
    """`load_path: latest` picks the newest COMPLETE checkpoint: a truncated file and a leftover .tmp are passed over."""
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.checkpoint import CheckpointManager, checkpoint_file_is_complete, find_latest_checkpoint
    pgm.reset()
    model = torch.nn.Linear(4, 4)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    cm = CheckpointManager()
    save_dir = str(tmp_path)
    for step in (1, 2):
        cm.save_checkpoint(model, opt, step, step * 100, os.path.join(save_dir, str(step)))
    assert find_latest_checkpoint(save_dir) == os.path.join(save_dir, "2")
    newest = cm._get_checkpoint_path(os.path.join(save_dir, "2"))
    with open(newest, "r+b") as f:                         # the file system lost the tail of the newest checkpoint
        f.truncate(os.path.getsize(newest) // 2)
    assert not checkpoint_file_is_complete(newest)
    assert find_latest_checkpoint(save_dir) == os.path.join(save_dir, "1")
    os.makedirs(os.path.join(save_dir, "3"))               # a save that died before the atomic rename
    with open(cm._get_checkpoint_path(os.path.join(save_dir, "3")) + ".tmp", "wb") as f:
        f.write(b"partial")
    assert find_latest_checkpoint(save_dir) == os.path.join(save_dir, "1")
    steps, tokens = cm.load_checkpoint(model, opt, os.path.join(save_dir, "1"))
    assert (steps, tokens) == (1, 100)
    with pytest.raises(Exception):
        cm.load_checkpoint(model, opt, os.path.join(save_dir, "2"))     # loading the damaged file fails loudly


def test_watchdog_abort_ends_the_process_with_the_timeout_exit_code():
    """A stalled step with `abort=True`: exit code 124, which the job template files under `timeout`."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = "\n".join(["import time", "from picotron_b200.utils.watchdog import StepWatchdog",
                      "w = StepWatchdog(timeout_s=0.3, abort=True)", "with w.step(7):", "    time.sleep(30)"])
    t0 = time.time()
    r = subprocess.run([sys.executable, "-c", code], cwd=root, capture_output=True, text=True, timeout=60)
    assert r.returncode == 124, (r.returncode, r.stderr[-500:])
    assert time.time() - t0 < 25
    assert "step 7" in (r.stdout + r.stderr)


# ------------------------------------------------------------------------------ kernel status word aborts the step
def _status_abort_worker(rank, world, inject_rank):
    """Two data-parallel Gloo ranks; the status reader of one rank reports a timed-out kernel wait in the second step."""
    from parallel_harness import make_config, _build
    from picotron_b200.trainer import KernelWaitTimeout
    tr = _build(make_config(1, 1, 1, world, grad_acc=2, layers=2))
    tr.step()                                              # a clean step goes through
    before = {n: p.detach().clone() for n, p in tr.model.module.named_parameters()}
    if rank == inject_rank:
        tr.status_reader = lambda: (5 << 24) | (1 << 16) | 3   # kernel 5 (all-reduce), site 1, block 3
    try:
        tr.step()
        outcome = "no error"
    except KernelWaitTimeout as e:
        outcome = f"raised: {e}"
    unchanged = all(torch.equal(before[n], p.detach()) for n, p in tr.model.module.named_parameters())
    return {"outcome": outcome, "unchanged": unchanged}


def test_nonzero_kernel_status_on_one_rank_aborts_the_step_on_every_rank():
    from dist_utils import run_distributed
    for r in run_distributed(_status_abort_worker, 2, 1):
        assert r["outcome"].startswith("raised") and "kernel id 5" in r["outcome"], r
        assert r["unchanged"], "the optimizer must not run on gradients that were not reduced"


# ------------------------------------------------------------------------------ `latest` is agreed on by all ranks
def _latest_worker(rank, world, save_dir):
    """tp2: step 2 was written completely, step 3 only by tp rank 0 (the job died during the save)."""
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.checkpoint import CheckpointManager, find_latest_checkpoint
    pgm.setup_process_group_manager(tp_size=world, cp_size=1, pp_size=1, dp_size=1)
    model = torch.nn.Linear(4, 4)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    cm = CheckpointManager()
    cm.save_checkpoint(model, opt, 2, 200, os.path.join(save_dir, "2"))
    if rank == 0:
        cm.save_checkpoint(model, opt, 3, 300, os.path.join(save_dir, "3"))
    dist.barrier()
    return find_latest_checkpoint(save_dir)


def test_latest_checkpoint_is_the_newest_step_that_every_shard_holds(tmp_path):
    from dist_utils import run_distributed
    save_dir = str(tmp_path)
    res = run_distributed(_latest_worker, 2, save_dir)
    assert res == [os.path.join(save_dir, "2")] * 2, res


# --------------------------------------------------------------------------------------------- silent replica divergence
def _divergence_worker(rank, world, corrupt):
    import torch
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.trainer import ReplicaDivergence, build_trainer
    cfg = {"distributed": {"tp_size": 2, "cp_size": 1, "pp_size": 1, "dp_size": 2, "use_cpu": True},
           "model": {"name": "tiny", "hidden_size": 32, "intermediate_size": 64, "vocab_size": 64, "num_hidden_layers": 2,
                     "num_attention_heads": 4, "num_key_value_heads": 2},
           "training": {"seed": 3, "learning_rate": 1e-2, "seq_length": 16, "micro_batch_size": 2,
                        "gradient_accumulation_steps": 2, "num_samples": 64, "verify_replicas_every": 2},
           "dataset": {"name": "synthetic"}}
    pgm.setup_process_group_manager(tp_size=2, cp_size=1, pp_size=1, dp_size=2)
    tr = build_trainer(cfg, init_dist=False)
    tr.step()
    tr.step()                                                            # step 2: checked, replicas agree
    raw = tr.model.module
    if corrupt == "dp" and rank == 3:                                    # one bit of one weight on one data-parallel replica
        with torch.no_grad():
            w = raw.decoder_layers[1].mlp.down_proj.weight
            w.view(torch.int32)[0, 0] ^= 1
    if corrupt == "tp" and pgm.get().tp_rank == 1:                       # a norm weight on one side of every TP pair
        with torch.no_grad():
            raw.final_norm.weight[3] += 1e-3
    tr.step()
    try:
        tr.step()                                                        # step 4: checked again
        return "clean"
    except ReplicaDivergence as e:
        return str(e)


def test_bitwise_replica_check_names_the_diverged_parameter_on_every_rank_of_its_group():
    assert run_distributed(_divergence_worker, 4, None) == ["clean"] * 4
    dp = run_distributed(_divergence_worker, 4, "dp")
    # ranks 1 and 3 form the data-parallel pair of tp_rank 1: both see it; the other pair stops with them
    assert "down_proj" in dp[1] and "down_proj" in dp[3] and "context/data-parallel" in dp[3]
    assert "another rank" in dp[0] and "another rank" in dp[2]
    tp = run_distributed(_divergence_worker, 4, "tp")
    assert all("final_norm.weight" in r and "tensor-parallel" in r for r in tp)


# --------------------------------------------------------------------------------------------- non-finite gradients
def _nonfinite_worker(rank, world):
    import torch
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.trainer import build_trainer
    cfg = {"distributed": {"tp_size": 1, "cp_size": 1, "pp_size": 2, "dp_size": 1, "use_cpu": True},
           "model": {"name": "tiny", "hidden_size": 32, "intermediate_size": 64, "vocab_size": 64, "num_hidden_layers": 2,
                     "num_attention_heads": 4, "num_key_value_heads": 2},
           "training": {"seed": 3, "learning_rate": 1e-2, "seq_length": 16, "micro_batch_size": 2,
                        "gradient_accumulation_steps": 2, "num_samples": 64, "skip_nonfinite_steps": True},
           "dataset": {"name": "synthetic"}}
    pgm.setup_process_group_manager(tp_size=1, cp_size=1, pp_size=2, dp_size=1)
    tr = build_trainer(cfg, init_dist=False)
    tr.step()
    before = [p.detach().clone() for p in tr.model.parameters()]
    if rank == 0:                                # a NaN appears in one gradient of the FIRST stage only
        w = next(tr.model.parameters())
        w.main_grad.view(-1)[0] = float("nan")   # survives the accumulation of the step's micro-batches
    tr.step()
    unchanged = all(torch.equal(p, b) for p, b in zip(tr.model.parameters(), before))
    out = {"unchanged": unchanged, "skipped": tr.skipped_steps, "step_idx": tr.step_idx}
    tr.step()                                    # buckets were cleared: the next step updates again
    out["moved"] = not all(torch.equal(p, b) for p, b in zip(tr.model.parameters(), before))
    out["step_idx_after"] = tr.step_idx
    return out


def test_a_nan_gradient_on_one_stage_makes_every_rank_skip_that_update():
    for r in run_distributed(_nonfinite_worker, 2):
        assert r["unchanged"] and r["skipped"] == 1 and r["step_idx"] == 1, r
        assert r["moved"] and r["step_idx_after"] == 2, r
