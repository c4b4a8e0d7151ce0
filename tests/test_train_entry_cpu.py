"""The user's path end to end on CPU: create_config.py -> torchrun train.py -> step log -> extract_metrics.py -> resume."""
import csv
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(nproc, config, port, log):
    env = {**os.environ, "OMP_NUM_THREADS": "1"}
    with open(log, "w") as f:
        return subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
                               "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "train.py"),
                               "--config", config], cwd=ROOT, env=env, stdout=f, stderr=subprocess.STDOUT, timeout=600)


def test_create_config_train_extract_metrics_and_resume(tmp_path):
    from dist_utils import free_port
    exp = tmp_path / "exp" / "sweep"
    out = subprocess.run([sys.executable, os.path.join(ROOT, "create_config.py"), "--out_dir", str(exp), "--exp_name",
                          "dp1_tp2_pp2_mbs2_ga2_sl32", "--tp", "2", "--pp", "2", "--model_name", "tiny-llama-test",
                          "--num_hidden_layers", "3", "--num_attention_heads", "4", "--num_key_value_heads", "2",
                          "--mbs", "2", "--seq_len", "32", "--grad_acc_steps", "2", "--use_cpu", "--dataset", "synthetic",
                          "--total_train_steps", "6", "--sequence_parallel"], capture_output=True, text=True, cwd=ROOT)
    assert out.returncode == 0, out.stderr
    run_dir = exp / "dp1_tp2_pp2_mbs2_ga2_sl32"
    cfg_path = run_dir / "config.json"
    cfg = json.load(open(cfg_path))
    cfg["checkpoint"].update(save_frequency=3, async_save=True)
    cfg["training"].update(num_samples=64, max_grad_norm=1.0, lr_schedule={"warmup_steps": 2, "decay": "cosine"},
                           eval_every=3, eval_batches=2, eval_samples=16)
    cfg["logging"]["metrics_jsonl"] = str(run_dir / "metrics.jsonl")
    json.dump(cfg, open(cfg_path, "w"))

    log = run_dir / "log_1.out"
    res = _torchrun(4, str(cfg_path), free_port(), log)
    text = open(log).read()
    assert res.returncode == 0, text[-3000:]
    steps = [ln for ln in text.splitlines() if "Step: " in ln and "Loss:" in ln]
    assert len(steps) == 6, text[-2000:]
    records = [json.loads(ln) for ln in open(run_dir / "metrics.jsonl")]
    rows = [r for r in records if "loss" in r]
    assert [r["step"] for r in rows] == [1, 2, 3, 4, 5, 6]
    assert [r["step"] for r in records if "val_loss" in r] == [3, 6] and text.count("Validation loss:") == 2
    assert rows[0]["lr"] < rows[1]["lr"] and rows[-1]["lr"] < rows[1]["lr"] and all(r["grad_norm"] > 0 for r in rows)
    assert rows[-1]["loss"] < rows[0]["loss"]
    for step in (3, 6):                                                  # background writes finished before exit
        files = os.listdir(os.path.join(cfg["checkpoint"]["save_dir"], str(step)))
        assert sum(f.endswith(".pth") for f in files) == 4 and sum(f.endswith(".done") for f in files) == 4, files

    # the authors' metrics tooling reads the log (needs more than 3 steps: it drops the first three)
    (run_dir / "status.txt").write_text("completed")
    sys.path.insert(0, ROOT)
    import extract_metrics as E
    E.main([str(tmp_path / "exp")])
    row = next(csv.DictReader(open(run_dir / "metrics.csv")))
    assert row["tp"] == "2" and row["pp"] == "2" and int(row["avg_tokens_s_gpu"]) > 0

    # resume from the newest complete step and train two more steps
    cfg["checkpoint"]["load_path"] = "latest"
    cfg["training"]["total_train_steps"] = 8
    cfg["logging"]["metrics_jsonl"] = str(run_dir / "metrics_resumed.jsonl")
    json.dump(cfg, open(cfg_path, "w"))
    log2 = run_dir / "log_2.out"
    res = _torchrun(4, str(cfg_path), free_port(), log2)
    assert res.returncode == 0, open(log2).read()[-3000:]
    resumed = [json.loads(ln) for ln in open(run_dir / "metrics_resumed.jsonl")]
    assert [r["step"] for r in resumed if "loss" in r] == [7, 8]


import pytest


@pytest.mark.parametrize("how", ["usr1_to_one_worker", "term_to_the_launcher"])
def test_a_stop_signal_on_one_rank_saves_the_current_step_on_all_ranks_and_exits_cleanly(tmp_path, how):
    """SIGUSR1 sent to a single rank, or SIGTERM sent to the launcher (what a scheduler does at a time limit; the launcher
    passes it on to its workers and gives them a grace period): the step in flight is finished and saved by all ranks."""
    import signal
    import time
    psutil = pytest.importorskip("psutil")
    from dist_utils import free_port
    save_dir = tmp_path / "ckpt"
    jsonl = tmp_path / "metrics.jsonl"
    cfg = {"distributed": {"tp_size": 2, "cp_size": 1, "pp_size": 1, "dp_size": 1, "use_cpu": True},
           "model": {"name": "tiny-llama-test", "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2},
           "training": {"seed": 1, "learning_rate": 1e-3, "seq_length": 32, "micro_batch_size": 2,
                        "gradient_accumulation_steps": 1, "total_train_steps": 100000, "num_samples": 64},
           "dataset": {"name": "synthetic"},
           "checkpoint": {"save_dir": str(save_dir), "save_frequency": 10 ** 9, "save_on_signal": True},
           "logging": {"metrics_jsonl": str(jsonl)}}
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(cfg))
    log = open(tmp_path / "log.out", "w")
    proc = subprocess.Popen([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                             "--master-addr", "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "train.py"),
                             "--config", str(cfg_path)], cwd=ROOT, env={**os.environ, "OMP_NUM_THREADS": "1"},
                            stdout=log, stderr=subprocess.STDOUT)
    try:
        deadline = time.time() + 120
        while time.time() < deadline and not (jsonl.exists() and len(jsonl.read_text().splitlines()) >= 2):
            time.sleep(0.2)
            assert proc.poll() is None, open(tmp_path / "log.out").read()[-2000:]
        workers = [p for p in psutil.Process(proc.pid).children(recursive=True)
                   if any(a.endswith("train.py") for a in p.cmdline())]
        assert len(workers) == 2, [p.cmdline() for p in psutil.Process(proc.pid).children(recursive=True)]
        if how == "usr1_to_one_worker":
            os.kill(workers[1].pid, signal.SIGUSR1)                      # only ONE rank is told
            assert proc.wait(timeout=120) == 0, open(tmp_path / "log.out").read()[-2000:]
        else:
            proc.send_signal(signal.SIGTERM)                             # the launcher reports the signal with its exit code
            proc.wait(timeout=120)
    finally:
        if proc.poll() is None:
            proc.kill()
        log.close()
    text = open(tmp_path / "log.out").read()
    assert "stop signal received" in text
    steps = os.listdir(save_dir)
    assert len(steps) == 1 and int(steps[0]) >= 2
    files = os.listdir(save_dir / steps[0])
    assert sum(f.endswith(".done") for f in files) == 2, files         # both tensor-parallel shards of that step
