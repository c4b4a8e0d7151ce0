"""Config generator, Slurm submitter, metrics extractor, utils, topology, data loader, checkpoint, watchdog."""
import json
import os
import subprocess
import sys
import time

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_create_config_cli(tmp_path):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "create_config.py"), "--out_dir", str(tmp_path), "--exp_name",
                          "dp2_tp2_pp2_mbs4_ga2_sl128", "--dp", "2", "--tp", "2", "--pp", "2", "--pp_engine", "afab",
                          "--model_name", "HuggingFaceTB/SmolLM-1.7B", "--num_hidden_layers", "5", "--mbs", "4",
                          "--seq_len", "128", "--grad_acc_steps", "2", "--use_cpu", "--dataset", "synthetic"],
                         capture_output=True, text=True, cwd=ROOT)
    assert out.returncode == 0, out.stderr
    cfg = json.load(open(tmp_path / "dp2_tp2_pp2_mbs4_ga2_sl128" / "config.json"))
    assert cfg["distributed"] == {**cfg["distributed"], "tp_size": 2, "dp_size": 2, "pp_size": 2, "cp_size": 1,
                                  "pp_engine": "afab", "use_cpu": True, "backend": "gloo"}
    assert cfg["model"]["num_hidden_layers"] == 5 and cfg["model"]["num_attention_heads"] == 32
    assert cfg["environment"]["FLASH_ATTEN"] == "0"
    assert cfg["training"]["micro_batch_size"] == 4 and cfg["training"]["gradient_accumulation_steps"] == 2
    for section in ("distributed", "model", "training", "dataset", "checkpoint", "logging", "environment"):
        assert section in cfg
    for key in ("pp_layer_split", "cp_layout", "sequence_parallel"):            # keys of this framework only appear when asked for
        assert key not in cfg["distributed"]
    assert "tie_word_embeddings" not in cfg["model"]


def test_create_config_optional_keys(tmp_path):
    sys.path.insert(0, ROOT)
    import create_config as C
    from picotron_b200.config import load_config, validate_config
    common = dict(out_dir=str(tmp_path), tp=1, dp=1, pp_engine="1f1b", model_name="HuggingFaceTB/SmolLM-1.7B",
                  num_hidden_layers=8, num_attention_heads=None, num_key_value_heads=None, grad_acc_steps=2, mbs=1,
                  seq_len=256, subset_name=None, use_cpu=True, dataset="synthetic")
    path = C.create_single_config(cp=2, pp=2, exp_name="a", pp_layer_split="5,3", cp_layout="zigzag", comm="nccl",
                                  tie_word_embeddings=True, sequence_parallel=True, **common)
    cfg = load_config(path)
    assert cfg["distributed"]["pp_layer_split"] == [5, 3] and cfg["distributed"]["cp_layout"] == "zigzag"
    assert cfg["distributed"]["comm"] == "nccl" and cfg["model"]["tie_word_embeddings"] is True
    assert cfg["distributed"]["sequence_parallel"] is True
    validate_config(cfg)
    path = C.create_single_config(cp=1, pp=2, exp_name="b", pp_layer_split="balanced", **common)
    assert json.load(open(path))["distributed"]["pp_layer_split"] == "balanced"
    with pytest.raises(SystemExit):
        C.create_single_config(cp=1, pp=2, exp_name="c", pp_layer_split="5,2,1", **common)
    with pytest.raises(SystemExit):
        C.create_single_config(cp=1, pp=2, exp_name="d", pp_layer_split="even", **common)


def test_submit_slurm_dry_run_and_status_machine(tmp_path):
    sys.path.insert(0, ROOT)
    import submit_slurm_jobs as S
    for name, dp in (("a_dp8", 8), ("b_dp16", 16)):
        d = tmp_path / "sweep" / name
        d.mkdir(parents=True)
        json.dump({"distributed": {"tp_size": 1, "cp_size": 1, "pp_size": 1, "dp_size": dp}}, open(d / "config.json", "w"))
    sched = S.submit_jobs(str(tmp_path / "sweep"), "high", None, 0, dry_run=True)
    assert [j.status for j in sched.job_lists] == [S.Status.PENDING, S.Status.PENDING]
    script = open(tmp_path / "sweep" / "b_dp16" / "job.slurm").read()
    assert "#SBATCH --nodes=2" in script and "--nproc_per_node=8" in script and "train.py --config" in script
    sched.job_lists[0].set_status(S.Status.FAIL)
    sched.job_lists[1].set_status(S.Status.COMPLETED)
    again = S.submit_jobs(str(tmp_path / "sweep"), "high", None, 1, only="fail", dry_run=True)
    assert [j.name for j in again.job_lists] == ["a_dp8"]
    assert S.Scheduler(str(tmp_path / "sweep"), "high").check_status()["completed"] == 1
    (tmp_path / "sweep" / "a_dp8" / "status.txt").write_text("bogus")
    with pytest.raises(ValueError):
        S.Scheduler(str(tmp_path / "sweep"), "high")


def test_extract_metrics_roundtrip_with_step_line(tmp_path):
    sys.path.insert(0, ROOT)
    import extract_metrics as E
    from picotron_b200.utils import format_step_line
    run = tmp_path / "exp" / "sweep1" / "dp8_tp1_pp1_cp2_mbs4_ga32_sl1024"
    run.mkdir(parents=True)
    lines = []
    for step in range(1, 9):
        tps_gpu = 1000.0 if step <= 3 else 43100.0
        lines.append("[default0]:" + format_step_line(0, step, 3.2, 1048576, tps_gpu * 8, tps_gpu, step * 1048576, None,
                                                      10.0 if step <= 3 else 49.8, 12.3))
    (run / "log_1.out").write_text("\n".join(lines) + "\n")
    (run / "status.txt").write_text("completed")
    E.main([str(tmp_path / "exp")])
    import csv
    row = next(csv.DictReader(open(run / "metrics.csv")))
    assert row["avg_tokens_s_gpu"] == "43100" and row["avg_mfu"] == "50" and row["cp"] == "2" and row["dp"] == "8"
    g = next(csv.DictReader(open(tmp_path / "exp" / "sweep1" / "global_metrics.csv")))
    assert g["status"] == "completed" and g["avg_tokens_s_gpu"] == "43100"


def test_utils_numbers_and_mfu():
    from picotron_b200.config import preset_model_config
    from picotron_b200.utils import flops_per_token, from_readable_format, get_mfu, to_readable_format
    assert to_readable_format(1_048_576) == "1.05M" and to_readable_format(43100) == "43.10K" and to_readable_format(12) == "12.00"
    assert from_readable_format("43.1K") == 43100.0
    mc = preset_model_config("HuggingFaceTB/SmolLM-1.7B")
    mc.max_position_embeddings = 1024
    assert mc.num_params() == 1_812_039_680
    assert abs(flops_per_token(mc.num_params(), mc) / 1e9 - 11.48) < 0.01
    assert abs(get_mfu(43.1e3, mc.num_params(), mc, theoretical_flops=989.5e12) - 50.0) < 0.1


def test_grid_topology_layout_matches_reference_order():
    from picotron_b200.process_group_manager import GridTopology
    t = GridTopology(tp_size=2, cp_size=1, pp_size=2, dp_size=2)
    # dp2 x tp2 x pp2: ranks (0,1) = stage 0 / dp 0, (2,3) = stage 1 / dp 0, (4,5) = stage 0 / dp 1
    assert t.coords(0) == (0, 0, 0, 0) and t.coords(1) == (0, 0, 0, 1) and t.coords(2) == (0, 1, 0, 0)
    assert t.coords(5) == (1, 0, 0, 1) and t.rank(1, 1, 0, 1) == 7
    assert t.tp_groups() == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert t.pp_groups() == [[0, 2], [1, 3], [4, 6], [5, 7]]
    assert t.dp_groups() == [[0, 4], [1, 5], [2, 6], [3, 7]]
    t2 = GridTopology(tp_size=1, cp_size=2, pp_size=1, dp_size=2)
    assert t2.cp_dp_groups() == [[0, 1, 2, 3]] and t2.cp_groups() == [[0, 1], [2, 3]]
    for topo in (t, t2):
        for r in range(topo.world_size):
            assert topo.rank(*topo.coords(r)) == r


def test_synthetic_loader_shapes_dp_sharding_and_wraparound():
    from picotron_b200.data import MicroBatchDataLoader, group_into_windows
    import numpy as np
    dl = MicroBatchDataLoader(micro_batch_size=2, seq_length=8, dataset_name="synthetic", tokenizer_name=None,
                              num_workers=0, num_proc=1, grad_acc_steps=3, device="cpu", num_samples=10, vocab_size=50)
    assert dl.global_batch_size == 6 and dl.seq_length_per_gpu == 8 and dl.num_global_micro_batches == 3
    b = next(dl)
    assert b["input_ids"].shape == (2, 8) and b["hidden_states"] is None
    assert torch.equal(b["input_ids"][:, 1:], b["target_ids"][:, :-1])
    assert torch.equal(b["position_ids"][0], torch.arange(8))
    first = b["input_ids"].clone()
    for _ in range(4):
        next(dl)
    assert dl.epoch == 0
    again = next(dl)                      # 5 batches per epoch -> wraps
    assert dl.epoch == 1 and torch.equal(again["input_ids"], first)
    w = group_into_windows(np.arange(20), 4)
    assert len(w) == 4 and list(w[1]) == [4, 5, 6, 7, 8]


def test_checkpoint_layout_resume_and_atomicity(tmp_path):
    from picotron_b200.checkpoint import CheckpointManager, find_latest_checkpoint
    from picotron_b200.config import ModelConfig
    from picotron_b200.models.llama import Llama
    from picotron_b200.optim import FusedAdamW
    from picotron_b200.parallel.data_parallel import DataParallelBucket
    cfg = ModelConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2,
                      num_key_value_heads=1, vocab_size=40, max_position_embeddings=8)
    torch.manual_seed(0)
    m = DataParallelBucket(Llama(cfg).to(torch.bfloat16))
    opt = FusedAdamW(m.parameters(), lr=1e-2)
    ids = torch.randint(0, 40, (2, 8))
    m(ids, target_ids=ids).backward()
    opt.step()
    cm = CheckpointManager()
    cm.save_checkpoint(m, opt, 7, 1234, str(tmp_path / "7"))
    f = tmp_path / "7" / "weights_tp_rank_world_size=0_1_pp_rank_world_size=0_1.pth"
    assert f.exists() and not (tmp_path / "7" / (f.name + ".tmp")).exists()
    ck = torch.load(f, weights_only=False)
    assert set(ck) >= {"model", "optimizer", "trained_steps", "trained_tokens"}
    assert "decoder_layers.0.attention.q_proj.weight" in ck["model"]
    torch.manual_seed(1)
    m2 = DataParallelBucket(Llama(cfg).to(torch.bfloat16))
    opt2 = FusedAdamW(m2.parameters(), lr=1e-2)
    (tmp_path / "9").mkdir()              # an empty (crashed) later directory is skipped
    assert find_latest_checkpoint(str(tmp_path)) == str(tmp_path / "7")
    steps, tokens = cm.load_checkpoint(m2, opt2, str(tmp_path / "7"))
    assert (steps, tokens) == (7, 1234)
    for a, b in zip(m.parameters(), m2.parameters()):
        assert torch.equal(a, b)
    st = opt2.state[next(iter(m2.parameters()))]
    assert st["exp_avg"].dtype == torch.float32 and st["master"].dtype == torch.float32
    with pytest.raises(FileNotFoundError):
        cm.load_checkpoint(m2, opt2, str(tmp_path / "9"))


def test_meta_device_init_and_materialise():
    from picotron_b200.checkpoint import init_model_with_dematerialized_weights, init_model_with_materialized_weights
    from picotron_b200.config import ModelConfig
    from picotron_b200.models.llama import Llama
    from picotron_b200.utils import assert_no_meta_tensors, get_num_params
    cfg = ModelConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2,
                      num_key_value_heads=1, vocab_size=40, max_position_embeddings=8)
    with init_model_with_dematerialized_weights():
        m = Llama(cfg)
    assert all(p.device.type == "meta" for p in m.parameters())
    with pytest.raises(AssertionError):
        assert_no_meta_tensors(m)
    m = init_model_with_materialized_weights(m, cfg)
    assert_no_meta_tensors(m)
    assert get_num_params(m) == cfg.num_params()
    assert float(m.decoder_layers[0].input_layernorm.weight.sum()) == 32.0


def test_step_watchdog_flags_a_stalled_step():
    from picotron_b200.utils.watchdog import StepWatchdog
    hits = []
    wd = StepWatchdog(timeout_s=0.2, on_timeout=hits.append)
    with wd.step(3):
        time.sleep(0.05)
    assert not wd.fired
    with wd.step(4):
        time.sleep(0.6)
    assert wd.fired and wd.fired_step == 4 and hits == [4]
    wd.close()


def test_bench_json_line_has_every_contract_key():
    """The one-line JSON of bench.py: keys and units the benchmark contract names (built here from fake timings)."""
    import argparse
    import importlib.util
    import json
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    args = argparse.Namespace(gpus=2, steps=3, warmup=3, impl="ours", layers=None, grad_acc=bench.GRAD_ACC)
    clocks = {"sm_mhz": 1600.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"]}
    out = bench.result_line(args, 2, 4.5, 4.6, clocks, 1234, "ours", {"gemm": "tcgen05"}, 1_812_039_680, 24)
    line = json.loads(json.dumps(out))
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches"):
        assert key in line, key
    tokens = bench.MBS * bench.SEQ * bench.GRAD_ACC * 2 * 3
    assert line["value"] == pytest.approx(tokens / 4.5) and line["n_gpus"] == 2 and line["scaling"] == "weak"
    assert line["e2e"]["value"] == pytest.approx(tokens / 4.6)
    assert line["e2e"]["h2d_bytes_per_step"] == 2 * bench.MBS * bench.SEQ * 8 * bench.GRAD_ACC * 2
    assert line["config"]["parallelism"] == "dp2" and line["config"]["seq_len"] == 1024
    assert "invalid" not in line
    short = bench.result_line(argparse.Namespace(**{**vars(args), "grad_acc": 2}), 1, 1.0, 1.0, clocks, 1, "ours", {}, 1, 2)
    assert "invalid" in short                                   # reduced configs are marked, never reported as the metric


def test_bench_prints_exactly_one_line_whatever_happens_to_the_secondary_measurement(capsys, monkeypatch):
    """`bench.py --gpus 8` appends the Llama-2-7B dp2.tp2.pp2 result; a failure there must not cost the headline line."""
    import argparse
    import importlib.util
    import json
    import sys
    import types
    spec = importlib.util.spec_from_file_location("bench_under_test2", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    args = argparse.Namespace(gpus=8, steps=2, warmup=3, impl="ours", layers=None, grad_acc=bench.GRAD_ACC, no_secondary=False)
    # fewer than 8 ranks: the line is printed as it is
    bench.with_secondary({"value": 1.0}, 0, 2, args, "ours")
    assert json.loads(capsys.readouterr().out.strip()) == {"value": 1.0}
    # 8 ranks, the second measurement raises: one line, with the error recorded
    fake = types.ModuleType("bench_configs")
    fake.measure_ours = lambda *a, **k: (_ for _ in ()).throw(RuntimeError("no peer access"))
    fake.measure_reference = fake.measure_ours
    monkeypatch.setitem(sys.modules, "bench_configs", fake)
    bench.with_secondary({"value": 2.0}, 0, 8, args, "ours")
    lines = [l for l in capsys.readouterr().out.strip().splitlines() if l]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["value"] == 2.0 and d["secondary"]["config"] == "llama7b_3d" and "no peer access" in d["secondary"]["error"]
    # 8 ranks, it succeeds: attached as `secondary`; other ranks print nothing
    fake.measure_ours = lambda name, steps, warmup: {"config": name, "tokens_per_second_per_gpu": 20000.0}
    bench.with_secondary({"value": 3.0}, 0, 8, args, "ours")
    assert json.loads(capsys.readouterr().out.strip())["secondary"]["tokens_per_second_per_gpu"] == 20000.0
    bench.with_secondary({}, 3, 8, args, "ours")
    assert capsys.readouterr().out.strip() == ""


def test_loader_position_carries_over_to_another_data_parallel_size():
    """4 batches of 2 on dp = 1 consumed 8 samples; a loader that is one of dp = 2 ranks with batches of 2 continues at global
    sample 8 (its cursor 2), not at its own cursor 4 (global sample 16)."""
    from types import SimpleNamespace
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.data import MicroBatchDataLoader

    def loader(dp_rank, dp):
        pgm.process_group_manager = SimpleNamespace(dp_world_size=dp, dp_rank=dp_rank, cp_world_size=1, cp_rank=0,
                                                    global_rank=dp_rank)
        try:
            return MicroBatchDataLoader(micro_batch_size=2, seq_length=8, dataset_name="synthetic", tokenizer_name=None,
                                        num_workers=0, num_proc=1, grad_acc_steps=1, device="cpu", num_samples=64, vocab_size=50)
        finally:
            pgm.reset()

    one = loader(0, 1)
    seen = [next(one)["input_ids"] for _ in range(4)]
    state = one.state_dict()
    assert state["samples_seen"] == 8
    following = torch.cat([next(one)["input_ids"] for _ in range(2)])            # global samples 8..11 in order
    two = [loader(r, 2) for r in range(2)]
    for ld in two:
        ld.load_state_dict(state)
        assert ld._cursor == 2
    b0, b1 = next(two[0])["input_ids"], next(two[1])["input_ids"]               # rank r holds samples r, r + 2, ...
    merged = torch.stack([b0[0], b1[0], b0[1], b1[1]])
    assert torch.equal(merged, following)
    same = loader(0, 1)
    same.load_state_dict(state)
    assert same._cursor == 4                                                     # unchanged layout: the cursor as saved


def test_create_config_set_writes_any_key_and_refuses_values_the_trainer_would_refuse(tmp_path):
    base = [sys.executable, os.path.join(ROOT, "create_config.py"), "--out_dir", str(tmp_path), "--model_name", "tiny-llama-test",
            "--num_hidden_layers", "2", "--num_attention_heads", "4", "--num_key_value_heads", "2", "--use_cpu",
            "--dataset", "synthetic", "--seq_len", "32"]
    out = subprocess.run(base + ["--exp_name", "ok", "--set", "training.zero1=true", "--set", "training.max_grad_norm=1.0",
                                 "--set", 'training.lr_schedule={"warmup_steps": 10, "decay": "cosine"}',
                                 "--set", "checkpoint.async_save=true", "--set", "logging.run_name=my run"],
                         capture_output=True, text=True, cwd=ROOT)
    assert out.returncode == 0, out.stderr
    cfg = json.load(open(tmp_path / "ok" / "config.json"))
    assert cfg["training"]["zero1"] is True and cfg["training"]["max_grad_norm"] == 1.0
    assert cfg["training"]["lr_schedule"] == {"warmup_steps": 10, "decay": "cosine"}
    assert cfg["checkpoint"]["async_save"] is True and cfg["logging"]["run_name"] == "my run"
    bad = subprocess.run(base + ["--exp_name", "bad", "--set", 'training.lr_schedule={"decay": "exponential"}'],
                         capture_output=True, text=True, cwd=ROOT)
    assert bad.returncode != 0 and not (tmp_path / "bad" / "config.json").exists()
    worse = subprocess.run(base + ["--exp_name", "worse", "--set", "nosuchsection.key=1"], capture_output=True, text=True, cwd=ROOT)
    assert worse.returncode != 0 and "section.key=value" in worse.stderr
