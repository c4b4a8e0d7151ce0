"""Tracing hooks (NVTX ranges, phase timers, profiler window) on a machine without a GPU."""
import json
import os

import torch

from picotron_b200.utils.tracing import PhaseTimer, ProfilerWindow, enable_nvtx, nvtx_enabled, nvtx_range


def test_nvtx_range_is_a_noop_without_cuda():
    enable_nvtx(True)
    try:
        assert nvtx_enabled() == torch.cuda.is_available()
        with nvtx_range("outer"):
            with nvtx_range("inner"):
                x = torch.ones(4).sum()
        assert float(x) == 4.0
    finally:
        enable_nvtx(False)
    assert not nvtx_enabled()


def test_phase_timer_accumulates_and_resets():
    t = PhaseTimer(torch.device("cpu"))
    for _ in range(3):
        with t.phase("a"):
            torch.randn(64, 64) @ torch.randn(64, 64)
    with t.phase("b"):
        pass
    s = t.summary()
    assert set(s) == {"a", "b"} and s["a"] > 0 and s["b"] >= 0
    assert t.summary() == {}                       # reset by the previous read
    off = PhaseTimer(torch.device("cpu"), enabled=False)
    with off.phase("x"):
        pass
    assert off.summary() == {}


def test_profiler_window_writes_one_trace(tmp_path):
    w = ProfilerWindow({"start_step": 2, "num_steps": 1, "dir": str(tmp_path)}, rank=3)
    for _ in range(4):
        torch.randn(32, 32) @ torch.randn(32, 32)
        w.step()
    w.close()
    path = os.path.join(str(tmp_path), "trace_rank3.json")
    assert os.path.exists(path)
    with open(path) as f:
        trace = json.load(f)
    assert "traceEvents" in trace and len(trace["traceEvents"]) > 0
    none = ProfilerWindow(False)
    none.step()
    none.close()


def test_trainer_reports_phase_timings_on_cpu():
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.trainer import build_trainer
    pgm.reset()
    cfg = {"distributed": {"tp_size": 1, "cp_size": 1, "pp_size": 1, "dp_size": 1, "use_cpu": True},
           "model": {"name": "tiny-test", "hidden_size": 32, "intermediate_size": 64, "vocab_size": 64,
                     "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2},
           "training": {"seed": 1, "learning_rate": 1e-3, "seq_length": 16, "micro_batch_size": 2,
                        "gradient_accumulation_steps": 2, "total_train_steps": 2},
           "dataset": {"name": "synthetic"}, "logging": {"phase_timers": True}}
    tr = build_trainer(cfg, init_dist=False)
    loss = tr.step()
    assert loss == loss                              # finite
    s = tr.timers.summary()
    assert {"micro_batches", "loss_average", "optimizer", "bucket_reset"} <= set(s)
    assert s["micro_batches"] > 0
