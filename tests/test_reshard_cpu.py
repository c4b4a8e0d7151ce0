"""A step saved on one tensor-/pipeline-parallel grid, re-cut for another, continues on the same loss trajectory."""
import os
import sys

import pytest

from dist_utils import run_distributed

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cfg(tp, pp, save_dir, load_path="", split=None, tie=False):
    return {"distributed": {"tp_size": tp, "cp_size": 1, "pp_size": pp, "dp_size": 1, "use_cpu": True,
                            **({"pp_layer_split": split} if split else {})},
            "model": {"name": "tiny", "hidden_size": 32, "intermediate_size": 64, "vocab_size": 64, "num_hidden_layers": 3,
                      "num_attention_heads": 4, "num_key_value_heads": 2, "dtype": "float32", "tie_word_embeddings": tie},
            "training": {"seed": 5, "learning_rate": 1e-2, "seq_length": 16, "micro_batch_size": 2,
                         "gradient_accumulation_steps": 2, "total_train_steps": 10, "num_samples": 64},
            "dataset": {"name": "synthetic"},
            "checkpoint": {"save_dir": save_dir, "save_frequency": 1000, "load_path": load_path}}


def _run_worker(rank, world, cfg, steps, save_after):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.trainer import build_trainer
    d = cfg["distributed"]
    pgm.setup_process_group_manager(tp_size=d["tp_size"], cp_size=1, pp_size=d["pp_size"], dp_size=1)
    tr = build_trainer(cfg, init_dist=False)
    losses = []
    for i in range(steps):
        losses.append(tr.step())
        if save_after and tr.step_idx == save_after:
            tr.save(os.path.join(cfg["checkpoint"]["save_dir"], str(tr.step_idx)))
    return {"losses": losses, "last": pgm.get().pp_is_last_stage, "start": tr.step_idx - steps}


def _losses(results):
    return [r for r in results if r["last"]][0]["losses"]


@pytest.mark.parametrize("tie", [False, True], ids=["untied", "tied"])
def test_resharded_checkpoint_continues_the_run_on_other_grids(tmp_path, tie):
    from picotron_b200.config import load_config, resolve_model_config
    from picotron_b200.reshard import grid_of, reshard_checkpoint
    a_dir = str(tmp_path / "a")
    # grid A: tp2 x pp2 with an uneven explicit layer split; 4 steps, the state after step 2 is saved
    cfg_a = _cfg(2, 2, a_dir, split=[2, 1], tie=tie)
    full = _losses(run_distributed(_run_worker, 4, cfg_a, 4, 2))
    assert grid_of(os.path.join(a_dir, "2")) == (2, 2)
    mc = resolve_model_config(load_config(cfg_a))
    # A -> B: one rank
    b_dir = str(tmp_path / "b")
    paths = reshard_checkpoint(os.path.join(a_dir, "2"), os.path.join(b_dir, "2"), mc, tp=1, pp=1, src_layer_split=[2, 1],
                               tie=tie)
    assert len(paths) == 1 and os.path.exists(paths[0] + ".done")
    res_b = run_distributed(_run_worker, 1, _cfg(1, 1, b_dir, load_path="latest", tie=tie), 3, 4)
    assert res_b[0]["start"] == 2
    assert _losses(res_b)[:2] == pytest.approx(full[2:], rel=2e-4)          # steps 3 and 4 as the original grid ran them
    # B (state after step 4) -> C: three pipeline stages; its next step is B's step 5
    c_dir = str(tmp_path / "c")
    reshard_checkpoint(os.path.join(b_dir, "4"), os.path.join(c_dir, "4"), mc, tp=1, pp=3, tie=tie)
    res_c = run_distributed(_run_worker, 3, _cfg(1, 3, c_dir, load_path=os.path.join(c_dir, "4"), tie=tie), 1, 0)
    assert _losses(res_c) == pytest.approx(_losses(res_b)[2:], rel=2e-4)
    # B -> D: cut along the tensor-parallel dimensions again (weights, moments), same next step
    d_dir = str(tmp_path / "d")
    reshard_checkpoint(os.path.join(b_dir, "4"), os.path.join(d_dir, "4"), mc, tp=2, pp=1, tie=tie)
    res_d = run_distributed(_run_worker, 2, _cfg(2, 1, d_dir, load_path=os.path.join(d_dir, "4"), tie=tie), 1, 0)
    assert _losses(res_d) == pytest.approx(_losses(res_b)[2:], rel=2e-4)


def test_reshard_cli_and_incomplete_source(tmp_path):
    import json
    sys.path.insert(0, ROOT)
    import reshard_checkpoint as cli
    from picotron_b200.reshard import grid_of
    a_dir = str(tmp_path / "a")
    cfg = _cfg(2, 1, a_dir)
    run_distributed(_run_worker, 2, cfg, 1, 1)
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(cfg))
    cli.main(["--config", str(cfg_path), "--src", os.path.join(a_dir, "1"), "--dst", str(tmp_path / "b" / "1"),
              "--tp", "1", "--pp", "2", "--pp_layer_split", "1,2"])
    assert grid_of(str(tmp_path / "b" / "1")) == (1, 2)
    os.remove(os.path.join(a_dir, "1", "weights_tp_rank_world_size=1_2_pp_rank_world_size=0_1.pth"))
    with pytest.raises(FileNotFoundError):
        grid_of(os.path.join(a_dir, "1"))
