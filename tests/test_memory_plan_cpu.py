"""The memory planner against what the package really allocates: parameters per rank and saved activations."""
import pytest
import torch

from dist_utils import run_distributed


def _tiny(**over):
    from picotron_b200.config import ModelConfig
    kw = dict(hidden_size=64, intermediate_size=160, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
              vocab_size=96, max_position_embeddings=32)
    kw.update(over)
    return ModelConfig(**kw)


def test_saved_activation_bytes_of_a_forward_pass_equal_the_plan():
    """Count every distinct tensor the autograd graph keeps after a forward pass (parameters excluded) and compare with
    the planner's activation figure for the same shape: the plan lists what the layer saves, tensor by tensor."""
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.models.llama import Llama
    from picotron_b200.utils.memory import plan_memory
    pgm.reset()
    mc = _tiny()
    B, S = 2, 32
    model = Llama(mc)
    ids = torch.randint(0, mc.vocab_size, (B, S))
    model(input_ids=ids, target_ids=ids).backward()      # the first forward packs q/k/v and gate/up into shared buffers
    param_ptrs = {p.untyped_storage().data_ptr() for p in model.parameters()}
    seen = {}

    def pack(t):
        ptr = t.untyped_storage().data_ptr()
        if ptr not in param_ptrs:
            seen[ptr] = max(seen.get(ptr, 0), t.untyped_storage().nbytes())
        return t

    with torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
        loss = model(input_ids=ids, target_ids=ids)
    measured = sum(seen.values())
    plan = plan_memory(mc, micro_batch_size=B, seq_length=S, dtype_bytes=4, fused_comm=False)
    assert plan.bytes["activations"] == pytest.approx(measured, rel=0.02), (plan.bytes["activations"], measured)
    loss.backward()


def _params_worker(rank, world, tp, pp, split):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.config import load_config, resolve_model_config
    from picotron_b200.trainer import build_trainer
    from picotron_b200.utils.memory import plan_all_stages
    cfg = load_config({
        "distributed": {"tp_size": tp, "cp_size": 1, "pp_size": pp, "dp_size": world // (tp * pp), "use_cpu": True,
                        **({"pp_layer_split": split} if split else {})},
        "model": {"name": "tiny", "preset": "tiny-llama-test", "num_hidden_layers": 5, "hidden_size": 64,
                  "intermediate_size": 160, "vocab_size": 96, "num_attention_heads": 4, "num_key_value_heads": 2,
                  "dtype": "float32"},
        "training": {"seed": 1, "learning_rate": 1e-3, "seq_length": 16, "micro_batch_size": 2,
                     "gradient_accumulation_steps": 2, "num_samples": 32},
        "dataset": {"name": "synthetic"}})
    pgm.setup_process_group_manager(tp_size=tp, cp_size=1, pp_size=pp, dp_size=world // (tp * pp))
    tr = build_trainer(cfg, init_dist=False)
    plans = plan_all_stages(resolve_model_config(cfg), cfg)
    g = pgm.get()
    return {"real": sum(p.numel() for p in tr.model.parameters()), "plan": plans[g.pp_rank].params}


@pytest.mark.parametrize("tp,pp,split", [(2, 2, None), (1, 3, None), (2, 2, [4, 1])], ids=["tp2_pp2", "pp3", "tp2_pp2_explicit"])
def test_parameters_per_rank_equal_the_plan(tp, pp, split):
    for r in run_distributed(_params_worker, tp * pp, tp, pp, split):
        assert r["real"] == r["plan"], r


def test_plan_of_the_benchmark_configurations_fits_a_b200_and_names_the_large_terms():
    from picotron_b200.config import preset_model_config
    from picotron_b200.utils.memory import B200_HBM_BYTES, plan_memory
    # headline: SmolLM-1.7B on one GPU, micro-batch 4 x 1024
    mc = preset_model_config("HuggingFaceTB/SmolLM-1.7B")
    p = plan_memory(mc, micro_batch_size=4, seq_length=1024, grad_acc_steps=32)
    assert p.params == 1_812_039_680 and p.bytes["weights"] + p.bytes["gradients"] + p.bytes["optimizer"] == 18 * p.params
    assert p.fits() and 30e9 < p.total < 60e9, p.summary()
    # Llama-2-7B on one GPU does not fit with fp32 master weights (18 bytes per parameter = 121 GB + activations) ...
    mc7 = preset_model_config("meta-llama/Llama-2-7b-hf")
    one = plan_memory(mc7, micro_batch_size=4, seq_length=4096, grad_acc_steps=32)
    assert not one.fits() and "does not fit" not in one.summary()
    # ... and fits the dp2 x tp2 x pp2 grid of the benchmark with room to spare; stage 0 keeps two micro-batches in flight
    s0 = plan_memory(mc7, tp=2, pp=2, dp=2, micro_batch_size=4, seq_length=1024, grad_acc_steps=32, stage=0)
    s1 = plan_memory(mc7, tp=2, pp=2, dp=2, micro_batch_size=4, seq_length=1024, grad_acc_steps=32, stage=1)
    assert s0.fits() and s1.fits() and s0.bytes["activations"] > 1.8 * s1.bytes["activations"] * 0.9
    assert s0.total < 0.5 * B200_HBM_BYTES
    # sequence parallelism halves the token-wise replicated activations
    sp = plan_memory(mc7, tp=2, pp=2, dp=2, micro_batch_size=4, seq_length=1024, grad_acc_steps=32, stage=0,
                     sequence_parallel=True)
    assert sp.bytes["activations"] < s0.bytes["activations"]
    # 32K tokens over cp = 8: the K/V gather and dK/dV areas appear in the workspace term
    mc1 = preset_model_config("meta-llama/Llama-3.2-1B")
    c = plan_memory(mc1, cp=8, micro_batch_size=1, seq_length=32768, grad_acc_steps=8)
    assert c.fits() and c.bytes["comm_workspaces"] > (64 << 20)


def test_train_dry_run_describes_the_stages_and_rejects_an_impossible_grid(tmp_path):
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = {"distributed": {"tp_size": 2, "cp_size": 2, "pp_size": 2, "dp_size": 1, "pp_layer_split": "balanced"},
           # the three shape overrides every config file carries (the template's defaults would shrink the model)
           "model": {"name": "meta-llama/Meta-Llama-3-8B", "num_hidden_layers": 32, "num_attention_heads": 32,
                     "num_key_value_heads": 8},
           "training": {"seq_length": 8192, "micro_batch_size": 1, "gradient_accumulation_steps": 16},
           "dataset": {"name": "synthetic"}}
    path = tmp_path / "config.json"
    path.write_text(json.dumps(cfg))
    out = subprocess.run([sys.executable, os.path.join(root, "train.py"), "--config", str(path), "--dry_run"],
                         capture_output=True, text=True, cwd=root)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "stage 0: layers 0-16 (17) + embedding" in out.stdout and "stage 1: layers 17-31 (15) + final_norm, final_proj" in out.stdout
    assert "8 ranks" in out.stdout and "131,072 tokens per optimizer step" in out.stdout and "WARNING" not in out.stdout
    cfg["distributed"]["tp_size"] = 3                                    # 8 KV heads over 3 ranks
    path.write_text(json.dumps(cfg))
    out = subprocess.run([sys.executable, os.path.join(root, "train.py"), "--config", str(path), "--dry_run"],
                         capture_output=True, text=True, cwd=root)
    assert out.returncode != 0 and "divisible" in out.stderr
