"""Generate an experiment directory with its ``config.json``.

    python create_config.py --out_dir tmp --exp_name llama-1B --dp 8 --model_name HuggingFaceTB/SmolLM-1.7B \
        --num_hidden_layers 15 --grad_acc_steps 32 --mbs 4 --seq_len 1024

Same flags and output location (``<out_dir>/<exp_name>/config.json``, an existing run directory is replaced) as the
reference's ``create_config.py:14-136``. The model shape defaults come from the offline presets of
``picotron_b200.config`` (the reference asks the HF hub); ``--dataset synthetic`` selects uniform-random tokens so
the resulting config runs with no network. Downloading safetensors is skipped when ``HF_HUB_OFFLINE=1``.
"""
import argparse
import json
import os
import shutil
from copy import deepcopy
from typing import Optional

from picotron_b200.config import MODEL_PRESETS

HERE = os.path.dirname(os.path.abspath(__file__))


def _model_defaults(model_name: str) -> dict:
    if model_name in MODEL_PRESETS:
        return MODEL_PRESETS[model_name]
    try:
        from transformers import AutoConfig
        hf = AutoConfig.from_pretrained(model_name, local_files_only=os.environ.get("HF_HUB_OFFLINE") == "1")
        return dict(num_hidden_layers=hf.num_hidden_layers, num_attention_heads=hf.num_attention_heads,
                    num_key_value_heads=hf.num_key_value_heads)
    except Exception as e:  # noqa: BLE001
        raise SystemExit(f"model '{model_name}' is not a preset ({sorted(MODEL_PRESETS)}) and its HF config is not "
                         f"available: {e}")


def create_single_config(out_dir: str, tp: int, cp: int, dp: int, pp: int, pp_engine: str, model_name: str,
                         num_hidden_layers: Optional[int], num_attention_heads: Optional[int],
                         num_key_value_heads: Optional[int], grad_acc_steps: int, mbs: int, seq_len: int,
                         subset_name: Optional[str], exp_name: str, use_wandb: bool = False, use_cpu: bool = False,
                         use_fused_adam: bool = False, hf_token: str = None, dataset: Optional[str] = None,
                         total_train_steps: Optional[int] = None) -> str:
    run_path = os.path.join(out_dir, exp_name)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(HERE, "template", "base_config.json"), "r") as f:
        cfg = deepcopy(json.load(f))

    defaults = _model_defaults(model_name)
    cfg["environment"]["HF_TOKEN"] = hf_token
    cfg["training"]["seq_length"] = seq_len
    cfg["checkpoint"]["save_dir"] = run_path
    cfg["dataset"]["subset_name"] = subset_name
    if dataset:
        cfg["dataset"]["name"] = dataset
    if total_train_steps:
        cfg["training"]["total_train_steps"] = total_train_steps
    cfg["model"]["name"] = model_name
    cfg["model"]["num_hidden_layers"] = defaults["num_hidden_layers"] if num_hidden_layers is None else num_hidden_layers
    cfg["model"]["num_attention_heads"] = defaults["num_attention_heads"] if num_attention_heads is None else num_attention_heads
    cfg["model"]["num_key_value_heads"] = defaults["num_key_value_heads"] if num_key_value_heads is None else num_key_value_heads
    cfg["model"]["use_fused_adam"] = use_fused_adam
    d = cfg["distributed"]
    d["tp_size"], d["cp_size"], d["dp_size"], d["pp_size"], d["pp_engine"], d["use_cpu"] = tp, cp, dp, pp, pp_engine, use_cpu
    if use_cpu:
        cfg["environment"]["FLASH_ATTEN"] = "0"
        d["backend"] = "gloo"
    cfg["logging"]["use_wandb"] = use_wandb
    cfg["logging"]["run_name"] = exp_name
    gbs = dp * mbs * grad_acc_steps
    print(f"Gbs_token: {gbs * seq_len:,}, Gbs: {gbs}, dp: {dp}, seq_len: {seq_len}, grad_acc_steps: {grad_acc_steps}, mbs: {mbs}")
    cfg["training"]["gradient_accumulation_steps"] = grad_acc_steps
    cfg["training"]["micro_batch_size"] = mbs

    if os.path.exists(run_path):
        shutil.rmtree(run_path)
    os.makedirs(run_path)
    path = os.path.join(run_path, "config.json")
    with open(path, "w") as f:
        json.dump(cfg, f, indent=4)
    return path


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--out_dir", type=str, help="Output directory to store the configs", default="tmp")
    p.add_argument("--tp", type=int, help="number of tensor parallelism", default=1)
    p.add_argument("--cp", type=int, help="number of context parallelism", default=1)
    p.add_argument("--dp", type=int, help="number of data parallelism", default=1)
    p.add_argument("--pp", type=int, help="number of pipeline parallelism", default=1)
    p.add_argument("--pp_engine", type=str, help="pipeline parallel engine", default="1f1b")
    p.add_argument("--model_name", type=str, help="Model name to create configs for", default="HuggingFaceTB/SmolLM-360M-Instruct")
    p.add_argument("--num_hidden_layers", type=int, help="Number of hidden layers", default=None)
    p.add_argument("--num_attention_heads", type=int, help="Number of attention heads", default=None)
    p.add_argument("--num_key_value_heads", type=int, help="Number of key value heads", default=None)
    p.add_argument("--grad_acc_steps", type=int, help="grad accumulation", default=1)
    p.add_argument("--mbs", type=int, help="micro batch size", default=1)
    p.add_argument("--seq_len", type=int, help="Sequence length", default=1024)
    p.add_argument("--subset_name", type=str, help="Subset name", default=None)
    p.add_argument("--exp_name", type=str, help="Experiment name", default="dummy_exp")
    p.add_argument("--use_wandb", action="store_true", help="Use wandb for logging")
    p.add_argument("--use_cpu", action="store_true", help="Use CPU for training")
    p.add_argument("--use_fused_adam", action="store_true", help="Use fused adam")
    p.add_argument("--hf_token", type=str, help="HF token")
    p.add_argument("--dataset", type=str, default=None, help="dataset name; 'synthetic' needs no network")
    p.add_argument("--total_train_steps", type=int, default=None)
    a = p.parse_args(argv)
    path = create_single_config(a.out_dir, a.tp, a.cp, a.dp, a.pp, a.pp_engine, a.model_name, a.num_hidden_layers,
                                a.num_attention_heads, a.num_key_value_heads, a.grad_acc_steps, a.mbs, a.seq_len,
                                a.subset_name, a.exp_name, a.use_wandb, a.use_cpu, a.use_fused_adam, a.hf_token,
                                a.dataset, a.total_train_steps)
    print(f"Configs created successfully! -> {path}")
    if a.dataset != "synthetic":
        from picotron_b200.utils import download_model
        download_model(a.model_name, a.hf_token)


if __name__ == "__main__":
    main()
