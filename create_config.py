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


def _print_memory_plan(cfg) -> None:
    """Per-stage memory estimate of the run against the 180 GB of a B200 (skipped for CPU runs and unknown shapes)."""
    if cfg["distributed"].get("use_cpu"):
        return
    try:
        from picotron_b200.config import resolve_model_config
        from picotron_b200.utils.memory import check_fits, plan_all_stages
        mc = resolve_model_config(cfg)
    except Exception:  # noqa: BLE001 - the estimate is a convenience; a shape that cannot be resolved offline is not an error here
        return
    for plan in plan_all_stages(mc, cfg):
        print("Memory per GPU, " + plan.summary())
    for warning in check_fits(mc, cfg):
        print("WARNING: " + warning)


def _parse_layer_split(text: str, pp: int):
    """"reference" / "balanced" pass through; "17,15" becomes [17, 15] and must name one count per pipeline stage."""
    if text in ("reference", "balanced"):
        return text
    try:
        counts = [int(x) for x in text.split(",")]
    except ValueError:
        raise SystemExit(f"--pp_layer_split is 'reference', 'balanced' or comma-separated layer counts, not '{text}'")
    if len(counts) != pp or min(counts) < 1:
        raise SystemExit(f"--pp_layer_split names {len(counts)} stages ({counts}); pp is {pp} and every stage needs a layer")
    return counts


def create_single_config(out_dir: str, tp: int, cp: int, dp: int, pp: int, pp_engine: str, model_name: str,
                         num_hidden_layers: Optional[int], num_attention_heads: Optional[int],
                         num_key_value_heads: Optional[int], grad_acc_steps: int, mbs: int, seq_len: int,
                         subset_name: Optional[str], exp_name: str, use_wandb: bool = False, use_cpu: bool = False,
                         use_fused_adam: bool = False, hf_token: str = None, dataset: Optional[str] = None,
                         total_train_steps: Optional[int] = None, pp_layer_split: Optional[str] = None,
                         cp_layout: Optional[str] = None, comm: Optional[str] = None,
                         tie_word_embeddings: bool = False, sequence_parallel: bool = False,
                         extra_keys: Optional[list] = None) -> str:
    """Fill ``template/base_config.json`` and write ``<out_dir>/<exp_name>/config.json``; returns that path.

    ``pp_layer_split`` ("reference", "balanced" or comma-separated layer counts, one per stage), ``cp_layout``
    ("contiguous" or "zigzag"), ``comm`` ("fused" or "nccl"), ``sequence_parallel`` (each TP rank keeps 1/tp of the tokens
    between the GEMMs) and ``tie_word_embeddings`` (LM head shares the embedding matrix) are keys the reference does not have; each is written only when given, so a config made with the reference's flags alone has the reference's keys alone."""
    with open(os.path.join(HERE, "template", "base_config.json")) as f:
        cfg = json.load(f)
    run_dir = os.path.join(out_dir, exp_name)
    shape = _model_defaults(model_name)
    overrides = {"num_hidden_layers": num_hidden_layers, "num_attention_heads": num_attention_heads,
                 "num_key_value_heads": num_key_value_heads}
    updates = {
        "distributed": {"tp_size": tp, "cp_size": cp, "pp_size": pp, "dp_size": dp, "pp_engine": pp_engine,
                        "use_cpu": use_cpu, **({"backend": "gloo"} if use_cpu else {})},
        "model": {"name": model_name, "use_fused_adam": use_fused_adam,
                  **{k: (shape[k] if v is None else v) for k, v in overrides.items()}},
        "training": {"seq_length": seq_len, "micro_batch_size": mbs, "gradient_accumulation_steps": grad_acc_steps,
                     **({"total_train_steps": total_train_steps} if total_train_steps else {})},
        "dataset": {"subset_name": subset_name, **({"name": dataset} if dataset else {})},
        "checkpoint": {"save_dir": run_dir},
        "logging": {"use_wandb": use_wandb, "run_name": exp_name},
        "environment": {"HF_TOKEN": hf_token, **({"FLASH_ATTEN": "0"} if use_cpu else {})},   # no CUDA-only kernels on CPU
    }
    if pp_layer_split is not None:
        updates["distributed"]["pp_layer_split"] = _parse_layer_split(pp_layer_split, pp)
    if cp_layout is not None:
        updates["distributed"]["cp_layout"] = cp_layout
    if comm is not None:
        updates["distributed"]["comm"] = comm
    if tie_word_embeddings:
        updates["model"]["tie_word_embeddings"] = True
    if sequence_parallel:
        updates["distributed"]["sequence_parallel"] = True
    for section, values in updates.items():
        cfg[section].update(values)
    for item in extra_keys or []:                  # --set section.key=value, value read as JSON (else kept as a string)
        path, _, raw = item.partition("=")
        section, _, key = path.partition(".")
        if not key or section not in cfg:
            raise SystemExit(f"--set wants section.key=value with section in {sorted(cfg)}, got '{item}'")
        try:
            value = json.loads(raw)
        except ValueError:
            value = raw
        cfg[section][key] = value
    from picotron_b200.config import load_config
    load_config(cfg)                               # the generated file must pass the checks the trainer applies

    sequences = dp * mbs * grad_acc_steps
    print(f"Gbs_token: {sequences * seq_len:,}, Gbs: {sequences}, dp: {dp}, seq_len: {seq_len}, "
          f"grad_acc_steps: {grad_acc_steps}, mbs: {mbs}")
    _print_memory_plan(cfg)
    if os.path.isdir(run_dir):                     # a run directory of the same name is replaced, not merged
        shutil.rmtree(run_dir)
    os.makedirs(run_dir)
    path = os.path.join(run_dir, "config.json")
    with open(path, "w") as f:
        json.dump(cfg, f, indent=4)
    return path


# (flag, type or None for a switch, default, help); names and defaults follow the reference's CLI
_FLAGS = [
    ("out_dir", str, "tmp", "directory that receives <exp_name>/config.json"),
    ("exp_name", str, "dummy_exp", "name of the run directory and of the run"),
    ("tp", int, 1, "tensor-parallel size"), ("cp", int, 1, "context-parallel size"),
    ("dp", int, 1, "data-parallel size"), ("pp", int, 1, "pipeline-parallel size"),
    ("pp_engine", str, "1f1b", "pipeline schedule: 1f1b or afab"),
    ("model_name", str, "HuggingFaceTB/SmolLM-360M-Instruct", "HF model id (shape preset / tokenizer)"),
    ("num_hidden_layers", int, None, "override the model's layer count"),
    ("num_attention_heads", int, None, "override the model's query-head count"),
    ("num_key_value_heads", int, None, "override the model's KV-head count"),
    ("grad_acc_steps", int, 1, "micro-batches per optimizer step"), ("mbs", int, 1, "sequences per micro-batch"),
    ("seq_len", int, 1024, "tokens per sequence"), ("subset_name", str, None, "dataset subset"),
    ("use_wandb", None, False, "log to Weights & Biases"), ("use_cpu", None, False, "Gloo/CPU run"),
    ("use_fused_adam", None, False, "kept for schema compatibility (the optimizer here is always fused)"),
    ("hf_token", str, None, "HF access token"),
    ("dataset", str, None, "dataset name; 'synthetic' needs no network"),
    ("total_train_steps", int, None, "override training.total_train_steps"),
    # not in the reference's CLI; written to the config only when given
    ("pp_layer_split", str, None, "decoder layers per pipeline stage: reference, balanced, or counts such as 17,15"),
    ("cp_layout", str, None, "tokens per context-parallel rank: contiguous or zigzag"),
    ("comm", str, None, "collectives: fused (peer-memory kernels) or nccl"),
    ("sequence_parallel", None, False, "each TP rank keeps 1/tp of the tokens between the tensor-parallel GEMMs"),
    ("tie_word_embeddings", None, False, "the LM head shares the embedding matrix (the reference always unties)"),
]


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    for name, typ, default, text in _FLAGS:
        if typ is None:
            parser.add_argument(f"--{name}", action="store_true", help=text)
        else:
            parser.add_argument(f"--{name}", type=typ, default=default, help=text)
    parser.add_argument("--set", action="append", default=[], metavar="SECTION.KEY=VALUE", dest="extra_keys",
                        help="any other key of the config, e.g. --set training.zero1=true --set training.max_grad_norm=1.0 "
                             "--set 'training.lr_schedule={\"warmup_steps\": 100, \"decay\": \"cosine\"}' (repeatable)")
    a = parser.parse_args(argv)
    path = create_single_config(
        out_dir=a.out_dir, tp=a.tp, cp=a.cp, dp=a.dp, pp=a.pp, pp_engine=a.pp_engine, model_name=a.model_name,
        num_hidden_layers=a.num_hidden_layers, num_attention_heads=a.num_attention_heads,
        num_key_value_heads=a.num_key_value_heads, grad_acc_steps=a.grad_acc_steps, mbs=a.mbs, seq_len=a.seq_len,
        subset_name=a.subset_name, exp_name=a.exp_name, use_wandb=a.use_wandb, use_cpu=a.use_cpu,
        use_fused_adam=a.use_fused_adam, hf_token=a.hf_token, dataset=a.dataset, total_train_steps=a.total_train_steps,
        pp_layer_split=a.pp_layer_split, cp_layout=a.cp_layout, comm=a.comm,
        tie_word_embeddings=a.tie_word_embeddings, sequence_parallel=a.sequence_parallel, extra_keys=a.extra_keys)
    print(f"Configs created successfully! -> {path}")
    if a.dataset != "synthetic":
        from picotron_b200.utils import download_model
        download_model(a.model_name, a.hf_token)


if __name__ == "__main__":
    main()
