"""Typed view of the JSON experiment file and offline model presets.

The JSON schema is the one written by ``create_config.py`` and read by ``train.py`` in the reference
(``template/base_config.json:1-52``, ``train.py:57-235``): sections ``distributed``, ``model``,
``training``, ``dataset``, ``checkpoint``, ``logging``, ``environment``. Keys the reference writes but
never reads (``distributed.backend``, ``model.dtype``, ``model.use_flash_attention``,
``logging.project_name``) are accepted and kept.

Additions (all optional, with defaults that reproduce the reference's behaviour):

* ``model.preset`` / explicit shape fields (``hidden_size``, ``intermediate_size``, ``vocab_size``,
  ``rope_theta``, ``rms_norm_eps``) so that a run needs no network: the reference asks the HF hub for
  ``AutoConfig`` (``train.py:154``), this package first looks the model name up in :data:`MODEL_PRESETS`.
* ``model.init`` in {"reference", "normal"}: reference = U(+-1/sqrt(in)) linears, N(0,1) embedding
  (``model.py:112-120,202-209,248``); normal = N(0, 0.02) everywhere.
* ``dataset.name == "synthetic"``: uniform-random token ids from a fixed seed instead of a HF dataset.
* ``distributed.comm`` in {"fused", "nccl"}: hand-written peer-memory collectives or their NCCL twins.
* ``training.master_weights``: keep an fp32 copy of every parameter inside the optimizer.
* ``distributed.cp_layout`` in {"contiguous", "zigzag"}: which tokens a context-parallel rank holds. "contiguous" is the
  reference's layout; "zigzag" (an early and a late half-chunk per rank) balances the causal attention work over the ranks.
* ``distributed.sequence_parallel``: between the tensor-parallel GEMMs every TP rank keeps 1/tp of the tokens (norms,
  residuals, pipeline messages); all-reduces become reduce-scatter + all-gather pairs. Not in the reference.
* ``checkpoint.save_on_signal``: SIGUSR1 / SIGTERM on any rank -> all ranks finish the step, save it and exit cleanly.
* ``checkpoint.async_save``: snapshot the state to host memory and write the files from a background thread.
* ``training.verify_replicas_every``: every n steps check bitwise that replicated parameters still agree between ranks.
* ``training.eval_every`` (+ ``eval_batches``, ``eval_samples``; ``dataset.eval_name`` / ``eval_split``): every n steps the
  mean loss over a fixed set of held-out micro-batches, forward only (also through the pipeline stages).
* ``training.zero1``: shard the optimizer state (moments, master weights) over the context/data-parallel replicas.
* ``training.skip_nonfinite_steps``: when the loss or any gradient of any rank is inf/NaN, all ranks skip that update.
* ``training.weight_decay``, ``training.adam_betas``, ``training.adam_eps``: AdamW hyper-parameters (the reference leaves them
  at the defaults of ``torch.optim.AdamW``, which are the defaults here).
* ``training.max_grad_norm``: clip the global gradient 2-norm (all shards of all stages) before the update; off when absent.
* ``training.lr_schedule``: ``{"warmup_steps": n, "decay": "constant" | "linear" | "cosine", "min_lr_ratio": r,
  "total_steps": n}`` (``total_steps`` defaults to ``total_train_steps``); constant learning rate when absent, as the reference.
* ``model.rope_scaling``: the ``rope_scaling`` dictionary of a Hugging Face config (``linear`` or ``llama3``); the reference
  ignores it, which matters only when pretrained long-context weights are loaded.
* ``model.tie_word_embeddings``: the LM head shares the embedding matrix (the reference always builds a separate head).
* ``distributed.pp_layer_split`` in {"reference", "balanced", [n0, n1, ...]}: decoder layers per pipeline stage. The
  reference splits evenly; "balanced" counts the LM head as work of the last stage and gives it fewer layers.
"""
from __future__ import annotations

import copy
import json
from dataclasses import dataclass
from typing import Any, Dict, Optional


@dataclass
class ModelConfig:
    """The fields the model reads (the reference takes them from a HF ``AutoConfig``, ``model.py:91-93,257-267``)."""

    hidden_size: int = 2048
    intermediate_size: int = 8192
    num_hidden_layers: int = 24
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    vocab_size: int = 49152
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_position_embeddings: int = 2048
    rope_scaling: Optional[dict] = None  # Hugging Face "rope_scaling" (linear, llama3); None = plain RoPE as the reference
    tie_word_embeddings: bool = False  # the reference never ties (checkpoint.py:89-102); parallel/tied_embeddings.py does
    name: str = "custom"

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    def num_params(self) -> int:
        """Untied parameter count (embedding and LM head both counted, as ``utils.py:51-80`` does)."""
        h, i, l, v = self.hidden_size, self.intermediate_size, self.num_hidden_layers, self.vocab_size
        kv = self.num_key_value_heads * self.head_dim
        per_layer = 2 * h + (h * h + 2 * kv * h + h * h) + 3 * h * i
        return 2 * v * h + l * per_layer + h


MODEL_PRESETS: Dict[str, Dict[str, Any]] = {
    # name -> shape. Values are the public architecture cards of these models.
    "HuggingFaceTB/SmolLM-1.7B": dict(hidden_size=2048, intermediate_size=8192, num_hidden_layers=24,
                                      num_attention_heads=32, num_key_value_heads=32, vocab_size=49152,
                                      rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=2048),
    "HuggingFaceTB/SmolLM-360M-Instruct": dict(hidden_size=960, intermediate_size=2560, num_hidden_layers=32,
                                               num_attention_heads=15, num_key_value_heads=5, vocab_size=49152,
                                               rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=2048),
    "HuggingFaceTB/SmolLM-135M": dict(hidden_size=576, intermediate_size=1536, num_hidden_layers=30,
                                      num_attention_heads=9, num_key_value_heads=3, vocab_size=49152,
                                      rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=2048),
    "meta-llama/Llama-2-7b-hf": dict(hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                                     num_attention_heads=32, num_key_value_heads=32, vocab_size=32000,
                                     rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=4096),
    "meta-llama/Llama-3.2-1B": dict(hidden_size=2048, intermediate_size=8192, num_hidden_layers=16,
                                    num_attention_heads=32, num_key_value_heads=8, vocab_size=128256,
                                    rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=131072),
    "meta-llama/Meta-Llama-3-8B": dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                                       num_attention_heads=32, num_key_value_heads=8, vocab_size=128256,
                                       rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=8192),
    "tiny-llama-test": dict(hidden_size=128, intermediate_size=256, num_hidden_layers=4,
                            num_attention_heads=4, num_key_value_heads=2, vocab_size=512,
                            rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=128),
}
# short aliases
MODEL_PRESETS["smollm-1.7b"] = MODEL_PRESETS["HuggingFaceTB/SmolLM-1.7B"]
MODEL_PRESETS["llama-2-7b"] = MODEL_PRESETS["meta-llama/Llama-2-7b-hf"]
MODEL_PRESETS["llama-3.2-1b"] = MODEL_PRESETS["meta-llama/Llama-3.2-1B"]
MODEL_PRESETS["llama-3-8b"] = MODEL_PRESETS["meta-llama/Meta-Llama-3-8B"]

_SHAPE_KEYS = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
               "num_key_value_heads", "vocab_size", "rms_norm_eps", "rope_theta")


def preset_model_config(name: str) -> Optional[ModelConfig]:
    if name in MODEL_PRESETS:
        return ModelConfig(name=name, **MODEL_PRESETS[name])
    return None


def resolve_model_config(config: Dict[str, Any]) -> ModelConfig:
    """Model shape for a run: preset (offline) or local HF ``AutoConfig``, then the JSON overrides.

    Mirrors ``train.py:152-159`` of the reference: ``num_hidden_layers``, ``num_attention_heads`` and
    ``num_key_value_heads`` of the ``model`` section override the base shape, and
    ``max_position_embeddings`` is set to ``training.seq_length``.
    """
    msec = config["model"]
    name = msec.get("preset") or msec["name"]
    mc = preset_model_config(name)
    if mc is None:
        try:  # offline-only lookup: never touches the network
            from transformers import AutoConfig
            hf = AutoConfig.from_pretrained(msec["name"], local_files_only=True)
            mc = ModelConfig(name=msec["name"], **{k: getattr(hf, k) for k in _SHAPE_KEYS})
        except Exception as e:  # noqa: BLE001
            if all(k in msec for k in ("hidden_size", "intermediate_size", "vocab_size")):
                mc = ModelConfig(name=msec["name"])
            else:
                raise ValueError(
                    f"model '{name}' is neither a preset ({sorted(MODEL_PRESETS)}) nor available offline, "
                    f"and the config gives no explicit shape") from e
    for k in _SHAPE_KEYS + ("tie_word_embeddings", "rope_scaling"):
        if k in msec and msec[k] is not None:
            setattr(mc, k, msec[k])
    mc.max_position_embeddings = config["training"]["seq_length"]
    assert mc.hidden_size % mc.num_attention_heads == 0
    assert mc.num_attention_heads % mc.num_key_value_heads == 0
    return mc


DEFAULT_CONFIG: Dict[str, Any] = {
    "distributed": {"tp_size": 1, "cp_size": 1, "pp_size": 1, "dp_size": 1, "pp_engine": "1f1b",
                    "backend": "nccl", "use_cpu": False, "comm": "fused"},
    "model": {"name": "HuggingFaceTB/SmolLM-360M-Instruct", "num_hidden_layers": 16,
              "num_attention_heads": 16, "num_key_value_heads": 4, "dtype": "bfloat16",
              "use_flash_attention": True, "use_fused_adam": True, "init": "reference"},
    "training": {"seed": 42, "learning_rate": 3e-4, "total_train_steps": 200, "seq_length": 1024,
                 "micro_batch_size": 32, "gradient_accumulation_steps": 1, "num_samples": 400000,
                 "max_tokens": None, "master_weights": True},
    "dataset": {"name": "roneneldan/TinyStories", "subset_name": None, "num_workers": 0, "num_proc": 1, "tokenizer": None},
    "checkpoint": {"save_dir": "ckpt", "save_frequency": 300, "load_path": ""},
    "logging": {"use_wandb": False, "project_name": "picotron", "run_name": None, "metrics_jsonl": None,
                "profile": False, "nvtx": False, "phase_timers": False},
    "environment": {"OMP_NUM_THREADS": "1", "TOKENIZERS_PARALLELISM": "false", "FLASH_ATTEN": "1",
                    "HF_TOKEN": None},
}


def load_config(path_or_dict) -> Dict[str, Any]:
    """Read a JSON experiment file and fill every missing key from :data:`DEFAULT_CONFIG`."""
    if isinstance(path_or_dict, dict):
        user = path_or_dict
    else:
        with open(path_or_dict, "r") as f:
            user = json.load(f)
    cfg = copy.deepcopy(DEFAULT_CONFIG)
    for section, values in user.items():
        if isinstance(values, dict):
            cfg.setdefault(section, {}).update(values)
        else:
            cfg[section] = values
    validate_config(cfg)
    return cfg


def validate_config(cfg: Dict[str, Any]) -> None:
    d, t = cfg["distributed"], cfg["training"]
    for k in ("tp_size", "cp_size", "pp_size", "dp_size"):
        assert int(d[k]) >= 1, f"distributed.{k} must be >= 1"
    assert d["pp_engine"] in ("1f1b", "afab"), f"Invalid pipeline parallel engine: {d['pp_engine']}"
    assert t["seq_length"] % d["cp_size"] == 0, "seq_length must be divisible by cp_size for Context Parallelism"
    assert d.get("comm", "fused") in ("fused", "nccl")
    assert d.get("cp_layout", "contiguous") in ("contiguous", "zigzag")
    if d.get("cp_layout") == "zigzag":
        assert t["seq_length"] % (2 * d["cp_size"]) == 0, "the zigzag layout needs seq_length divisible by 2 * cp_size"
    if d.get("sequence_parallel"):
        assert (t["seq_length"] // d["cp_size"]) % d["tp_size"] == 0, \
            "sequence parallelism needs the tokens of a rank's sequence chunk to be divisible by tp_size"
    sched = t.get("lr_schedule")
    if sched:
        assert sched.get("decay", "constant") in ("constant", "linear", "cosine"), "training.lr_schedule.decay"
        assert int(sched.get("warmup_steps", 0)) >= 0 and 0.0 <= float(sched.get("min_lr_ratio", 0.0)) <= 1.0
    assert not t.get("max_grad_norm") or float(t["max_grad_norm"]) > 0, "training.max_grad_norm must be positive"
    split = d.get("pp_layer_split", "reference")
    assert split in ("reference", "balanced") or (isinstance(split, (list, tuple)) and len(split) == int(d["pp_size"])), \
        "distributed.pp_layer_split is 'reference', 'balanced' or a list with one layer count per pipeline stage"


def world_size_of(cfg: Dict[str, Any]) -> int:
    d = cfg["distributed"]
    return d["tp_size"] * d["cp_size"] * d["pp_size"] * d["dp_size"]
