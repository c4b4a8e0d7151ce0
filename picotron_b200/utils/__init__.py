"""Logging, seeding, metrics and small helpers (surface of the reference's ``picotron/utils.py:13-116``)."""
from __future__ import annotations

import builtins
import fcntl
import json
import os
import random
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from .. import process_group_manager as pgm

_LOCK_FILE = __file__


def print(*args, is_print_rank: bool = True, **kwargs):  # noqa: A001 - same name as the reference helper
    """Print under an exclusive file lock so lines of different ranks do not interleave."""
    if not is_print_rank:
        return
    with open(_LOCK_FILE, "r") as fh:
        fcntl.flock(fh, fcntl.LOCK_EX)
        try:
            builtins.print(*args, **kwargs)
        finally:
            fcntl.flock(fh, fcntl.LOCK_UN)


def set_all_seed(seed: int) -> None:
    for module in (random, np.random):
        module.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def to_readable_format(num, precision: int = 2) -> str:
    for bound, suffix in ((1e12, "T"), (1e9, "B"), (1e6, "M"), (1e3, "K")):
        if num >= bound:
            return f"{num / bound:.{precision}f}{suffix}"
    return f"{num:.{precision}f}"


def from_readable_format(text):
    """Inverse of :func:`to_readable_format` ("43.1K" -> 43100.0)."""
    if not isinstance(text, str):
        return text
    t = text.strip().upper()
    try:
        return float(t)
    except ValueError:
        pass
    mult = {"T": 1e12, "B": 1e9, "M": 1e6, "K": 1e3}
    if t[-1] not in mult:
        raise ValueError(f"Unknown suffix: {t[-1]}")
    return float(t[:-1]) * mult[t[-1]]


# dense bf16 tensor-core peak of one B200 (the reference's default is the H100 figure 989.5e12, utils.py:43)
B200_PEAK_BF16_FLOPS = 2.25e15


def peak_flops(default: float = B200_PEAK_BF16_FLOPS) -> float:
    """Peak used for MFU: env ``PICOTRON_PEAK_FLOPS``, else the nominal dense bf16 peak of a B200."""
    v = os.environ.get("PICOTRON_PEAK_FLOPS")
    return float(v) if v else default


def flops_per_token(num_params: int, model_config) -> float:
    """``6 N + 12 L H S`` -- the formula of ``utils.py:43-49`` (N includes embedding and LM head)."""
    return 6 * num_params + 12 * model_config.num_hidden_layers * model_config.hidden_size * \
        model_config.max_position_embeddings


def get_mfu(tokens_per_second, num_params, model_config, theoretical_flops: Optional[float] = None) -> float:
    """Model FLOPs utilisation in percent; ``tokens_per_second`` is per GPU."""
    peak = theoretical_flops if theoretical_flops is not None else peak_flops()
    return tokens_per_second * flops_per_token(num_params, model_config) / peak * 100


_TP_SHARDED = ("attention", "mlp", "embed", "final_proj")


def get_num_params(model) -> int:
    """Global parameter count: TP-sharded tensors times ``tp``, summed over PP stages (``utils.py:51-80``).

    A weight shared by the embedding and the LM head (``model.tie_word_embeddings``) is counted once per use, as the
    two copies of a pipeline-parallel run are: the count feeds the MFU formula, which reads it as matmul work."""
    g = pgm.get()
    local = 0
    for name, p in model.named_parameters(remove_duplicate=False):
        local += p.numel() * (g.tp_world_size if any(k in name.lower() for k in _TP_SHARDED) else 1)
    if g.pp_world_size > 1:
        dev = next(model.parameters()).device
        t = torch.tensor(local, dtype=torch.int64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=g.pp_group)
        return int(t.item())
    return local


def assert_no_meta_tensors(model) -> None:
    meta = [f"Parameter '{n}' with shape {tuple(p.shape)}" for n, p in model.named_parameters()
            if p.device.type == "meta"]
    meta += [f"Buffer '{n}' with shape {tuple(b.shape)}" for n, b in model.named_buffers() if b.device.type == "meta"]
    assert not meta, f"Found {len(meta)} meta tensors:\n" + "\n".join(meta)


def average_loss_across_dp_cp_ranks(loss, device) -> float:
    g = pgm.get()
    t = torch.tensor([loss if loss is not None else 0.0], dtype=torch.float32, device=device)
    if g.pp_is_last_stage and g.cp_dp_world_size > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=g.cp_dp_group)
        t /= g.cp_dp_world_size
    return t.item()


def download_model(model_name: str, hf_token: Optional[str]) -> Optional[str]:
    """Fetch the HF safetensors of ``model_name`` (``utils.py:101-116``). Skipped when offline."""
    dst = os.path.join("hf_model", model_name)
    if os.path.exists(os.path.join(dst, "config.json")):
        print(f"Model {model_name} already exists at {dst}")
        return dst
    if os.environ.get("HF_HUB_OFFLINE") == "1":
        print(f"HF_HUB_OFFLINE=1: not downloading {model_name}; the run starts from random init")
        return None
    import glob
    import huggingface_hub
    os.makedirs(dst, exist_ok=True)
    huggingface_hub.snapshot_download(model_name, repo_type="model", local_dir="hf_model_safetensors", token=hf_token,
                                      allow_patterns=["*.safetensors", "*.json"])
    if not glob.glob("hf_model_safetensors/*.safetensors"):
        raise ValueError(f"Model {model_name} does not have SafeTensors files.")
    return "hf_model_safetensors"


class MetricsWriter:
    """Appends one JSON object per training step to a file (in addition to the stdout step line)."""

    def __init__(self, path: Optional[str]):
        self.path = path
        if path:
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)

    def write(self, **fields) -> None:
        if not self.path:
            return
        with open(self.path, "a") as f:
            f.write(json.dumps(fields) + "\n")


def format_step_line(rank, step, loss, tokens_per_step, tokens_per_second, tokens_per_second_per_gpu,
                     trained_tokens, max_tokens, mfu, memory_gb) -> str:
    """The step line of ``train.py:248-258`` (parsed by ``extract_metrics.py``)."""
    return (f"[rank {rank}] "
            f"Step: {step:<5d} | "
            f"Loss: {loss:6.4f} | "
            f"Global batch size: {to_readable_format(tokens_per_step):>7s} | "
            f"Tokens/s: {to_readable_format(tokens_per_second):>7s} | "
            f"Tokens/s/GPU: {to_readable_format(tokens_per_second_per_gpu):>7s} | "
            f"Tokens: {to_readable_format(trained_tokens):>7s}{('/' + to_readable_format(max_tokens)) if max_tokens else ''} | "
            f"MFU: {mfu:5.2f}% | "
            f"Memory usage: {memory_gb:6.2f}GB")
