"""Model materialisation and per-(tp, pp)-rank checkpoints.

Checkpoint layout (``checkpoint.py:243-289`` of the reference): ``<save_dir>/<step>/`` holds one file per
tensor/pipeline coordinate, ``weights_tp_rank_world_size={tp}_{tp_size}_pp_rank_world_size={pp}_{pp_size}.pth``,
with keys ``model``, ``optimizer``, ``trained_steps``, ``trained_tokens``; only ``dp_rank == 0 and cp_rank == 0``
write. State-dict keys follow the module tree and keep global layer indices under PP.

Differences: the data-parallel wrapper is unwrapped by inspection (the reference dereferences
``model.module`` whenever ``cp*dp > 1`` and crashes for CP-only jobs), files are written atomically
(temp file + rename) so that a crash never leaves a truncated checkpoint, ``load_checkpoint`` maps to
the current device, and :func:`find_latest_checkpoint` lets a restarted job resume on its own.

Initialisation: ``init_model_with_dematerialized_weights`` builds the module tree on the meta device;
``init_model_with_materialized_weights`` allocates real tensors and calls ``reset_parameters()``. The
reference reads HF safetensors at this point only to obtain correctly shaped tensors and then
overwrites them with random values (``checkpoint.py:51-53,109-111``), so here the file read is skipped
unless ``load_pretrained=True`` asks for the actual weights (TP slicing rules of
``checkpoint.py:161-222``).
"""
from __future__ import annotations

import contextlib
import copy
import json
import os
import re
import threading
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from . import process_group_manager as pgm
from .utils import assert_no_meta_tensors


@contextlib.contextmanager
def init_model_with_dematerialized_weights(include_buffers: bool = False):
    """Create every parameter (optionally buffer) registered inside the context on the meta device."""
    old_param = nn.Module.register_parameter
    old_buf = nn.Module.register_buffer

    def register_empty_parameter(module, name, param):
        old_param(module, name, param)
        if param is not None:
            cur = module._parameters[name]
            module._parameters[name] = type(cur)(cur.to(torch.device("meta")), requires_grad=cur.requires_grad)

    def register_empty_buffer(module, name, buffer, persistent=True):
        old_buf(module, name, buffer, persistent=persistent)
        if buffer is not None:
            module._buffers[name] = module._buffers[name].to(torch.device("meta"))

    try:
        nn.Module.register_parameter = register_empty_parameter
        if include_buffers:
            nn.Module.register_buffer = register_empty_buffer
        yield
    finally:
        nn.Module.register_parameter = old_param
        if include_buffers:
            nn.Module.register_buffer = old_buf


def _barrier():
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def init_model_with_materialized_weights(model, model_config, save_dir: Optional[str] = None,
                                         load_pretrained: bool = False, device="cpu"):
    """Give every meta parameter real storage on ``device`` and initialise it."""
    im = InitializationManager(model, model_config)
    if len(im.get_layer_names_in_sft_format()) == 0:
        raise Exception("Some ranks has no layers. There are too many ranks and not enough layers to distribute.")
    for module in model.modules():
        for name, p in list(module._parameters.items()):
            if p is not None and p.device.type == "meta":
                module._parameters[name] = nn.Parameter(torch.empty(p.shape, dtype=p.dtype, device=device),
                                                        requires_grad=p.requires_grad)
    assert_no_meta_tensors(model)
    im.init_model_parameters()
    if load_pretrained and save_dir is not None:
        im.load_safetensors(save_dir)
    _barrier()
    return model


class InitializationManager:
    DECODER_COMPONENTS = ["input_layernorm", "mlp.down_proj", "mlp.gate_proj", "mlp.up_proj",
                          "post_attention_layernorm", "self_attn.k_proj", "self_attn.o_proj",
                          "self_attn.q_proj", "self_attn.v_proj"]

    def __init__(self, model, model_config):
        self.model = model
        self.model_config = model_config

    def init_model_parameters(self):
        self.model.reset_parameters()

    def _is_pp(self) -> bool:
        return hasattr(self.model, "layer_distribution")

    def get_layer_names_in_sft_format(self) -> List[str]:
        """HF safetensors names of the tensors this (pp) rank owns."""
        g = pgm.get()
        ids = self.model.layer_distribution if self._is_pp() else range(self.model_config.num_hidden_layers)
        names = [f"model.layers.{i}.{c}.weight" for i in ids for c in self.DECODER_COMPONENTS]
        if self._is_pp():
            if g.pp_is_first_stage:
                names.insert(0, "model.embed_tokens.weight")
            elif g.pp_is_last_stage:
                names.append("model.norm.weight")
        else:
            names.insert(0, "model.embed_tokens.weight")
            names.append("model.norm.weight")
        return names

    _RENAMES = (("model.", ""), ("layers.", "decoder_layers."), ("embed_tokens", "embedding"),
                ("self_attn.", "attention."), ("o_proj", "out_proj"), ("lm_head", "final_proj"))

    def convert_safetensors_to_hf_name(self, sft_name: str) -> str:
        out = sft_name
        for a, b in self._RENAMES:
            out = out.replace(a, b)
        return re.sub(r"^norm", "final_norm", out)

    def adjust_tensor_size(self, tensor: torch.Tensor, name: str) -> torch.Tensor:
        """Cut this TP rank's shard out of a full HF tensor (and trim/pad head counts that were overridden)."""
        g = pgm.get()
        tp_rank, tp = g.tp_rank, g.tp_world_size
        cfg = self.model_config
        hidden = cfg.hidden_size
        if "embedding.weight" in name or "final_proj.weight" in name:
            per = cfg.vocab_size // tp
            return tensor if tensor.shape[0] == per else tensor[tp_rank * per:(tp_rank + 1) * per]
        if "attention" in name:
            head_dim = hidden // cfg.num_attention_heads
            if "out_proj.weight" in name:
                per = hidden // tp
                return tensor if tensor.shape[1] == per else tensor[:, per * tp_rank:per * (tp_rank + 1)]
            if "q_proj.weight" in name:
                full = cfg.num_attention_heads * head_dim
            elif "k_proj.weight" in name or "v_proj.weight" in name:
                full = cfg.num_key_value_heads * head_dim
            else:
                return tensor
            if tensor.shape[0] > full:
                tensor = tensor[:full]
            elif tensor.shape[0] < full:
                tensor = torch.cat([tensor, torch.zeros(full - tensor.shape[0], tensor.shape[1], dtype=tensor.dtype)])
            per = full // tp
            return tensor[tp_rank * per:(tp_rank + 1) * per]
        if "mlp" in name:
            per = cfg.intermediate_size // tp
            if "up_proj.weight" in name or "gate_proj.weight" in name:
                return tensor if tensor.shape[0] == per else tensor[tp_rank * per:(tp_rank + 1) * per]
            if "down_proj.weight" in name:
                return tensor if tensor.shape[1] == per else tensor[:, tp_rank * per:(tp_rank + 1) * per]
        return tensor

    def load_safetensors(self, save_dir: str) -> None:
        from safetensors import safe_open
        names = self.get_layer_names_in_sft_format()
        index_path = os.path.join(save_dir, "model.safetensors.index.json")
        weight_map: Dict[str, str] = {}
        if os.path.exists(index_path):
            with open(index_path) as f:
                weight_map = json.load(f)["weight_map"]
        state = {}
        for sft in names:
            path = os.path.join(save_dir, weight_map.get(sft, "model.safetensors"))
            with safe_open(path, framework="pytorch", device="cpu") as f:
                ours = self.convert_safetensors_to_hf_name(sft)
                state[ours] = self.adjust_tensor_size(f.get_tensor(sft), ours)
        own = dict(self.model.named_parameters())
        # the LM head is optional: checkpoints of tied models have none (the head then keeps its random init, as in the reference)
        g = pgm.get()
        if "final_proj.weight" in own and (not self._is_pp() or g.pp_is_last_stage):
            head_file = os.path.join(save_dir, weight_map.get("lm_head.weight", "model.safetensors"))
            if os.path.exists(head_file):
                with safe_open(head_file, framework="pytorch", device="cpu") as f:
                    if "lm_head.weight" in f.keys():
                        state["final_proj.weight"] = self.adjust_tensor_size(f.get_tensor("lm_head.weight"), "final_proj.weight")
        with torch.no_grad():
            for k, v in state.items():
                own[k].copy_(v.to(own[k].dtype))


def _host_copy(obj):
    """Deep copy of a (nested) state with every tensor cloned into host memory: a snapshot the training loop cannot
    change under the background writer."""
    if torch.is_tensor(obj):
        return obj.detach().to("cpu", copy=True)
    if isinstance(obj, dict):
        return {k: _host_copy(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_host_copy(v) for v in obj)
    return copy.deepcopy(obj)


def unwrap(model):
    """Strip data-parallel wrappers (anything exposing ``.module`` and a bucket manager or sync flag)."""
    while hasattr(model, "module") and hasattr(model, "require_backward_grad_sync"):
        model = model.module
    return model


class CheckpointManager:
    def __init__(self):
        g = pgm.get()
        self.tp_rank, self.pp_rank = g.tp_rank, g.pp_rank
        self.tp_world_size, self.pp_world_size = g.tp_world_size, g.pp_world_size
        self.cp_dp_world_size = g.cp_dp_world_size
        self.dp_rank, self.cp_rank = g.dp_rank, g.cp_rank

    def _get_checkpoint_path(self, out_dir: str) -> str:
        name = (f"weights_tp_rank_world_size={self.tp_rank}_{self.tp_world_size}"
                f"_pp_rank_world_size={self.pp_rank}_{self.pp_world_size}.pth")
        return os.path.join(out_dir, name)

    def save_checkpoint(self, model, optimizer, trained_steps, trained_tokens, out_dir, extra: Optional[dict] = None,
                        asynchronous: bool = False):
        """Write this rank's shard (writers: ``dp_rank == cp_rank == 0``).

        ``asynchronous``: the state is copied to host memory now and written by a background thread, so training resumes
        after the copy instead of after the file system; ``wait()`` (called by the next save and at the end of
        training) joins the writer and re-raises its error. A step directory counts only once its ``.done`` markers
        exist, so a run that dies during a background write resumes from the step before.
        """
        path = self._get_checkpoint_path(out_dir)
        # an optimizer sharded over the replicas reassembles its state collectively: every rank of the group takes part
        sharded = getattr(optimizer, "shard_group", None) is not None
        optimizer_state = optimizer.state_dict() if sharded else None
        if self.dp_rank == 0 and self.cp_rank == 0:
            os.makedirs(out_dir, exist_ok=True)
            ckpt = {"model": unwrap(model).state_dict(),
                    "optimizer": optimizer_state if sharded else optimizer.state_dict(),
                    "trained_steps": trained_steps, "trained_tokens": trained_tokens}
            if extra:
                ckpt.update(extra)
            if not asynchronous:
                self._write(ckpt, path)
                return
            self.wait()                                          # one write in flight at a time
            snapshot = _host_copy(ckpt)
            self._error = None
            self._writer = threading.Thread(target=self._write_guarded, args=(snapshot, path), daemon=False)
            self._writer.start()

    @staticmethod
    def _write(ckpt, path: str) -> None:
        tmp = path + ".tmp"
        torch.save(ckpt, tmp)
        os.replace(tmp, path)                                    # readers never see a half-written file ...
        with open(path + ".done", "w") as f:                     # ... and can tell a later truncation from its size
            f.write(str(os.path.getsize(path)))

    def _write_guarded(self, ckpt, path: str) -> None:
        try:
            self._write(ckpt, path)
        except BaseException as e:  # noqa: BLE001 - handed to the training thread by wait()
            self._error = e

    def wait(self) -> None:
        """Join the background writer of an asynchronous save, if any, and raise what it raised."""
        writer = getattr(self, "_writer", None)
        if writer is not None:
            writer.join()
            self._writer = None
        err, self._error = getattr(self, "_error", None), None
        if err is not None:
            raise RuntimeError(f"background checkpoint write failed: {err!r}") from err

    def load_checkpoint(self, model, optimizer, out_dir) -> Tuple[int, int]:
        path = self._get_checkpoint_path(out_dir)
        if not os.path.exists(path):
            raise FileNotFoundError(f"Checkpoint not found at {path}")
        raw = unwrap(model)
        device = next(raw.parameters()).device
        ckpt = torch.load(path, map_location=device, weights_only=False)
        own = dict(raw.named_parameters(remove_duplicate=False))        # a tied weight appears under both of its names
        with torch.no_grad():  # copy in place: parameters may alias packed storage and bucket views
            missing = set(own) - set(ckpt["model"])
            unexpected = set(ckpt["model"]) - set(own)
            if missing or unexpected:
                raise RuntimeError(f"state dict mismatch: missing {sorted(missing)}, unexpected {sorted(unexpected)}")
            for k, v in ckpt["model"].items():
                own[k].copy_(v)
        optimizer.load_state_dict(ckpt["optimizer"])
        self.last_loaded = ckpt
        return ckpt["trained_steps"], ckpt["trained_tokens"]


def find_latest_checkpoint(save_dir: str) -> Optional[str]:
    """Highest-numbered ``<save_dir>/<step>/`` that is complete for EVERY (tp, pp) coordinate of the job.

    Each rank lists the steps whose file for its own coordinate is complete; the ranks then agree on the largest step
    that all of them hold (a save that died after some coordinates had written step N and others had not must not make
    the shards of one model resume from different steps). Collective over the world group when one is initialised.
    """
    cm = CheckpointManager()
    mine = []
    if os.path.isdir(save_dir):
        for s in sorted((int(d) for d in os.listdir(save_dir) if d.isdigit()), reverse=True):
            if checkpoint_file_is_complete(cm._get_checkpoint_path(os.path.join(save_dir, str(s)))):
                mine.append(s)
    common = set(mine)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        gathered = [None] * dist.get_world_size()
        dist.all_gather_object(gathered, mine)
        for steps in gathered:
            common &= set(steps)
    return os.path.join(save_dir, str(max(common))) if common else None


def checkpoint_file_is_complete(path: str) -> bool:
    """The file exists and, when its ``.done`` marker is present, still has the size recorded after it was written
    (a checkpoint without marker, e.g. one written by the reference, is taken as complete)."""
    if not os.path.exists(path):
        return False
    marker = path + ".done"
    if not os.path.exists(marker):
        return True
    try:
        with open(marker) as f:
            return int(f.read().strip()) == os.path.getsize(path)
    except (OSError, ValueError):
        return False


# ----------------------------------------------------------------------------------------------
# export in Hugging Face naming (the inverse of InitializationManager.load_safetensors)
# ----------------------------------------------------------------------------------------------
_HF_SHARD_DIM = {"attention.q_proj": 0, "attention.k_proj": 0, "attention.v_proj": 0, "attention.out_proj": 1,
                 "mlp.gate_proj": 0, "mlp.up_proj": 0, "mlp.down_proj": 1, "embedding": 0, "final_proj": 0}


def _hf_name(ours: str) -> str:
    name = ours.replace("decoder_layers.", "layers.").replace("attention.", "self_attn.").replace("out_proj", "o_proj")
    if name.startswith("embedding."):
        return "model.embed_tokens." + name[len("embedding."):]
    if name.startswith("final_norm."):
        return "model.norm." + name[len("final_norm."):]
    if name.startswith("final_proj."):
        return "lm_head." + name[len("final_proj."):]
    return "model." + name


def export_hf_safetensors(model, out_dir: str) -> Optional[str]:
    """Write the model's weights as safetensors under Hugging Face Llama names (``model.layers.N.self_attn.q_proj.weight``,
    ``lm_head.weight``, ...), readable by ``transformers`` and by ``init_model_with_materialized_weights(load_pretrained=True)``.

    Tensor-parallel shards are gathered over the TP group; every pipeline stage writes one file
    ``model-<stage+1>-of-<stages>.safetensors`` and the first stage adds ``model.safetensors.index.json``. Only the ranks
    with ``dp_rank == cp_rank == tp_rank == 0`` write. Returns the path of the file this rank wrote (or None).
    The reference can read pretrained weights (``checkpoint.py:51-113``) but has no way back; this is that way.
    """
    from safetensors.torch import save_file
    g = pgm.get()
    raw = unwrap(model)
    tensors = {}
    for name, p in raw.named_parameters():
        t = p.detach()
        dim = next((d for key, d in _HF_SHARD_DIM.items() if key + "." in name), None)
        if g.tp_world_size > 1 and dim is not None:
            parts = [torch.empty_like(t) for _ in range(g.tp_world_size)]
            dist.all_gather(parts, t.contiguous(), group=g.tp_group)
            t = torch.cat(parts, dim=dim)
        tensors[_hf_name(name)] = t.to("cpu").contiguous().clone()
    writer = g.dp_rank == 0 and g.cp_rank == 0 and g.tp_rank == 0
    fname = "model.safetensors" if g.pp_world_size == 1 else f"model-{g.pp_rank + 1:05d}-of-{g.pp_world_size:05d}.safetensors"
    path = os.path.join(out_dir, fname)
    if writer:
        os.makedirs(out_dir, exist_ok=True)
        save_file(tensors, path, metadata={"format": "pt"})
    if g.pp_world_size > 1:
        names = [None] * g.pp_world_size
        dist.all_gather_object(names, (fname, sorted(tensors)), group=g.pp_group)
        if writer and g.pp_is_first_stage:
            weight_map = {n: f for f, ns in names for n in ns}
            with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
                json.dump({"metadata": {}, "weight_map": weight_map}, f, indent=2)
    _barrier()
    return path if writer else None
