"""Re-cut a training checkpoint for another tensor-/pipeline-parallel grid (weights AND optimizer state).

A checkpoint is one file per (tp rank, pp stage) (``checkpoint.py``; names and contents as in the reference,
``picotron/checkpoint.py:232-262``), so a run can only resume on the grid that wrote it; the reference has no way around
that. After losing part of an allocation, or to continue a run on more GPUs, this module reads every shard of a saved
step, reassembles each tensor (parameter, Adam moments, fp32 master copy), and writes the files another ``tp x pp`` grid
expects, so that ``checkpoint.load_path`` works there. Data- and context-parallel sizes never appear in a checkpoint and
can change freely (the data-loader position is copied as it is; it also records the global number of samples consumed, from
which a loader of another data-parallel size finds its place).

The layout of a rank -- which parameters it owns, in which order the optimizer numbers them, with which shard shapes --
is not restated here: each rank's modules are built on the meta device under a communicator-free stand-in for the
process grid (``process_group_manager.layout_grid``), with the same surgery the trainer applies, and read off.

Everything happens on the CPU, holding one full copy of the step in host memory (18 bytes per parameter with fp32 master
weights).
"""
from __future__ import annotations

import os
import re
from typing import Dict, List, Optional, Tuple

import torch

from . import process_group_manager as pgm
from .checkpoint import _HF_SHARD_DIM, init_model_with_dematerialized_weights

_FILE = re.compile(r"weights_tp_rank_world_size=(\d+)_(\d+)_pp_rank_world_size=(\d+)_(\d+)\.pth$")
_STATE_TENSORS = ("exp_avg", "exp_avg_sq", "master")


def checkpoint_file(tp_rank: int, tp: int, pp_rank: int, pp: int) -> str:
    return f"weights_tp_rank_world_size={tp_rank}_{tp}_pp_rank_world_size={pp_rank}_{pp}.pth"


def grid_of(step_dir: str) -> Tuple[int, int]:
    """(tp, pp) of the grid that wrote ``step_dir``, checked for completeness."""
    found = [m for m in (_FILE.match(f) for f in sorted(os.listdir(step_dir))) if m]
    if not found:
        raise FileNotFoundError(f"no checkpoint shards in {step_dir}")
    tp, pp = int(found[0].group(2)), int(found[0].group(4))
    have = {(int(m.group(1)), int(m.group(3))) for m in found if int(m.group(2)) == tp and int(m.group(4)) == pp}
    missing = [(t, p) for t in range(tp) for p in range(pp) if (t, p) not in have]
    if missing:
        raise FileNotFoundError(f"{step_dir} lacks the shards of (tp rank, pp stage) {missing} of its {tp} x {pp} grid")
    return tp, pp


def shard_dim(name: str) -> Optional[int]:
    """Dimension along which tensor parallelism cuts parameter ``name`` (None: replicated)."""
    return next((d for key, d in _HF_SHARD_DIM.items() if key + "." in name), None)


def rank_layout(model_config, tp: int, pp: int, tp_rank: int, pp_rank: int, pp_layer_split="reference",
                tie: bool = False) -> Tuple[List[Tuple[str, Tuple[int, ...]]], List[str]]:
    """What rank (tp_rank, pp_rank) of a ``tp x pp`` grid holds.

    Returns ``(state_dict_entries, optimizer_order)``: the (name, shard shape) pairs of the rank's model state dict in
    its order, and the names in the order the optimizer numbers the parameters (a tied weight appears once).
    """
    from .models.llama import Llama
    from .parallel import pipeline_parallel as _pp
    from .parallel.tensor_parallel import apply_tensor_parallel
    saved_split = _pp.LAYER_SPLIT
    with pgm.layout_grid(tp_rank, tp, pp_rank, pp):
        try:
            _pp.LAYER_SPLIT = pp_layer_split
            with init_model_with_dematerialized_weights():
                model = Llama(config=model_config)
                if tp > 1:
                    model = apply_tensor_parallel(model)
                if pp > 1:
                    model = _pp.PipelineParallel(model, model_config)
            if tie and pp == 1:
                model.final_proj.weight = model.embedding.weight
        finally:
            _pp.LAYER_SPLIT = saved_split
        entries = [(n, tuple(p.shape)) for n, p in model.named_parameters(remove_duplicate=False)]
        order = [n for n, _ in model.named_parameters()]
    return entries, order


def _merge(pieces: List[torch.Tensor], dim: Optional[int]) -> torch.Tensor:
    return pieces[0] if dim is None or len(pieces) == 1 else torch.cat(pieces, dim=dim)


def _cut(full: torch.Tensor, dim: Optional[int], tp: int, tp_rank: int, shape: Tuple[int, ...]) -> torch.Tensor:
    out = full if dim is None or tp == 1 else torch.chunk(full, tp, dim=dim)[tp_rank]
    assert tuple(out.shape) == tuple(shape), f"shard shape {tuple(out.shape)} where the target rank expects {shape}"
    return out.contiguous().clone()


def load_full_state(step_dir: str, model_config, pp_layer_split="reference", tie: bool = False) -> Dict:
    """Read every shard of ``step_dir`` and reassemble: ``{"tensors": {kind: {name: full tensor}}, "steps": {name: int},
    "param_groups": [...], "meta": {...}}`` with kind in {param, exp_avg, exp_avg_sq, master}."""
    tp, pp = grid_of(step_dir)
    pieces: Dict[str, Dict[str, List[torch.Tensor]]] = {k: {} for k in ("param",) + _STATE_TENSORS}
    steps: Dict[str, int] = {}
    meta, groups = None, None
    for pp_rank in range(pp):
        for tp_rank in range(tp):
            ckpt = torch.load(os.path.join(step_dir, checkpoint_file(tp_rank, tp, pp_rank, pp)), map_location="cpu",
                              weights_only=False)
            entries, order = rank_layout(model_config, tp, pp, tp_rank, pp_rank, pp_layer_split, tie)
            names = [n for n, _ in entries]
            if sorted(names) != sorted(ckpt["model"]):
                raise RuntimeError(f"shard (tp {tp_rank}, pp {pp_rank}) of {step_dir} holds {sorted(ckpt['model'])[:3]}... "
                                   f"where the given model shape and layer split produce {sorted(names)[:3]}...")
            for n in names:
                pieces["param"].setdefault(n, []).append(ckpt["model"][n])
            opt = ckpt["optimizer"]
            ids = [i for grp in opt["param_groups"] for i in grp["params"]]
            assert len(ids) == len(order), "optimizer of the shard numbers a different set of parameters than its model"
            for pid, n in zip(ids, order):
                st = opt["state"].get(pid)
                if not st:
                    continue
                steps[n] = int(st["step"])
                for kind in _STATE_TENSORS:
                    if kind in st:
                        pieces[kind].setdefault(n, []).append(st[kind])
            if meta is None:
                meta = {k: v for k, v in ckpt.items() if k not in ("model", "optimizer")}
                groups = [{k: v for k, v in grp.items() if k != "params"} for grp in opt["param_groups"]]
    tensors = {kind: {n: _merge(ps[:tp] if shard_dim(n) is not None else ps[:1], shard_dim(n)) for n, ps in by.items()}
               for kind, by in pieces.items()}
    return {"tensors": tensors, "steps": steps, "param_groups": groups, "meta": meta, "src_grid": (tp, pp)}


def _lookup(full: Dict[str, torch.Tensor], name: str) -> Optional[torch.Tensor]:
    if name in full:
        return full[name]
    # a tied pair has one entry when its source held both uses on one stage, two when it was split over stages
    twin = {"final_proj.weight": "embedding.weight", "embedding.weight": "final_proj.weight"}.get(name)
    return full.get(twin) if twin else None


def reshard_checkpoint(src_dir: str, dst_dir: str, model_config, tp: int, pp: int, src_layer_split="reference",
                       dst_layer_split="reference", tie: bool = False) -> List[str]:
    """Write the shards of a ``tp x pp`` grid for the step saved in ``src_dir`` into ``dst_dir``; returns the paths."""
    state = load_full_state(src_dir, model_config, src_layer_split, tie)
    T = state["tensors"]
    os.makedirs(dst_dir, exist_ok=True)
    written = []
    for pp_rank in range(pp):
        for tp_rank in range(tp):
            entries, order = rank_layout(model_config, tp, pp, tp_rank, pp_rank, dst_layer_split, tie)
            model_sd = {}
            for n, shape in entries:
                full = _lookup(T["param"], n)
                if full is None:
                    raise KeyError(f"the source checkpoint has no tensor for {n}")
                model_sd[n] = _cut(full, shard_dim(n), tp, tp_rank, shape)
            shapes = dict(entries)
            opt_state = {}
            for i, n in enumerate(order):
                src_name = n if n in state["steps"] else {"final_proj.weight": "embedding.weight",
                                                         "embedding.weight": "final_proj.weight"}.get(n)
                if src_name not in state["steps"]:
                    continue                                   # saved before the first optimizer step
                st = {"step": state["steps"][src_name]}
                for kind in _STATE_TENSORS:
                    full = _lookup(T[kind], n)
                    if full is not None:
                        st[kind] = _cut(full, shard_dim(n), tp, tp_rank, shapes[n])
                opt_state[i] = st
            groups = [dict(g) for g in state["param_groups"]]
            assert len(groups) == 1, "one parameter group is what the trainer builds"
            groups[0]["params"] = list(range(len(order)))
            ckpt = {"model": model_sd, "optimizer": {"state": opt_state, "param_groups": groups}, **state["meta"]}
            path = os.path.join(dst_dir, checkpoint_file(tp_rank, tp, pp_rank, pp))
            tmp = path + ".tmp"
            torch.save(ckpt, tmp)
            os.replace(tmp, path)
            with open(path + ".done", "w") as f:               # the completeness marker `find_latest_checkpoint` looks for
                f.write(str(os.path.getsize(path)))
            written.append(path)
    return written
