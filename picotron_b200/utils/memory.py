"""Per-GPU memory plan of a run: will this grid fit the 180 GB of a B200, and what takes the space.

The reference has no such tool (its users find out from ``torch.cuda.memory_reserved()`` in the step line,
``train.py:257``). The arithmetic below follows what this package actually keeps:

* **model state** per parameter this rank owns: the weight in the compute dtype, its fp32 gradient-bucket slot
  (``DataParallelBucket``), two fp32 Adam moments and, unless ``training.master_weights`` is off, an fp32 master copy
  (``FusedAdamW``): 2 + 4 + 8 + 4 = 18 bytes for bf16.
* **activations** per micro-batch in flight: exactly the tensors ``DecoderLayerFn`` saves for its hand-written
  backward (layer input, both normed inputs, packed post-RoPE qkv, attention output and LSE, mid residual, gate/up
  pre-activations, SwiGLU output, two rstd vectors), the embedding's and the final norm's inputs, and the head's
  input gradient, which the fused linear + cross entropy produces during the forward pass.
* **micro-batches in flight**: 1 without pipeline parallelism, all of a step's under AFAB, ``pp - stage`` under 1F1B.
* **transients**: the largest short-lived buffers of a layer's backward pass and the ``[chunk, V / tp]`` logits of the head.
* **communication workspaces** of the fused collectives (symmetric memory): the gradient buckets themselves are the
  data-parallel workspace (already counted as gradients) plus a staging area; the tensor-parallel ring of four slots;
  the context-parallel K/V publication, gather and fp32 dK/dV areas.

The caching allocator's fragmentation and NCCL's own buffers are not modelled; ``headroom`` is what is left for them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

B200_HBM_BYTES = 180 * 10 ** 9          # what the part is sold as; nvidia-smi reports 183,359 MiB


@dataclass
class MemoryPlan:
    stage: int
    params: int                          # parameters this rank owns
    bytes: Dict[str, int] = field(default_factory=dict)

    @property
    def total(self) -> int:
        return sum(self.bytes.values())

    @property
    def headroom(self) -> int:
        return B200_HBM_BYTES - self.total

    def fits(self, capacity: int = B200_HBM_BYTES, reserve: float = 0.08) -> bool:
        """True when the plan leaves ``reserve`` of the capacity for the allocator, NCCL and the CUDA context."""
        return self.total <= capacity * (1.0 - reserve)

    def summary(self) -> str:
        gib = 1 << 30
        parts = ", ".join(f"{k} {v / gib:.1f}" for k, v in self.bytes.items() if v)
        return (f"stage {self.stage}: {self.total / gib:.1f} GiB of {B200_HBM_BYTES / gib:.0f} GiB "
                f"({parts}; {self.params / 1e9:.2f} B parameters on this rank)")


def layers_of_stage(model_config, pp: int, stage: int, split="reference") -> int:
    """Decoder layers on pipeline stage ``stage`` for ``distributed.pp_layer_split`` = ``split``."""
    n = model_config.num_hidden_layers
    if isinstance(split, (list, tuple)):
        return int(split[stage])
    if split == "balanced" and pp > 1:
        from ..parallel.pipeline_parallel import balanced_layer_split
        return balanced_layer_split(model_config, pp)[stage]
    return n // pp + (1 if stage < n % pp else 0)


def params_of_rank(model_config, tp: int, pp: int, stage: int, split="reference", tie: bool = False) -> int:
    """Parameters one rank of pipeline stage ``stage`` holds (TP shards of the matrices, whole norm vectors)."""
    h, i, v = model_config.hidden_size, model_config.intermediate_size, model_config.vocab_size
    kv = model_config.num_key_value_heads * (h // model_config.num_attention_heads)
    layer = (2 * h * h + 2 * kv * h + 3 * h * i) // tp + 2 * h
    n = layers_of_stage(model_config, pp, stage, split) * layer
    if stage == 0:
        n += v * h // tp
    if stage == pp - 1:
        n += h + (0 if tie and pp == 1 else v * h // tp)
    return n


def layer_activation_bytes(model_config, tokens: int, batch: int, tp: int, dtype_bytes: int = 2,
                           sequence_parallel: bool = False) -> int:
    """Bytes one decoder layer keeps from forward to backward for ``tokens`` tokens (``batch`` sequences) on one rank."""
    h, i = model_config.hidden_size, model_config.intermediate_size
    d = h // model_config.num_attention_heads
    hq, hkv = model_config.num_attention_heads // tp, model_config.num_key_value_heads // tp
    rep = tokens // tp if sequence_parallel else tokens            # rows of the token-wise replicated tensors
    saved = 4 * rep * h * dtype_bytes                              # layer input, normed input, mid residual, second normed input
    saved += 2 * rep * 4                                           # two fp32 rstd vectors
    saved += tokens * (hq + 2 * hkv) * d * dtype_bytes             # packed q, k, v after RoPE
    saved += tokens * hq * d * dtype_bytes                         # attention output
    saved += tokens * hq * 4                                       # fp32 log-sum-exp per (token, head)
    saved += tokens * 3 * (i // tp) * dtype_bytes                  # gate/up pre-activations and silu(gate) * up
    return saved


def plan_memory(model_config, tp: int = 1, cp: int = 1, pp: int = 1, dp: int = 1, micro_batch_size: int = 1,
                seq_length: int = 1024, grad_acc_steps: int = 1, pp_engine: str = "1f1b", stage: int = 0,
                dtype_bytes: int = 2, master_weights: bool = True, sequence_parallel: bool = False,
                pp_layer_split="reference", tie_word_embeddings: bool = False, fused_comm: bool = True,
                ce_chunk_tokens: int = 2048, zero1: bool = False) -> MemoryPlan:
    """Memory plan of one rank on pipeline stage ``stage``."""
    mc = model_config
    h, v = mc.hidden_size, mc.vocab_size
    sp = sequence_parallel and tp > 1
    tokens = micro_batch_size * seq_length // cp                   # tokens of one micro-batch on this rank
    rep = tokens // tp if sp else tokens
    n = params_of_rank(mc, tp, pp, stage, pp_layer_split, tie_word_embeddings)
    plan = MemoryPlan(stage=stage, params=n)
    b = plan.bytes
    b["weights"] = n * dtype_bytes
    b["gradients"] = n * 4
    b["optimizer"] = n * (12 if master_weights else 8) // (cp * dp if zero1 else 1)   # training.zero1: one owner per parameter

    # ---- activations
    layers = layers_of_stage(mc, pp, stage, pp_layer_split)
    per_mb = layers * layer_activation_bytes(mc, tokens, micro_batch_size, tp, dtype_bytes, sp)
    if stage == 0:
        per_mb += tokens * 8                                       # token ids kept by the embedding's backward
    if stage == pp - 1:
        per_mb += rep * h * dtype_bytes + rep * 4                  # final norm: its input and rstd
        per_mb += tokens * h * dtype_bytes                         # dh, produced by the fused head during the forward pass
        if sp:
            per_mb += tokens * h * dtype_bytes                     # the gathered head input
    if pp > 1 and stage > 0:
        per_mb += rep * h * dtype_bytes                            # the received activation (pooled buffer)
    if pp > 1 and stage < pp - 1:
        per_mb += rep * h * dtype_bytes                            # the stage's output, kept until its gradient arrives
    in_flight = 1 if pp == 1 else (grad_acc_steps if pp_engine == "afab" else min(pp - stage, grad_acc_steps))
    b["activations"] = per_mb * in_flight

    # ---- transients: the backward of one layer, or the head's logits chunk, whichever is larger
    i_loc = mc.intermediate_size // tp
    d = h // mc.num_attention_heads
    qkv_cols = (mc.num_attention_heads + 2 * mc.num_key_value_heads) // tp * d
    layer_bwd = tokens * (2 * i_loc + 2 * h + qkv_cols) * dtype_bytes + tokens * (mc.num_attention_heads // tp) * d * 4
    head = min(ce_chunk_tokens, tokens) * (v // tp) * dtype_bytes if stage == pp - 1 else 0
    b["transients"] = max(layer_bwd, head)

    # ---- symmetric-memory workspaces of the fused collectives
    ws = 0
    if fused_comm:
        if cp * dp > 1:
            ws += 64 << 20                                         # staging area of the gradient all-reduce
        if tp > 1:
            ws += 4 * tokens * h * dtype_bytes + (128 << 10)       # ring of four [tokens, hidden] slots + statistics scratch
        if cp > 1:
            kv = 2 * tokens * (mc.num_key_value_heads // tp) * d
            ws += kv * dtype_bytes                                 # this rank's published K/V chunk
            ws += (cp - 1) * kv * dtype_bytes                      # the gathered remote chunks
            ws += 2 * (cp - 1) * kv * 4                            # fp32 dK/dV partials for the other ranks, and theirs for us
    b["comm_workspaces"] = ws
    return plan


def plan_all_stages(model_config, config: dict) -> List[MemoryPlan]:
    """Plans for every pipeline stage of a run described by a loaded config dictionary."""
    d, t, m = config["distributed"], config["training"], config["model"]
    return [plan_memory(model_config, tp=d["tp_size"], cp=d["cp_size"], pp=d["pp_size"], dp=d["dp_size"],
                        micro_batch_size=t["micro_batch_size"], seq_length=t["seq_length"],
                        grad_acc_steps=t["gradient_accumulation_steps"], pp_engine=d.get("pp_engine", "1f1b"), stage=s,
                        dtype_bytes=4 if m.get("dtype") == "float32" else 2,
                        master_weights=bool(t.get("master_weights", True)),
                        sequence_parallel=bool(d.get("sequence_parallel", False)),
                        pp_layer_split=d.get("pp_layer_split", "reference"),
                        tie_word_embeddings=bool(m.get("tie_word_embeddings", False)), zero1=bool(t.get("zero1", False)),
                        fused_comm=d.get("comm", "fused") == "fused" and not d.get("use_cpu", False))
            for s in range(d["pp_size"])]


def check_fits(model_config, config: dict, capacity: Optional[int] = None) -> List[str]:
    """Human-readable warnings for the stages whose plan does not fit the device (empty list: everything fits)."""
    cap = capacity or B200_HBM_BYTES
    return [f"{p.summary()} -- does not fit {cap / (1 << 30):.0f} GiB with 8 % reserve: raise tp/pp/cp, lower the "
            f"micro-batch, shard the optimizer over the replicas (training.zero1) or, with tp > 1, enable "
            f"distributed.sequence_parallel"
            for p in plan_all_stages(model_config, config) if not p.fits(cap)]


def describe_run(config: dict) -> List[str]:
    """What a run of ``config`` would put on each pipeline stage, without any GPU or process group: the layers and the
    parameter tensors of tensor-parallel rank 0 of every stage (built on the meta device with the trainer's own
    surgery, so an impossible grid -- heads not divisible by tp, more stages than layers -- fails here the way it would
    at start-up), the memory plan, and the tokens per optimizer step. Returns the report as lines."""
    from ..config import resolve_model_config
    from ..reshard import rank_layout
    d, t, m = config["distributed"], config["training"], config["model"]
    mc = resolve_model_config(config)
    tp, pp = d["tp_size"], d["pp_size"]
    world = tp * pp * d["cp_size"] * d["dp_size"]
    tokens = t["micro_batch_size"] * t["gradient_accumulation_steps"] * d["dp_size"] * t["seq_length"]
    lines = [f"{mc.name}: {mc.num_hidden_layers} layers, hidden {mc.hidden_size}, {mc.num_attention_heads} query / "
             f"{mc.num_key_value_heads} KV heads, vocabulary {mc.vocab_size}; {mc.num_params() / 1e9:.2f} B parameters (untied count)",
             f"grid: dp {d['dp_size']} x pp {pp} x cp {d['cp_size']} x tp {tp} = {world} ranks; {tokens:,} tokens per optimizer step; "
             f"{t['seq_length'] // d['cp_size']} tokens of a sequence per rank"]
    plans = plan_all_stages(mc, config)
    for stage in range(pp):
        entries, _ = rank_layout(mc, tp, pp, 0, stage, d.get("pp_layer_split", "reference"),
                                 bool(m.get("tie_word_embeddings", False)))
        layers = sorted({int(n.split(".")[1]) for n, _ in entries if n.startswith("decoder_layers.")})
        extras = [k for k in ("embedding", "final_norm", "final_proj") if any(n.startswith(k + ".") for n, _ in entries)]
        lines.append(f"stage {stage}: layers {layers[0]}-{layers[-1]} ({len(layers)})" + (f" + {', '.join(extras)}" if extras else "")
                     + f"; {len(entries)} parameter tensors per rank")
        lines.append("  memory per GPU, " + plans[stage].summary())
    lines += ["WARNING: " + w for w in check_fits(mc, config)]
    return lines
