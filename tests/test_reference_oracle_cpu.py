"""Parity with the reference's OWN modules, run on CPU/Gloo as the oracle (skipped when no reference install is present).

The unmodified reference sources are expected under ``baseline/_ref`` (``picotron/`` and ``train.py``). They import
flash-attn unconditionally and call ``torch.cuda.synchronize()`` after every pipeline message, so the worker process
puts empty stand-ins for the three flash-attn modules into ``sys.modules`` (they are never called with ``FLASH_ATTEN=0``)
and makes ``torch.cuda.synchronize`` a no-op; nothing in the reference's files is changed. Both implementations get the
same weights (copied by parameter name: the state-dict names are identical by design) and the same batches; losses and
gradients must agree to float32 round-off.

Covered: tensor parallel (tp2: the reference's Column/Row/VocabParallel modules and its logits all-gather against the
fused TP layer and the statistics-only cross entropy), bucketed data parallel with gradient accumulation (dp2: the
reference's ``train_step`` and ``DataParallelBucket``), both pipeline schedules (pp2 1F1B and AFAB, with the reference's
loss scaling switched on in this package), ring attention over two sequence chunks (cp2 x dp2: the reference averages
gradients over the context-parallel ranks only when a data-parallel wrapper is present, so the grid has dp = 2), and the
full 8-rank grid dp2 x tp2 x pp2.
"""
import os
import sys
import types
from types import SimpleNamespace

import pytest
import torch

from dist_utils import run_distributed

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
pytestmark = pytest.mark.skipif(not os.path.exists(os.path.join(REF, "picotron", "model.py")),
                                reason="no reference sources under baseline/_ref")

SHAPE = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
             vocab_size=96, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=16)
MBS, SEQ, GRAD_ACC = 2, 16, 2


def _prepare_reference(rank):
    """Make the reference importable in this (CPU-only) process without touching its files."""
    os.environ.update(FLASH_ATTEN="0", DEVICE="cpu", DTYPE="float32", LOCAL_RANK=str(rank), HF_TOKEN="offline",
                      WANDB_MODE="disabled")
    os.environ.pop("CONTEXT_PARALLEL", None)
    for name in ("flash_attn", "flash_attn.flash_attn_interface", "flash_attn.layers", "flash_attn.layers.rotary",
                 "flash_attn.ops", "flash_attn.ops.triton", "flash_attn.ops.triton.layer_norm"):
        sys.modules[name] = types.ModuleType(name)
    sys.modules["flash_attn.flash_attn_interface"].flash_attn_func = None
    sys.modules["flash_attn.layers.rotary"].apply_rotary_emb = None
    sys.modules["flash_attn.ops.triton.layer_norm"].layer_norm_fn = None
    try:
        import wandb  # noqa: F401
    except Exception:  # noqa: BLE001
        sys.modules["wandb"] = types.ModuleType("wandb")
    torch.cuda.synchronize = lambda *a, **k: None
    if REF not in sys.path:
        sys.path.insert(0, REF)


class _Loader:
    """The few attributes and the batch dict the reference's step functions read (``train.py:29-55``)."""

    def __init__(self, dp_rank, vocab, n, cp_rank=0, cp=1):
        self.grad_acc_steps, self.micro_batch_size, self.seq_length_per_gpu = GRAD_ACC, MBS, SEQ // cp
        self.lo, self.hi = cp_rank * (SEQ // cp), (cp_rank + 1) * (SEQ // cp)      # contiguous chunk of this CP rank
        g = torch.Generator().manual_seed(1234 + dp_rank)
        self.batches = [torch.randint(0, vocab, (MBS, SEQ + 1), generator=g) for _ in range(n)]
        self.i = 0

    def __iter__(self):
        return self

    def __next__(self):
        ids = self.batches[self.i % len(self.batches)]
        self.i += 1
        return {"input_ids": ids[:, :-1][:, self.lo:self.hi].contiguous(),
                "target_ids": ids[:, 1:][:, self.lo:self.hi].contiguous(),
                "position_ids": torch.arange(self.lo, self.hi).unsqueeze(0).expand(MBS, -1).contiguous(),
                "hidden_states": None}


def _copy_weights(ref_model, our_model):
    ref = dict(ref_model.named_parameters())
    ours = dict(our_model.named_parameters())
    assert set(ref) == set(ours), (sorted(set(ref) ^ set(ours)))
    with torch.no_grad():
        for n, p in ours.items():
            assert p.shape == ref[n].shape, (n, p.shape, ref[n].shape)
            p.copy_(ref[n])


def _max_rel(a, b):
    return float((a - b).abs().max() / (b.abs().max() + 1e-12))


def _worker(rank, world, mode):
    _prepare_reference(rank)
    tp, pp, dp, cp = GRIDS[mode]
    afab = mode.endswith("afab")
    device = torch.device("cpu")
    ref_cfg = SimpleNamespace(**SHAPE)
    # ------------------------------------------------------------------ the reference
    import picotron.process_group_manager as rpgm
    rpgm.setup_process_group_manager(tp_size=tp, cp_size=cp, pp_size=pp, dp_size=dp)
    from picotron.model import Llama as RefLlama
    from picotron.tensor_parallel.tensor_parallel import apply_tensor_parallel as ref_apply_tp
    from picotron.data_parallel.data_parallel import DataParallelBucket as RefDPB
    from picotron.pipeline_parallel.pipeline_parallel import PipelineParallel as RefPP
    from picotron.pipeline_parallel.pipeline_parallel import train_step_pipeline_1f1b as ref_1f1b
    from picotron.pipeline_parallel.pipeline_parallel import train_step_pipeline_afab as ref_afab
    from picotron.context_parallel.context_parallel import apply_context_parallel as ref_apply_cp
    import train as ref_train
    torch.manual_seed(7)
    ref = RefLlama(ref_cfg)
    if tp > 1:
        ref = ref_apply_tp(ref)
    if cp > 1:
        ref = ref_apply_cp(ref)
    if pp > 1:
        ref = RefPP(ref, ref_cfg)
    ref_raw = ref
    if dp > 1:
        ref = RefDPB(ref)
    ref.train()
    # ------------------------------------------------------------------ this package, same grid, same weights
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.config import ModelConfig
    from picotron_b200.models.llama import Llama
    from picotron_b200.parallel import pipeline_parallel as our_pp
    from picotron_b200.parallel.context_parallel import apply_context_parallel
    from picotron_b200.parallel.data_parallel import DataParallelBucket
    from picotron_b200.parallel.tensor_parallel import apply_tensor_parallel
    from picotron_b200.trainer import train_step
    g = pgm.setup_process_group_manager(tp_size=tp, cp_size=cp, pp_size=pp, dp_size=dp)
    ours = Llama(ModelConfig(**SHAPE))
    if tp > 1:
        ours = apply_tensor_parallel(ours)
    if cp > 1:
        ours = apply_context_parallel(ours)
    if pp > 1:
        ours = our_pp.PipelineParallel(ours, ModelConfig(**SHAPE))
    _copy_weights(ref_raw, ours)
    ours_raw = ours
    ours = DataParallelBucket(ours)
    ours.train()
    # ------------------------------------------------------------------ one optimizer step's worth of micro-batches each
    def loader():
        return _Loader(g.dp_rank, SHAPE["vocab_size"], GRAD_ACC, g.cp_rank, cp)

    shapes = (MBS, SEQ // cp, SHAPE["hidden_size"])
    if pp > 1:
        our_pp.REFERENCE_LOSS_SCALING = True             # the reference back-propagates the unscaled micro-batch loss
        ref_step = ref_afab if afab else ref_1f1b
        our_step = our_pp.train_step_pipeline_afab if afab else our_pp.train_step_pipeline_1f1b
        ref_loss = ref_step(ref, loader(), shapes, device, torch.float32)
        our_loss = our_step(ours, loader(), shapes, device, torch.float32)
        our_pp.REFERENCE_LOSS_SCALING = False
    else:
        ref_loss = ref_train.train_step(ref, loader(), device)
        our_loss = train_step(ours, loader(), device)
    out = {"ref_loss": float(ref_loss), "our_loss": float(our_loss), "last": bool(g.pp_is_last_stage), "errs": {}}
    ref_params = dict(ref_raw.named_parameters())
    for n, p in ours_raw.named_parameters():
        rg = ref_params[n].main_grad if dp * cp > 1 else ref_params[n].grad
        out["errs"][n] = _max_rel(p.main_grad.float(), rg.float())
    return out


# mode -> (tp, pp, dp, cp)
GRIDS = {"tp2": (2, 1, 1, 1), "dp2": (1, 1, 2, 1), "pp2": (1, 2, 1, 1), "pp2_afab": (1, 2, 1, 1), "cp2_dp2": (1, 1, 2, 2),
         "dp2_tp2_pp2": (2, 2, 2, 1)}


@pytest.mark.parametrize("mode", list(GRIDS))
def test_losses_and_gradients_match_the_reference_modules(mode):
    tp, pp, dp, cp = GRIDS[mode]
    for r in run_distributed(_worker, tp * pp * dp * cp, mode, timeout=600):
        if r["last"]:
            assert abs(r["ref_loss"] - r["our_loss"]) < 2e-5 * max(1.0, abs(r["ref_loss"])), r
        worst = max(r["errs"].items(), key=lambda kv: kv[1])
        assert worst[1] < 2e-4, f"{mode}: gradient of {worst[0]} differs from the reference by {worst[1]:.2e} (relative)"
