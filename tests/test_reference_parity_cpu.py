"""CPU counterparts of the reference's own test scripts and of paths those scripts leave out.

* ``tests/test_tensor_parallel.py`` of the reference: Column/Row parallel linears against one ``nn.Linear`` whose weight
  is chunked across ranks (forward and all gradients, bias included), here under Gloo instead of NCCL.
* ``tests/test_dataloader.py::test_cp_behavior``: the context-parallel slice of a batch equals the same columns of the
  un-split batch; the loader restarts after its last batch.
* pretrained weights from a safetensors file, cut per TP rank (``checkpoint.py:161-222`` of the reference).
"""
import json
import os

import numpy as np
import pytest
import torch
import torch.nn as nn

from dist_utils import run_distributed


# --------------------------------------------------------------------------------------------- tensor parallel linears
def _tp_linear_worker(rank, world):
    import torch.distributed as dist
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear
    pgm.setup_process_group_manager(tp_size=world, cp_size=1, pp_size=1, dp_size=1)
    torch.manual_seed(42)                                   # every rank builds the same full layer and input
    B, S, fin, fout = 2, 4, 8, 16
    full = nn.Linear(fin, fout, bias=True)
    x = torch.randn(B, S, fin, requires_grad=True)
    y_full = full(x)
    y_full.sum().backward()

    col = ColumnParallelLinear(fin, fout, bias=True, gather_output=True)
    row = RowParallelLinear(fin, fout, bias=True)
    with torch.no_grad():
        col.weight.copy_(full.weight.chunk(world, dim=0)[rank])
        col.bias.copy_(full.bias.chunk(world, dim=0)[rank])
        row.weight.copy_(full.weight.chunk(world, dim=1)[rank])
        row.bias.copy_(full.bias)
    xc = x.detach().clone().requires_grad_(True)
    yc = col(xc)
    yc.sum().backward()
    xr = x.detach().clone().chunk(world, dim=-1)[rank].contiguous().requires_grad_(True)
    yr = row(xr)
    yr.sum().backward()
    return {
        "col_fwd": float((yc - y_full).abs().max()), "row_fwd": float((yr - y_full).abs().max()),
        "col_dw": float((col.weight.grad - full.weight.grad.chunk(world, dim=0)[rank]).abs().max()),
        "col_db": float((col.bias.grad - full.bias.grad.chunk(world, dim=0)[rank]).abs().max()),
        "col_dx": float((xc.grad - x.grad).abs().max()),
        "row_dw": float((row.weight.grad - full.weight.grad.chunk(world, dim=1)[rank]).abs().max()),
        "row_db": float((row.bias.grad - full.bias.grad).abs().max()),
        "row_dx": float((xr.grad - x.grad.chunk(world, dim=-1)[rank]).abs().max()),
    }


def test_column_and_row_parallel_linear_match_one_linear_tp2():
    for r in run_distributed(_tp_linear_worker, 2):
        for k, v in r.items():
            assert v < 1e-5, (k, v)


def test_column_and_row_parallel_linear_match_one_linear_tp4():
    for r in run_distributed(_tp_linear_worker, 4):
        for k, v in r.items():
            assert v < 1e-5, (k, v)


# --------------------------------------------------------------------------------------------- data loader
def _cp_loader_worker(rank, world):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.data import MicroBatchDataLoader
    pgm.setup_process_group_manager(tp_size=1, cp_size=world, pp_size=1, dp_size=1)
    kw = dict(micro_batch_size=2, seq_length=16, dataset_name="synthetic", tokenizer_name=None, num_workers=0, num_proc=1,
              grad_acc_steps=1, device=torch.device("cpu"), num_samples=6, vocab_size=97, seed=7, pin_memory=False)
    split = MicroBatchDataLoader(**kw)
    pgm.reset()
    whole = MicroBatchDataLoader(**kw)                       # single-process grid: cp = 1, sees whole sequences
    out = {"seq_per_gpu": split.seq_length_per_gpu, "ok": True, "restarts": False}
    first = None
    for i in range(5):                                       # 6 samples / micro-batch 2 = 3 batches per epoch
        a, b = next(split), next(whole)
        lo, hi = rank * split.seq_length_per_gpu, (rank + 1) * split.seq_length_per_gpu
        out["ok"] &= bool(torch.equal(a["input_ids"], b["input_ids"][:, lo:hi]))
        out["ok"] &= bool(torch.equal(a["target_ids"], b["target_ids"][:, lo:hi]))
        out["ok"] &= bool(torch.equal(a["position_ids"][0], torch.arange(lo, hi)))
        if i == 0:
            first = b["input_ids"].clone()
        if i == 3:
            out["restarts"] = bool(torch.equal(b["input_ids"], first))
    out["epoch"] = whole.epoch
    return out


def test_context_parallel_slices_of_the_loader_and_restart():
    for r in run_distributed(_cp_loader_worker, 2):
        assert r["seq_per_gpu"] == 8
        assert r["ok"] and r["restarts"] and r["epoch"] == 1


class _CharTokenizer:
    """Stand-in for a HF tokenizer: one id per character."""

    def __call__(self, texts, return_attention_mask=False, return_token_type_ids=False):
        return {"input_ids": [[ord(c) % 251 for c in t] for t in texts]}


def test_text_is_concatenated_and_cut_into_overlapping_windows():
    from picotron_b200.data import MicroBatchDataLoader, group_into_windows
    texts = ["hello world, ", "this is a tokenizer-free test. ", "abc"]
    out = MicroBatchDataLoader.tokenizer_group_text(texts, _CharTokenizer(), 8)["input_ids"]
    flat = np.asarray([ord(c) % 251 for c in "".join(texts)])
    assert all(len(w) == 9 for w in out)
    assert len(out) == (len(flat) - 1) // 8
    for i, w in enumerate(out):                              # stride = sequence_length, windows overlap by one token
        assert np.array_equal(w, flat[i * 8:i * 8 + 9])
    assert group_into_windows(np.arange(5), 8) == []


# --------------------------------------------------------------------------------------------- pretrained weights
def _write_hf_checkpoint(path, cfg, sharded):
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(3)
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    d = H // cfg["num_attention_heads"]
    t = {"model.embed_tokens.weight": torch.randn(V, H, generator=g), "model.norm.weight": torch.randn(H, generator=g)}
    for i in range(L):
        p = f"model.layers.{i}."
        t[p + "input_layernorm.weight"] = torch.randn(H, generator=g)
        t[p + "post_attention_layernorm.weight"] = torch.randn(H, generator=g)
        t[p + "self_attn.q_proj.weight"] = torch.randn(cfg["num_attention_heads"] * d, H, generator=g)
        t[p + "self_attn.k_proj.weight"] = torch.randn(cfg["num_key_value_heads"] * d, H, generator=g)
        t[p + "self_attn.v_proj.weight"] = torch.randn(cfg["num_key_value_heads"] * d, H, generator=g)
        t[p + "self_attn.o_proj.weight"] = torch.randn(H, H, generator=g)
        t[p + "mlp.gate_proj.weight"] = torch.randn(I, H, generator=g)
        t[p + "mlp.up_proj.weight"] = torch.randn(I, H, generator=g)
        t[p + "mlp.down_proj.weight"] = torch.randn(H, I, generator=g)
    os.makedirs(path, exist_ok=True)
    if not sharded:
        save_file(t, os.path.join(path, "model.safetensors"))
    else:
        names = sorted(t)
        half = len(names) // 2
        files = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
        weight_map = {}
        for fn, ns in files.items():
            save_file({n: t[n] for n in ns}, os.path.join(path, fn))
            weight_map.update({n: fn for n in ns})
        with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
            json.dump({"weight_map": weight_map}, f)
    return t


_HF_CFG = dict(hidden_size=32, intermediate_size=64, vocab_size=96, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2)


def _pretrained_worker(rank, world, path):
    from safetensors import safe_open
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.checkpoint import init_model_with_dematerialized_weights, init_model_with_materialized_weights
    from picotron_b200.config import ModelConfig
    from picotron_b200.models.llama import Llama
    from picotron_b200.parallel.tensor_parallel import apply_tensor_parallel
    pgm.setup_process_group_manager(tp_size=world, cp_size=1, pp_size=1, dp_size=1)
    cfg = ModelConfig(**_HF_CFG, max_position_embeddings=32)
    with init_model_with_dematerialized_weights():
        model = Llama(cfg)
        if world > 1:
            model = apply_tensor_parallel(model)
    model = init_model_with_materialized_weights(model, cfg, save_dir=path, load_pretrained=True)
    full = {}
    for fn in os.listdir(path):
        if fn.endswith(".safetensors"):
            with safe_open(os.path.join(path, fn), framework="pytorch", device="cpu") as f:
                for k in f.keys():
                    full[k] = f.get_tensor(k)
    sd = dict(model.named_parameters())
    errs = {}

    def shard(t, dim):
        return t.chunk(world, dim=dim)[rank]
    errs["embedding"] = float((sd["embedding.weight"] - shard(full["model.embed_tokens.weight"], 0)).abs().max())
    errs["norm"] = float((sd["final_norm.weight"] - full["model.norm.weight"]).abs().max())
    for i in range(cfg.num_hidden_layers):
        p, q = f"model.layers.{i}.", f"decoder_layers.{i}."
        errs[f"q{i}"] = float((sd[q + "attention.q_proj.weight"] - shard(full[p + "self_attn.q_proj.weight"], 0)).abs().max())
        errs[f"k{i}"] = float((sd[q + "attention.k_proj.weight"] - shard(full[p + "self_attn.k_proj.weight"], 0)).abs().max())
        errs[f"o{i}"] = float((sd[q + "attention.out_proj.weight"] - shard(full[p + "self_attn.o_proj.weight"], 1)).abs().max())
        errs[f"up{i}"] = float((sd[q + "mlp.up_proj.weight"] - shard(full[p + "mlp.up_proj.weight"], 0)).abs().max())
        errs[f"down{i}"] = float((sd[q + "mlp.down_proj.weight"] - shard(full[p + "mlp.down_proj.weight"], 1)).abs().max())
        errs[f"ln{i}"] = float((sd[q + "input_layernorm.weight"] - full[p + "input_layernorm.weight"]).abs().max())
    # the LM head is not part of the checkpoint (the reference always creates an untied one): it keeps its random init
    errs["head_is_finite"] = 0.0 if bool(torch.isfinite(sd["final_proj.weight"]).all()) else 1.0
    return errs


def test_pretrained_safetensors_single_file_single_rank(tmp_path):
    path = str(tmp_path / "hf")
    _write_hf_checkpoint(path, _HF_CFG, sharded=False)
    for r in run_distributed(_pretrained_worker, 1, path):
        assert max(r.values()) == 0.0, r


def test_pretrained_safetensors_sharded_index_tp2(tmp_path):
    path = str(tmp_path / "hf")
    _write_hf_checkpoint(path, _HF_CFG, sharded=True)
    for r in run_distributed(_pretrained_worker, 2, path):
        assert max(r.values()) == 0.0, r


def test_local_text_file_with_byte_tokenizer_end_to_end(tmp_path):
    """The HF branch of the loader (datasets.map + grouping) on a local text file with the offline byte tokenizer."""
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.data import ByteTokenizer, MicroBatchDataLoader
    pgm.reset()
    lines = [f"line {i}: the quick brown fox jumps over the lazy dog." for i in range(40)]
    path = tmp_path / "corpus.txt"
    path.write_text("\n".join(lines))
    dl = MicroBatchDataLoader(micro_batch_size=2, seq_length=32, dataset_name=str(path), tokenizer_name="bytes",
                              num_workers=0, num_proc=1, grad_acc_steps=1, device=torch.device("cpu"), pin_memory=False)
    stream = np.concatenate([np.frombuffer(t.encode(), dtype=np.uint8).astype(np.int64) for t in lines])
    n_windows = (len(stream) - 1) // 32
    assert len(dl.tokenized_dataset) == n_windows
    b = next(dl)
    assert b["input_ids"].shape == (2, 32) and b["target_ids"].shape == (2, 32)
    assert torch.equal(b["input_ids"][0], torch.from_numpy(stream[:32]))
    assert torch.equal(b["target_ids"][0], torch.from_numpy(stream[1:33]))          # targets are the inputs shifted by one
    assert torch.equal(b["input_ids"][1], torch.from_numpy(stream[32:64]))           # stride = seq_length
    assert ByteTokenizer().decode(b["input_ids"][0].tolist()).startswith("line 0: the quick")


def _export_roundtrip_worker(rank, world, tp, pp, path, tie=False):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.checkpoint import (export_hf_safetensors, init_model_with_dematerialized_weights,
                                          init_model_with_materialized_weights)
    from picotron_b200.config import ModelConfig
    from picotron_b200.models.llama import Llama
    from picotron_b200.parallel.pipeline_parallel import PipelineParallel
    from picotron_b200.parallel.tensor_parallel import apply_tensor_parallel
    pgm.setup_process_group_manager(tp_size=tp, cp_size=1, pp_size=pp, dp_size=world // (tp * pp))
    cfg = ModelConfig(**_HF_CFG, max_position_embeddings=32)

    def build(load):
        with init_model_with_dematerialized_weights():
            m = Llama(cfg)
            if tp > 1:
                m = apply_tensor_parallel(m)
            if pp > 1:
                m = PipelineParallel(m, cfg)
        m = init_model_with_materialized_weights(m, cfg, save_dir=path, load_pretrained=load)
        if tie:
            from picotron_b200.parallel.tied_embeddings import tie_word_embeddings
            tie_word_embeddings(m)
        return m

    torch.manual_seed(11)
    src = build(False)
    with torch.no_grad():                                   # make every tensor distinctive, norms included
        for i, p in enumerate(src.parameters()):
            p.add_(0.01 * (i + 1))
    export_hf_safetensors(src, path)
    torch.manual_seed(999)
    dst = build(True)
    return {n: float((p - dict(dst.named_parameters())[n]).abs().max()) for n, p in src.named_parameters()}


def test_hf_export_round_trip_single_rank(tmp_path):
    from safetensors import safe_open
    path = str(tmp_path / "export")
    for r in run_distributed(_export_roundtrip_worker, 1, 1, 1, path):
        assert max(r.values()) == 0.0, r
    with safe_open(os.path.join(path, "model.safetensors"), framework="pytorch", device="cpu") as f:
        keys = set(f.keys())
    assert {"model.embed_tokens.weight", "model.norm.weight", "lm_head.weight", "model.layers.1.self_attn.o_proj.weight",
            "model.layers.0.mlp.gate_proj.weight", "model.layers.0.input_layernorm.weight"} <= keys


def test_hf_export_of_a_tied_model_has_no_lm_head_and_loads_back_tied(tmp_path):
    """Tied checkpoints in Hugging Face form carry the embedding only (as SmolLM's and Llama-3.2-1B's do); loading one with
    ``tie_word_embeddings`` gives the head the pretrained matrix instead of the random one an untied build keeps."""
    from safetensors import safe_open
    path = str(tmp_path / "export")
    for r in run_distributed(_export_roundtrip_worker, 2, 2, 1, path, True):
        assert "final_proj.weight" not in r and max(r.values()) == 0.0, r
    with safe_open(os.path.join(path, "model.safetensors"), framework="pytorch", device="cpu") as f:
        assert "lm_head.weight" not in set(f.keys()) and "model.embed_tokens.weight" in set(f.keys())


def test_hf_export_round_trip_tp2_pp2(tmp_path):
    path = str(tmp_path / "export")
    for r in run_distributed(_export_roundtrip_worker, 4, 2, 2, path):
        assert max(r.values()) == 0.0, r
    assert os.path.exists(os.path.join(path, "model.safetensors.index.json"))
    with open(os.path.join(path, "model.safetensors.index.json")) as f:
        wm = json.load(f)["weight_map"]
    assert wm["model.embed_tokens.weight"].startswith("model-00001-of-00002")
    assert wm["lm_head.weight"].startswith("model-00002-of-00002")


@pytest.mark.parametrize("variant", ["untied", "tied_llama3_rope"])
def test_logits_equal_hugging_face_llama_on_the_same_safetensors(tmp_path, variant):
    """A random Hugging Face ``LlamaForCausalLM`` is written as safetensors and read through the pretrained-weights path;
    both implementations must then compute the same logits (names, GQA head layout, half-split RoPE, RMSNorm, SwiGLU)."""
    transformers = pytest.importorskip("transformers")
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.checkpoint import init_model_with_dematerialized_weights, init_model_with_materialized_weights
    from picotron_b200.config import ModelConfig
    from picotron_b200.models.llama import Llama
    from picotron_b200.parallel.tied_embeddings import tie_word_embeddings
    tied = variant != "untied"
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 16} if tied else None
    shape = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                 vocab_size=96, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=32)
    torch.manual_seed(0)
    hf_cfg = transformers.LlamaConfig(**shape, tie_word_embeddings=tied, attention_bias=False, mlp_bias=False,
                                      rope_scaling=dict(scaling) if scaling else None)
    hf = transformers.LlamaForCausalLM(hf_cfg).float().eval()
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    pgm.reset()
    mc = ModelConfig(**shape, rope_scaling=scaling, tie_word_embeddings=tied)
    with init_model_with_dematerialized_weights():
        ours = Llama(mc)
    ours = init_model_with_materialized_weights(ours, mc, save_dir=str(tmp_path), load_pretrained=True)
    if tied:
        tie_word_embeddings(ours)
    ids = torch.randint(0, 96, (2, 32))
    with torch.no_grad():
        want = hf(input_ids=ids).logits
        got = ours(input_ids=ids)
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)


def test_greedy_decoding_picks_the_tokens_hugging_face_generate_picks(tmp_path):
    transformers = pytest.importorskip("transformers")
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.checkpoint import init_model_with_dematerialized_weights, init_model_with_materialized_weights
    from picotron_b200.config import ModelConfig
    from picotron_b200.generate import greedy_generate
    from picotron_b200.models.llama import Llama
    shape = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                 vocab_size=96, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=32)
    torch.manual_seed(1)
    hf = transformers.LlamaForCausalLM(transformers.LlamaConfig(**shape, tie_word_embeddings=False)).float().eval()
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    pgm.reset()
    mc = ModelConfig(**shape)
    with init_model_with_dematerialized_weights():
        ours = Llama(mc)
    ours = init_model_with_materialized_weights(ours, mc, save_dir=str(tmp_path), load_pretrained=True)
    prompt = torch.randint(1, 96, (3, 5))
    want = hf.generate(prompt, max_new_tokens=12, do_sample=False, pad_token_id=0, eos_token_id=None)
    got = greedy_generate(ours, prompt, max_new_tokens=12)
    assert torch.equal(got, want), (got, want)
    # an end-of-sequence id stops a row; the others go on
    eos = int(want[0, 7])
    stopped = greedy_generate(ours, prompt, max_new_tokens=12, eos_token_id=eos)
    assert torch.equal(stopped[0, :8], want[0, :8]) and bool((stopped[0, 8:] == 0).all())
