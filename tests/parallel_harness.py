"""Run one training step of a tiny model on a dp x pp x cp x tp Gloo grid and compare with the oracle.

Each rank returns its parameter shards and fp32 gradient buckets; the parent reassembles the full
model from the shards, recomputes loss and gradients with the plain-PyTorch oracle on the whole global
batch and checks every shard against the matching slice.
"""
import torch

import oracle
from picotron_b200.config import ModelConfig, load_config

import os

VOCAB, SEQ, MBS = 96, 16, 2


def kv_heads() -> int:
    """KV heads of the test model: 2 (grouped-query attention), or PICOTRON_TEST_KV_HEADS (4 for tensor parallelism over 4)."""
    return int(os.environ.get("PICOTRON_TEST_KV_HEADS", "2"))


GPU = {"on": False}          # set by the GPU tests: bf16 on CUDA/NCCL, wider model (head_dim 64)


def make_config(tp, cp, pp, dp, engine="1f1b", grad_acc=2, layers=4, split=None, cp_layout=None, tie=False, sp=False,
                zero1=False):
    gpu = GPU["on"]
    return load_config({
        "distributed": {"tp_size": tp, "cp_size": cp, "pp_size": pp, "dp_size": dp, "pp_engine": engine,
                        "use_cpu": not gpu, **({"pp_layer_split": split} if split else {}),
                        **({"cp_layout": cp_layout} if cp_layout else {}), **({"sequence_parallel": True} if sp else {})},
        "model": {"name": "tiny", "preset": "tiny-llama-test", "num_hidden_layers": layers, "num_attention_heads": 4,
                  "num_key_value_heads": kv_heads(), "hidden_size": 256 if gpu else 64, "intermediate_size": 512 if gpu else 128,
                  "vocab_size": VOCAB, "dtype": "bfloat16" if gpu else "float32", "init": "normal" if gpu else "reference",
                  "tie_word_embeddings": tie},
        "training": {"seed": 7, "learning_rate": 1e-3, "total_train_steps": 1, "seq_length": SEQ,
                     "micro_batch_size": MBS, "gradient_accumulation_steps": grad_acc, "num_samples": 64,
                     "master_weights": False, "zero1": zero1},
        "dataset": {"name": "synthetic"},
    })


def worker(rank, world_size, tp, cp, pp, dp, engine, grad_acc, layers, gpu=False, graph=False, split=None, cp_layout=None,
           tie=False, sp=False, clip=0.0, zero1=False):
    GPU["on"] = gpu
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.parallel.pipeline_parallel import train_step_pipeline_1f1b, train_step_pipeline_afab
    from picotron_b200.trainer import train_step
    from picotron_b200.utils import average_loss_across_dp_cp_ranks
    cfg = make_config(tp, cp, pp, dp, engine, grad_acc, layers, split, cp_layout, tie, sp, zero1)
    tr = _build(cfg)
    _add_host_jitter(rank)
    g = pgm.get()
    if pp > 1:
        fn = train_step_pipeline_afab if engine == "afab" else train_step_pipeline_1f1b
        loss = fn(tr.model, tr.data_loader, tr.tensor_shapes, tr.device, tr.dtype)
    elif graph:
        # the accumulation micro-batches replayed from the CUDA graph the trainer captured (collectives included)
        from picotron_b200.trainer import train_step_graphed
        assert tr.graphed is not None, "the trainer did not capture the micro-batch"
        loss = train_step_graphed(tr.model, tr.data_loader, tr.device, tr.graphed)
    else:
        loss = train_step(tr.model, tr.data_loader, tr.device)
    loss = average_loss_across_dp_cp_ranks(loss, tr.device)
    if tie:
        from picotron_b200.parallel.tied_embeddings import sync_tied_embedding_grads
        sync_tied_embedding_grads(tr.model)              # what Trainer.step does before the optimizer update
    from picotron_b200.parallel.tp_communications import sync_sequence_parallel_grads
    sync_sequence_parallel_grads(tr.model)               # as Trainer.step does; a no-op unless sequence parallelism is on
    grad_norm = 0.0
    if clip:
        from picotron_b200.optim import clip_grad_norm_
        grad_norm = float(clip_grad_norm_(tr.model, clip))
    raw = tr.model.module
    recv_buffers = 0
    if pp > 1:
        from picotron_b200.parallel.pp_communications import get_p2p
        recv_buffers = get_p2p().pool.allocated
    out = {"coords": (g.dp_rank, g.pp_rank, g.cp_rank, g.tp_rank), "loss": loss, "last": g.pp_is_last_stage,
           "recv_buffers": recv_buffers, "grad_norm": grad_norm, "n_layers": len(getattr(raw, "layer_distribution", range(layers))),
           "params": {n: p.detach().clone() for n, p in raw.named_parameters()},
           "grads": {n: p.main_grad.detach().clone() for n, p in raw.named_parameters()}}
    # a full optimizer step must also run
    tr.optimizer.step()
    tr.model.reset()
    if zero1:
        from picotron_b200.trainer import verify_replicas
        verify_replicas(tr.model)                        # the owners' broadcasts left every replica with the same weights
    return out


def _add_host_jitter(rank):
    """PICOTRON_TEST_JITTER_MS=n: every pipeline send and receive of this rank is preceded by a random host delay of up
    to n ms (seeded per rank), which shuffles the relative progress of the stages; a schedule whose correctness leans on a
    particular interleaving of the ranks then deadlocks or mixes up messages, a correct one gives the same numbers."""
    import os
    import random
    import time
    ms = float(os.environ.get("PICOTRON_TEST_JITTER_MS", "0"))
    if ms <= 0:
        return
    from picotron_b200.parallel.pp_communications import PipelineP2P
    rng = random.Random(1000 + rank)

    def delayed(fn):
        def wrapper(*a, **k):
            time.sleep(rng.random() * ms / 1e3)
            return fn(*a, **k)
        return wrapper
    for name in ("send", "wait_recv", "post_recv"):
        setattr(PipelineP2P, name, delayed(getattr(PipelineP2P, name)))


def _build(cfg):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.trainer import build_trainer
    d = cfg["distributed"]
    pgm.setup_process_group_manager(d["tp_size"], d["cp_size"], d["pp_size"], d["dp_size"])
    return build_trainer(cfg, init_dist=False)


_COL = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj", "embedding", "final_proj")
_ROW = ("out_proj", "down_proj")


def _shard_dim(name):
    if any(k in name for k in _COL):
        return 0
    if any(k in name for k in _ROW):
        return 1
    return None


def assemble_full_params(results, tp, pp):
    """The whole model's parameters from the shards of the dp = 0, cp = 0 ranks; also the results keyed by coordinates."""
    full = {}
    by = {r["coords"]: r for r in results}
    for p_ in range(pp):
        names = by[(0, p_, 0, 0)]["params"].keys()
        for n in names:
            dim = _shard_dim(n)
            shards = [by[(0, p_, 0, t)]["params"][n] for t in range(tp)]
            full[n] = shards[0] if dim is None else torch.cat(shards, dim=dim)
    return full, by


def eval_worker(rank, world_size, tp, cp, pp, dp, sp=False):
    """Build the trainer with held-out data, evaluate before any training; returns the loss and the parameter shards."""
    from picotron_b200 import process_group_manager as pgm
    cfg = make_config(tp, cp, pp, dp, "1f1b", 2, 4, sp=sp)
    cfg["training"].update(eval_every=1, eval_batches=3, eval_samples=16)
    tr = _build(cfg)
    g = pgm.get()
    before = [p.main_grad.clone() for p in tr.model.module.parameters()]
    loss = tr.evaluate()
    again = tr.evaluate()                                 # the same batches at every call
    untouched = all(torch.equal(p.main_grad, b) for p, b in zip(tr.model.module.parameters(), before))
    return {"coords": (g.dp_rank, g.pp_rank, g.cp_rank, g.tp_rank), "loss": loss, "again": again, "untouched": untouched,
            "last": g.pp_is_last_stage, "params": {n: p.detach().clone() for n, p in tr.model.module.named_parameters()}}


def check_eval(results, tp, cp, pp, dp):
    full, _ = assemble_full_params([{**r, "params": {k: v.float() for k, v in r["params"].items()}} for r in results], tp, pp)
    mc = ModelConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
                     num_key_value_heads=kv_heads(), vocab_size=VOCAB, max_position_embeddings=SEQ)
    from picotron_b200.data import SyntheticTokenDataset
    ds = SyntheticTokenDataset(16, SEQ + 1, VOCAB, seed=8)               # the trainer's seed + 1
    rows = [ds[(d_ + j * dp) % 16]["input_ids"] for d_ in range(dp) for j in range(3 * MBS)]
    ids = torch.stack(rows)
    ref_loss, _ = oracle.loss_and_grads(full, mc, ids[:, :-1], ids[:, 1:])
    for r in results:
        assert r["untouched"], f"evaluation changed a gradient buffer on {r['coords']}"
        if r["last"]:
            assert abs(r["loss"] - float(ref_loss)) < 2e-4 and r["again"] == r["loss"], (r["coords"], r["loss"], float(ref_loss))


def check(results, tp, cp, pp, dp, grad_acc, layers, gpu=False, tie=False, clip=0.0):
    GPU["on"] = gpu
    cfg = make_config(tp, cp, pp, dp, "1f1b", grad_acc, layers)
    mc = ModelConfig(hidden_size=256 if gpu else 64, intermediate_size=512 if gpu else 128, num_hidden_layers=layers,
                     num_attention_heads=4, num_key_value_heads=kv_heads(), vocab_size=VOCAB, max_position_embeddings=SEQ)
    results = [{**r, "params": {k: v.float() for k, v in r["params"].items()},
                "grads": {k: v.float() for k, v in r["grads"].items()}} for r in results]
    full, by = assemble_full_params(results, tp, pp)
    if tie:
        if pp == 1:                  # one parameter with two uses: the state dict of a rank lists it once
            assert "final_proj.weight" not in full
            full["final_proj.weight"] = full["embedding.weight"]
        else:                        # two copies, equal after the start-up broadcast
            torch.testing.assert_close(full["final_proj.weight"], full["embedding.weight"], rtol=0, atol=0)
    # ---- replicas hold identical parameters
    for r in results:
        d_, p_, c_, t_ = r["coords"]
        for n, v in r["params"].items():
            torch.testing.assert_close(v, by[(0, p_, 0, t_)]["params"][n], rtol=0, atol=0)
    # ---- the global batch, in the order the loader hands it out
    from picotron_b200.data import SyntheticTokenDataset
    ds = SyntheticTokenDataset(64, SEQ + 1, VOCAB, seed=7)
    rows = []
    for d_ in range(dp):
        for j in range(grad_acc * MBS):
            rows.append(ds[(d_ + j * dp) % 64]["input_ids"])
    ids = torch.stack(rows)
    ref_loss, ref_grads = oracle.loss_and_grads(full, mc, ids[:, :-1], ids[:, 1:])
    if tie:                          # the gradient of a shared matrix is the sum over its uses
        both = ref_grads["embedding.weight"] + ref_grads["final_proj.weight"]
        ref_grads["embedding.weight"] = ref_grads["final_proj.weight"] = both
    if clip:                         # every distinct parameter counts once in the global norm (a tied matrix is one parameter)
        distinct = {n: v for n, v in ref_grads.items() if not (tie and n == "final_proj.weight")}
        total = float(torch.sqrt(sum((v.double() ** 2).sum() for v in distinct.values())))
        assert total > clip, "choose a clip value below the gradient norm so that the test exercises the scaling"
        for r in results:
            assert abs(r["grad_norm"] - total) < 1e-4 * total, (r["coords"], r["grad_norm"], total)
        ref_grads = {n: v * (clip / (total + 1e-6)) for n, v in ref_grads.items()}
    # ---- loss (reported on last-stage ranks) and gradient shards
    for r in results:
        if r["last"]:
            assert abs(r["loss"] - float(ref_loss)) < (5e-2 if gpu else 2e-4), (r["coords"], r["loss"], float(ref_loss))
        _, _, _, t_ = r["coords"]
        for n, gshard in r["grads"].items():
            dim = _shard_dim(n)
            ref = ref_grads[n]
            if dim is not None and tp > 1:
                ref = torch.chunk(ref, tp, dim=dim)[t_]
            if gpu:
                err = float((gshard - ref).norm() / (ref.norm() + 1e-12))
                assert err < 6e-2, f"{n} @ {r['coords']}: relative gradient error {err:.4f}"
            else:
                torch.testing.assert_close(gshard, ref, rtol=2e-4, atol=2e-6,
                                           msg=lambda s, n=n, c=r["coords"]: f"{n} @ {c}: {s}")
