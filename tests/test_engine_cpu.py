"""Engine-level behaviour on CPU: naive data parallelism, config validation, checkpoint resume of a whole trainer."""
import copy
import os

import pytest
import torch

from dist_utils import run_distributed


def _tiny_cfg(tmp=None, **over):
    cfg = {"distributed": {"tp_size": 1, "cp_size": 1, "pp_size": 1, "dp_size": 1, "use_cpu": True},
           "model": {"name": "tiny-test", "hidden_size": 32, "intermediate_size": 64, "vocab_size": 64,
                     "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2},
           "training": {"seed": 3, "learning_rate": 1e-2, "seq_length": 16, "micro_batch_size": 2,
                        "gradient_accumulation_steps": 2, "total_train_steps": 10, "num_samples": 64},
           "dataset": {"name": "synthetic"}, "checkpoint": {"save_dir": tmp or "./ckpt", "save_frequency": 1000, "load_path": ""}}
    for k, v in over.items():
        cfg[k].update(v)
    return cfg


# --------------------------------------------------------------------------------------------- naive data parallelism
def _naive_dp_worker(rank, world):
    import torch.distributed as dist
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.config import ModelConfig
    from picotron_b200.models.llama import Llama
    from picotron_b200.parallel.data_parallel import DataParallelNaive
    pgm.setup_process_group_manager(tp_size=1, cp_size=1, pp_size=1, dp_size=world)
    cfg = ModelConfig(hidden_size=32, intermediate_size=64, vocab_size=64, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=16)
    torch.manual_seed(0)
    base = Llama(cfg)
    local = copy.deepcopy(base)
    ddp = DataParallelNaive(copy.deepcopy(base))
    g = torch.Generator().manual_seed(100 + rank)                        # a different batch per rank
    ids = torch.randint(0, 64, (2, 16), generator=g)
    tgt = torch.randint(0, 64, (2, 16), generator=g)
    local(input_ids=ids, target_ids=tgt).backward()
    ddp(input_ids=ids, target_ids=tgt).backward()
    worst = 0.0
    for (n, p), (_, q) in zip(local.named_parameters(), ddp.module.named_parameters()):
        mean = p.grad.clone()
        dist.all_reduce(mean)
        mean /= world
        worst = max(worst, float((q.grad - mean).abs().max()))
    # no_sync(): gradients stay local
    ddp.zero_grad()
    with ddp.no_sync():
        ddp(input_ids=ids, target_ids=tgt).backward()
    local_only = max(float((q.grad - p.grad).abs().max())
                     for (_, p), (_, q) in zip(local.named_parameters(), ddp.module.named_parameters()))
    return {"sync_err": worst, "no_sync_err": local_only}


def test_naive_data_parallel_averages_gradients_and_no_sync_keeps_them_local():
    for r in run_distributed(_naive_dp_worker, 2):
        assert r["sync_err"] < 1e-6 and r["no_sync_err"] < 1e-6, r


# --------------------------------------------------------------------------------------------- config validation
def test_config_validation_rejects_bad_grids_and_engines():
    from picotron_b200.config import load_config, validate_config, world_size_of
    cfg = load_config(_tiny_cfg())
    validate_config(cfg)
    assert world_size_of(cfg) == 1
    with pytest.raises(AssertionError):                                  # load_config validates what it reads
        load_config(_tiny_cfg(distributed={"pp_engine": "interleaved"}))
    with pytest.raises(AssertionError):
        load_config(_tiny_cfg(distributed={"cp_size": 3}))               # 16 tokens are not divisible by cp = 3
    with pytest.raises(AssertionError):
        load_config(_tiny_cfg(distributed={"comm": "mpi"}))
    cfg["distributed"]["dp_size"] = 0
    with pytest.raises(AssertionError):
        validate_config(cfg)


# --------------------------------------------------------------------------------------------- trainer resume
def test_trainer_resumes_from_the_latest_checkpoint_with_the_same_losses(tmp_path):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.trainer import build_trainer
    save_dir = str(tmp_path / "ckpt")
    pgm.reset()
    a = build_trainer(_tiny_cfg(save_dir), init_dist=False)
    losses = [a.step() for _ in range(4)]                                # uninterrupted run
    pgm.reset()
    b = build_trainer(_tiny_cfg(save_dir), init_dist=False)
    first = [b.step() for _ in range(2)]
    b.save(os.path.join(save_dir, str(b.step_idx)))
    pgm.reset()
    c = build_trainer(_tiny_cfg(save_dir, checkpoint={"load_path": "latest"}), init_dist=False)
    assert c.step_idx == 2 and c.trained_tokens == b.trained_tokens
    resumed = [c.step() for _ in range(2)]
    assert first == pytest.approx(losses[:2], rel=1e-6)
    assert resumed == pytest.approx(losses[2:], rel=1e-5)                # weights, Adam state and data position restored


def test_training_on_a_local_text_file_with_the_byte_tokenizer_reduces_the_loss(tmp_path):
    """No network, no synthetic data: a text file, the built-in byte tokenizer and a tiny model; the loss must fall."""
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.trainer import build_trainer
    path = tmp_path / "corpus.txt"
    path.write_text("\n".join("abcabcabc abcabcabc abcabcabc" for _ in range(64)))
    cfg = _tiny_cfg(str(tmp_path / "ckpt"), model={"vocab_size": 256}, dataset={"name": str(path), "tokenizer": "bytes"},
                    training={"num_samples": None, "learning_rate": 3e-2})
    pgm.reset()
    tr = build_trainer(cfg, init_dist=False)
    losses = [tr.step() for _ in range(12)]
    assert losses[0] > 3.0 and losses[-1] < 0.5 * losses[0], losses


# --------------------------------------------------------------------------------------------- tied embedding / LM head
def test_tied_trainer_shares_one_parameter_trains_and_resumes(tmp_path):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.trainer import build_trainer
    save_dir = str(tmp_path / "ckpt")
    tie = {"tie_word_embeddings": True}
    pgm.reset()
    a = build_trainer(_tiny_cfg(save_dir, model=tie), init_dist=False)
    raw = a.model.module
    assert raw.final_proj.weight is raw.embedding.weight
    assert "final_proj.weight" not in dict(raw.named_parameters())      # one parameter: one Adam state, one bucket slice
    # the parameter count that feeds the MFU formula still counts the matrix once per use
    pgm.reset()
    untied = build_trainer(_tiny_cfg(save_dir), init_dist=False)
    assert a.num_params == untied.num_params
    pgm.reset()
    a = build_trainer(_tiny_cfg(save_dir, model=tie), init_dist=False)
    losses = [a.step() for _ in range(4)]
    assert losses[-1] < losses[0]
    pgm.reset()
    b = build_trainer(_tiny_cfg(save_dir, model=tie), init_dist=False)
    [b.step() for _ in range(2)]
    b.save(os.path.join(save_dir, str(b.step_idx)))
    pgm.reset()
    c = build_trainer(_tiny_cfg(save_dir, model=tie, checkpoint={"load_path": "latest"}), init_dist=False)
    assert c.model.module.final_proj.weight is c.model.module.embedding.weight
    resumed = [c.step() for _ in range(2)]
    assert resumed == pytest.approx(losses[2:], rel=1e-5)
    # evaluation under no_grad adds nothing to the shared bucket slice and leaves the use counter where it was
    w = c.model.module.embedding.weight
    before = w.main_grad.clone()
    batch = next(c.data_loader)
    with torch.no_grad():
        c.model(input_ids=batch["input_ids"], target_ids=batch["target_ids"])
    assert torch.equal(w.main_grad, before) and getattr(w, "_grad_seen", 0) == 0


def _tied_pp_worker(rank, world, steps):
    import torch.distributed as dist
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.trainer import build_trainer
    cfg = _tiny_cfg(distributed={"pp_size": 2, "dp_size": world // 2}, model={"tie_word_embeddings": True})
    pgm.setup_process_group_manager(tp_size=1, cp_size=1, pp_size=2, dp_size=world // 2)
    tr = build_trainer(cfg, init_dist=False)
    g = pgm.get()
    losses = [tr.step() for _ in range(steps)]
    raw = tr.model.module
    w = raw.embedding.weight if g.pp_is_first_stage else raw.final_proj.weight
    return {"coords": (g.dp_rank, g.pp_rank), "w": w.detach().clone(), "losses": losses, "last": g.pp_is_last_stage}


def test_tied_copies_on_the_first_and_last_stage_stay_bitwise_equal_over_optimizer_steps():
    res = run_distributed(_tied_pp_worker, 4, 3)
    by = {r["coords"]: r for r in res}
    for d in range(2):
        assert torch.equal(by[(d, 0)]["w"], by[(d, 1)]["w"])             # embedding (stage 0) == head (stage 1)
    assert torch.equal(by[(0, 0)]["w"], by[(1, 0)]["w"])                 # and the data-parallel replicas agree
    last = [r for r in res if r["last"]][0]["losses"]
    assert last[-1] < last[0]


# --------------------------------------------------------------------------------------------- sequence parallelism
def _sp_trainer_worker(rank, world, sp, steps):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.trainer import build_trainer
    cfg = _tiny_cfg(distributed={"tp_size": 2, "pp_size": 2, "sequence_parallel": sp})
    pgm.setup_process_group_manager(tp_size=2, cp_size=1, pp_size=2, dp_size=1)
    tr = build_trainer(cfg, init_dist=False)
    assert tr.tensor_shapes == (2, 8 if sp else 16, 32)                  # pipeline messages carry 1/tp of the tokens
    losses = [tr.step() for _ in range(steps)]
    norm = tr.model.module.decoder_layers[str(tr.model.module.layer_distribution[0])].input_layernorm.weight
    return {"losses": losses, "last": pgm.get().pp_is_last_stage, "norm": norm.detach().clone(),
            "coords": (pgm.get().pp_rank, pgm.get().tp_rank)}


def test_sequence_parallel_training_follows_the_same_trajectory_as_plain_tensor_parallelism():
    plain = run_distributed(_sp_trainer_worker, 4, False, 4)
    sp = run_distributed(_sp_trainer_worker, 4, True, 4)
    a = [r for r in plain if r["last"]][0]["losses"]
    b = [r for r in sp if r["last"]][0]["losses"]
    assert b == pytest.approx(a, rel=1e-4) and b[-1] < b[0]
    by = {r["coords"]: r for r in sp}
    for stage in range(2):       # the norm weights stay replicated over the TP pair: their gradients were summed before Adam
        assert torch.equal(by[(stage, 0)]["norm"], by[(stage, 1)]["norm"])
        torch.testing.assert_close(by[(stage, 0)]["norm"], {r["coords"]: r for r in plain}[(stage, 0)]["norm"],
                                   rtol=1e-4, atol=1e-5)


# --------------------------------------------------------------------------------------------- lr schedule, clipping
def test_lr_schedule_curve_and_trainer_applies_it_with_clipping():
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.optim import lr_at
    from picotron_b200.trainer import build_trainer
    assert lr_at(7, 1e-3, None) == 1e-3
    sched = {"warmup_steps": 4, "decay": "cosine", "min_lr_ratio": 0.1, "total_steps": 12}
    curve = [lr_at(s, 1.0, sched) for s in range(14)]
    assert curve[:4] == pytest.approx([0.25, 0.5, 0.75, 1.0]) and curve[4] == pytest.approx(1.0)
    assert all(a >= b for a, b in zip(curve[4:], curve[5:])) and curve[12] == pytest.approx(0.1) and curve[13] == pytest.approx(0.1)
    assert lr_at(8, 1.0, {**sched, "decay": "linear"}) == pytest.approx(0.1 + 0.9 * 0.5)
    pgm.reset()
    tr = build_trainer(_tiny_cfg(training={"lr_schedule": {"warmup_steps": 2, "decay": "linear", "total_steps": 6},
                                           "max_grad_norm": 0.01}), init_dist=False)
    seen = []
    for _ in range(4):
        before = [p.detach().clone() for p in tr.model.parameters()]
        tr.step()
        seen.append(tr.optimizer.param_groups[0]["lr"])
        assert float(tr.last_grad_norm) > 0.01                       # the tiny model's gradients are far above the limit
        moved = max(float((p.detach() - b).abs().max()) for p, b in zip(tr.model.parameters(), before))
        assert 0 < moved <= 1.5 * seen[-1]                           # an Adam step moves a weight by about lr at most
    assert seen == pytest.approx([0.005, 0.01, 0.01, 0.0075])      # two warm-up steps, then linear to 0 at step 6
    with pytest.raises(AssertionError):
        from picotron_b200.config import load_config
        load_config(_tiny_cfg(training={"lr_schedule": {"decay": "exponential"}}))
    # AdamW hyper-parameters: torch's defaults unless the config names others
    assert tr.optimizer.defaults["betas"] == (0.9, 0.999) and tr.optimizer.defaults["weight_decay"] == 0.01
    pgm.reset()
    other = build_trainer(_tiny_cfg(training={"weight_decay": 0.1, "adam_betas": [0.9, 0.95], "adam_eps": 1e-6}), init_dist=False)
    group = other.optimizer.param_groups[0]
    assert group["weight_decay"] == 0.1 and tuple(group["betas"]) == (0.9, 0.95) and group["eps"] == 1e-6
    other.step()


# --------------------------------------------------------------------------------------------- asynchronous checkpoint
def test_asynchronous_save_snapshots_the_state_of_its_step(tmp_path, monkeypatch):
    """The background writer is held back while training goes on and changes every weight; the file must still hold
    the state of the step that was saved, and a writer error must surface in wait()."""
    import threading
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.checkpoint import CheckpointManager
    from picotron_b200.trainer import build_trainer
    save_dir = str(tmp_path / "ckpt")
    pgm.reset()
    a = build_trainer(_tiny_cfg(save_dir), init_dist=False)
    losses = [a.step() for _ in range(4)]
    gate = threading.Event()
    real_write = CheckpointManager._write
    monkeypatch.setattr(CheckpointManager, "_write", staticmethod(lambda ckpt, path: (gate.wait(30), real_write(ckpt, path))))
    pgm.reset()
    b = build_trainer(_tiny_cfg(save_dir, checkpoint={"async_save": True}), init_dist=False)
    [b.step() for _ in range(2)]
    b.save(os.path.join(save_dir, "2"))
    assert not os.path.exists(os.path.join(save_dir, "2", "weights_tp_rank_world_size=0_1_pp_rank_world_size=0_1.pth.done"))
    b.step()                                                             # training continues while the write is pending
    gate.set()
    b.checkpoint_manager.wait()
    pgm.reset()
    c = build_trainer(_tiny_cfg(save_dir, checkpoint={"load_path": "latest"}), init_dist=False)
    assert c.step_idx == 2
    assert [c.step() for _ in range(2)] == pytest.approx(losses[2:], rel=1e-5)
    # a failing writer is reported, not swallowed
    monkeypatch.setattr(CheckpointManager, "_write", staticmethod(lambda ckpt, path: (_ for _ in ()).throw(OSError("disk full"))))
    b.save(os.path.join(save_dir, "3"))
    with pytest.raises(RuntimeError, match="disk full"):
        b.checkpoint_manager.wait()


# --------------------------------------------------------------------------------------------- sharded optimizer (ZeRO-1)
def _zero1_worker(rank, world, zero1, tp, pp, save_dir, steps, load):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.trainer import build_trainer, verify_replicas
    dp = world // (tp * pp)
    cfg = _tiny_cfg(save_dir, distributed={"tp_size": tp, "pp_size": pp, "dp_size": dp},
                    training={"zero1": zero1, "max_grad_norm": 0.5}, checkpoint={"load_path": "latest" if load else ""})
    pgm.setup_process_group_manager(tp_size=tp, cp_size=1, pp_size=pp, dp_size=dp)
    tr = build_trainer(cfg, init_dist=False)
    losses = [tr.step() for _ in range(steps)]
    verify_replicas(tr.model)                                            # the broadcast kept the replicas bitwise equal
    if save_dir and not load:
        tr.save(os.path.join(save_dir, str(tr.step_idx)))
    g = pgm.get()
    raw = tr.model.module
    n_state = sum(1 for p in raw.parameters() if len(tr.optimizer.state[p]))
    return {"losses": losses, "last": g.pp_is_last_stage, "coords": (g.dp_rank, g.pp_rank, g.tp_rank), "states": n_state,
            "n_params": sum(1 for _ in raw.parameters()), "w": next(raw.parameters()).detach().clone()}


@pytest.mark.parametrize("tp,pp,world", [(1, 1, 2), (2, 2, 8)], ids=["dp2", "dp2_tp2_pp2"])
def test_optimizer_sharded_over_the_replicas_trains_exactly_like_the_unsharded_one(tmp_path, tp, pp, world):
    plain = run_distributed(_zero1_worker, world, False, tp, pp, "", 3, False)
    shard = run_distributed(_zero1_worker, world, True, tp, pp, str(tmp_path / "z"), 3, False)
    a = [r for r in plain if r["last"]][0]
    b = [r for r in shard if r["last"]][0]
    assert b["losses"] == a["losses"]                                    # the same update, computed by one owner each
    by_p, by_s = {r["coords"]: r for r in plain}, {r["coords"]: r for r in shard}
    for c in by_p:
        assert torch.equal(by_p[c]["w"], by_s[c]["w"])
    for r in shard:                                                      # each replica keeps state for its share only
        assert 0 < r["states"] < r["n_params"], r
    pair = [r for r in shard if r["coords"][1:] == (0, 0)]
    assert sum(r["states"] for r in pair) == pair[0]["n_params"]
    if world > 2:
        return
    # the checkpoint is an ordinary one: an UNSHARDED run resumes from it, and a sharded one too, on the same trajectory
    longer = [r for r in run_distributed(_zero1_worker, world, False, tp, pp, "", 5, False) if r["last"]][0]["losses"]
    for zero1 in (False, True):
        res = [r for r in run_distributed(_zero1_worker, world, zero1, tp, pp, str(tmp_path / "z"), 2, True) if r["last"]][0]
        assert res["losses"] == pytest.approx(longer[3:], rel=1e-6), (zero1, res["losses"], longer)


def test_validation_loss_on_a_second_text_file_falls_while_training_on_the_first(tmp_path):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.trainer import build_trainer
    train_txt, val_txt = tmp_path / "train.txt", tmp_path / "val.txt"
    train_txt.write_text("\n".join("abcabcabc abcabcabc abcabcabc" for _ in range(64)))
    val_txt.write_text("\n".join("abcabc abcabcabcabc abcabc" for _ in range(24)))     # same language, other text
    cfg = _tiny_cfg(str(tmp_path / "ckpt"), model={"vocab_size": 256},
                    dataset={"name": str(train_txt), "tokenizer": "bytes", "eval_name": str(val_txt)},
                    training={"num_samples": None, "learning_rate": 3e-2, "eval_every": 4, "eval_batches": 2})
    pgm.reset()
    tr = build_trainer(cfg, init_dist=False)
    before = tr.evaluate()
    position = tr.data_loader.state_dict()
    assert tr.evaluate() == before and tr.data_loader.state_dict() == position      # evaluation leaves the training stream alone
    for _ in range(12):
        tr.step()
    after = tr.evaluate()
    assert before > 3.0 and after < 0.6 * before, (before, after)
