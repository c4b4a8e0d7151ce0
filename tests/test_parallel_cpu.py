"""Every parallel strategy and both pipeline engines on CPU/Gloo against the single-process oracle."""
import pytest

from dist_utils import run_distributed
import parallel_harness as H


def _run(tp=1, cp=1, pp=1, dp=1, engine="1f1b", grad_acc=2, layers=4, tie=False, sp=False, clip=0.0):
    world = tp * cp * pp * dp
    res = run_distributed(H.worker, world, tp, cp, pp, dp, engine, grad_acc, layers, False, False, None, None, tie, sp,
                          clip)
    H.check(res, tp, cp, pp, dp, grad_acc, layers, tie=tie, clip=clip)
    return res


def test_single_rank():
    _run()


def test_tensor_parallel_2():
    _run(tp=2)


def test_data_parallel_2():
    _run(dp=2)


def test_context_parallel_2():
    _run(cp=2)


@pytest.mark.parametrize("engine", ["afab", "1f1b"])
def test_pipeline_parallel_2(engine):
    _run(pp=2, engine=engine, grad_acc=3)


def test_pipeline_1f1b_uneven_layers_3_stages():
    _run(pp=3, engine="1f1b", grad_acc=4, layers=4)


def test_pipeline_1f1b_receive_buffers_come_from_a_bounded_pool():
    """8 micro-batches through 2 stages: 16 messages per boundary, but the receive buffers are recycled. A stage holds at
    most (warm-up + 1) activations for pending backward passes plus the one posted ahead, and 2 gradient buffers."""
    pp, n_mb = 2, 8
    for r in _run(pp=pp, engine="1f1b", grad_acc=n_mb):
        stage = r["coords"][1]
        in_flight = (pp - stage - 1) + 1
        bound = (in_flight + 1 if stage > 0 else 0) + (2 if stage < pp - 1 else 0)
        assert 0 < r["recv_buffers"] <= bound, (stage, r["recv_buffers"], bound)


def test_cp2_dp2():
    _run(cp=2, dp=2)


def test_4d_grid_dp2_tp2_pp2_1f1b():
    _run(tp=2, pp=2, dp=2, engine="1f1b", grad_acc=2)


def test_tp2_cp2_pp2_1f1b():
    _run(tp=2, cp=2, pp=2, engine="1f1b", grad_acc=2)


def test_pipeline_with_an_uneven_explicit_layer_split():
    """3 + 1 layers over two stages (what "balanced" does for a model with a heavy LM head): same loss and gradients."""
    res = run_distributed(H.worker, 2, 1, 1, 2, 1, "1f1b", 3, 4, False, False, [3, 1])
    H.check(res, 1, 1, 2, 1, 3, 4)
    assert sorted(r["n_layers"] for r in res) == [1, 3]


def test_balanced_layer_split_gives_the_last_stage_fewer_layers_when_the_head_is_heavy():
    from picotron_b200.config import MODEL_PRESETS, ModelConfig
    from picotron_b200.parallel.pipeline_parallel import balanced_layer_split
    big_vocab = ModelConfig(**{**MODEL_PRESETS["meta-llama/Meta-Llama-3-8B"], "max_position_embeddings": 8192})
    assert balanced_layer_split(big_vocab, 2) == [17, 15]
    per = balanced_layer_split(big_vocab, 4)
    assert sum(per) == 32 and per[-1] < per[0] and min(per) >= 1
    small_vocab = ModelConfig(**{**MODEL_PRESETS["meta-llama/Llama-2-7b-hf"], "max_position_embeddings": 1024})
    assert balanced_layer_split(small_vocab, 2) == [16, 16]


@pytest.mark.parametrize("cp,dp", [(2, 1), (4, 1), (2, 2)])
def test_context_parallel_zigzag_layout(cp, dp):
    """Rank r holds half-chunks r and 2 cp - 1 - r: same loss and gradients as the single-process oracle."""
    res = run_distributed(H.worker, cp * dp, 1, cp, 1, dp, "1f1b", 2, 2, False, False, None, "zigzag")
    H.check(res, 1, cp, 1, dp, 2, 2)


def test_zigzag_positions_cover_the_sequence_once_and_balance_the_causal_work():
    import torch
    from picotron_b200.parallel.context_parallel import local_token_positions, _zigzag_pairs
    cp, S = 4, 64
    allpos = torch.cat([local_token_positions(S, r, cp, "zigzag") for r in range(cp)])
    assert sorted(allpos.tolist()) == list(range(S))
    assert local_token_positions(S, 1, cp, "zigzag").tolist() == list(range(8, 16)) + list(range(48, 56))
    assert local_token_positions(S, 1, cp, "contiguous").tolist() == list(range(16, 32))
    work = [sum(0.5 if diag else 1.0 for src in range(cp) for (_, _, diag) in _zigzag_pairs(r, src)) for r in range(cp)]
    assert len(set(work)) == 1, work                      # every rank computes the same number of half-blocks


def test_pipeline_1f1b_with_receives_posted_ahead(monkeypatch):
    """The optional mode in which the receive of micro-batch k + 1 is posted before micro-batch k computes."""
    monkeypatch.setenv("PICOTRON_PP_POST_AHEAD", "1")          # read by the spawned ranks when they import the package
    _run(pp=2, engine="1f1b", grad_acc=4)
    _run(pp=2, engine="afab", grad_acc=3)


@pytest.mark.parametrize("ahead", ["0", "1"], ids=["recv_when_needed", "recv_posted_ahead"])
def test_pipeline_schedules_do_not_depend_on_the_relative_speed_of_the_stages(monkeypatch, ahead):
    """Random host delays (up to 15 ms, different on every rank) before every pipeline send and receive: 3 uneven stages,
    6 micro-batches, both engines, both receive-posting modes; loss and gradients must still equal the oracle."""
    monkeypatch.setenv("PICOTRON_TEST_JITTER_MS", "15")
    monkeypatch.setenv("PICOTRON_PP_POST_AHEAD", ahead)
    _run(pp=3, engine="1f1b", grad_acc=6, layers=4)
    _run(pp=3, engine="afab", grad_acc=6, layers=4)


@pytest.mark.parametrize("grid", [dict(), dict(tp=2), dict(dp=2), dict(pp=2), dict(pp=3, grad_acc=3),
                                  dict(tp=2, pp=2, dp=2)], ids=["single", "tp2", "dp2", "pp2", "pp3", "dp2_tp2_pp2"])
def test_tied_embedding_and_lm_head(grid):
    """``model.tie_word_embeddings``: the shared matrix gets the sum of the embedding's and the head's gradient, on one
    rank (one parameter, two uses) as over the first and last pipeline stage (two copies, gradients added)."""
    _run(tie=True, **grid)


@pytest.mark.parametrize("grid", [dict(tp=2), dict(tp=2, dp=2), dict(tp=2, pp=2), dict(tp=2, pp=2, engine="afab"),
                                  dict(tp=2, cp=2), dict(tp=2, pp=2, dp=2), dict(tp=2, tie=True), dict(tp=2, pp=2, tie=True)],
                         ids=["tp2", "tp2_dp2", "tp2_pp2", "tp2_pp2_afab", "tp2_cp2", "dp2_tp2_pp2", "tp2_tied",
                              "tp2_pp2_tied"])
def test_sequence_parallel(grid):
    """``distributed.sequence_parallel``: each TP rank normalises and carries 1/tp of the tokens, the GEMMs see all of them
    (all-gather in, reduce-scatter out), pipeline messages shrink by tp; loss and every gradient shard equal the oracle,
    the norm-weight gradients after their sum over the TP group."""
    _run(sp=True, **grid)


@pytest.mark.parametrize("grid", [dict(), dict(tp=2, pp=2, dp=2), dict(tp=2, pp=2, tie=True), dict(tp=2, cp=2, sp=True)],
                         ids=["single", "dp2_tp2_pp2", "tp2_pp2_tied", "tp2_cp2_sp"])
def test_global_gradient_norm_clipping(grid):
    """``training.max_grad_norm``: the norm is taken over every distinct parameter of the model, whatever grid its shards
    live on (TP shards summed, replicated norm weights and the second copy of a tied matrix counted once), and every
    shard is scaled by the same factor."""
    _run(clip=0.05, **grid)


@pytest.mark.parametrize("grid", [dict(tp=1, cp=1, pp=1, dp=1), dict(tp=2, cp=1, pp=2, dp=2), dict(tp=1, cp=2, pp=1, dp=2),
                                  dict(tp=2, cp=1, pp=3, dp=1, sp=True)], ids=["single", "dp2_tp2_pp2", "cp2_dp2", "tp2_pp3_sp"])
def test_evaluation_loss_on_held_out_batches(grid):
    """``Trainer.evaluate``: forward passes only (through the pipeline stages too), the mean over the data-parallel ranks'
    batches equals the oracle's loss on the same rows, no gradient buffer changes, a second call gives the same number."""
    sp = grid.pop("sp", False)
    world = grid["tp"] * grid["cp"] * grid["pp"] * grid["dp"]
    res = run_distributed(H.eval_worker, world, grid["tp"], grid["cp"], grid["pp"], grid["dp"], sp)
    H.check_eval(res, grid["tp"], grid["cp"], grid["pp"], grid["dp"])


def test_every_option_at_once_on_eight_ranks():
    """tp2 x cp2 x pp2 with the zigzag sequence layout, sequence parallelism, a tied head (two pipeline copies), gradient
    clipping and the optimizer sharded over the context-parallel pair: the gradients still equal the oracle's."""
    res = run_distributed(H.worker, 8, 2, 2, 2, 1, "1f1b", 2, 4, False, False, None, "zigzag", True, True, 0.05, True)
    H.check(res, 2, 2, 2, 1, 2, 4, tie=True, clip=0.05)


def test_tensor_parallel_over_four_ranks_plain_and_sequence_parallel(monkeypatch):
    monkeypatch.setenv("PICOTRON_TEST_KV_HEADS", "4")          # 4 query and 4 KV heads: one of each per rank
    _run(tp=4)
    _run(tp=4, sp=True)
    _run(tp=4, pp=2, sp=True, tie=True)


@pytest.mark.parametrize("engine", ["afab", "1f1b"])
def test_four_pipeline_stages_with_fewer_and_more_micro_batches_than_stages(engine):
    _run(pp=4, engine=engine, grad_acc=2, layers=4)           # fewer micro-batches than stages: warm-up is cut short
    _run(pp=4, engine=engine, grad_acc=7, layers=4)


def test_context_parallel_over_four_ranks_with_data_parallel_pairs():
    _run(cp=4, dp=2)
