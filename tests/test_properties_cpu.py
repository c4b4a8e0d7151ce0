"""Property tests (hypothesis) of the pure functions the engine leans on: grid arithmetic, layer splits, sequence layouts,
the learning-rate curve, the text windowing, the memory plan."""
import numpy as np
import pytest
import torch

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings, strategies as st  # noqa: E402

sizes = st.sampled_from([1, 2, 3, 4, 8])


@settings(max_examples=60, deadline=None, derandomize=True)
@given(tp=sizes, cp=sizes, pp=sizes, dp=sizes)
def test_grid_coordinates_are_a_bijection_and_every_group_family_partitions_the_ranks(tp, cp, pp, dp):
    from picotron_b200.process_group_manager import GridTopology
    t = GridTopology(tp_size=tp, cp_size=cp, pp_size=pp, dp_size=dp)
    world = t.world_size
    assert sorted(t.rank(*t.coords(r)) for r in range(world)) == list(range(world))
    for groups, size in ((t.tp_groups(), tp), (t.cp_groups(), cp), (t.pp_groups(), pp), (t.dp_groups(), dp),
                         (t.cp_dp_groups(), cp * dp), (t.pp_dp_groups(), pp * dp)):
        assert all(len(g) == size for g in groups)
        assert sorted(r for g in groups for r in g) == list(range(world))          # every rank in exactly one group
    for g in t.tp_groups():                                                        # a TP group differs in the tp coordinate only
        assert len({t.coords(r)[:3] for r in g}) == 1
    ends = t.pp_end_groups()
    assert all(t.coords(a)[1] == 0 and t.coords(b)[1] == pp - 1 for a, b in ends) and len(ends) == tp * cp * dp


@settings(max_examples=80, deadline=None, derandomize=True)
@given(layers=st.integers(1, 80), pp=st.integers(1, 8), hidden=st.sampled_from([512, 2048, 4096]),
       vocab=st.sampled_from([32000, 49152, 128256]), seq=st.sampled_from([1024, 8192]))
def test_balanced_layer_split_keeps_every_layer_once_and_never_beats_the_even_split_on_the_slowest_stage(layers, pp, hidden, vocab, seq):
    from picotron_b200.config import ModelConfig
    from picotron_b200.parallel.pipeline_parallel import balanced_layer_split
    if pp > layers:
        return
    mc = ModelConfig(hidden_size=hidden, intermediate_size=4 * hidden, num_hidden_layers=layers, num_attention_heads=hidden // 64,
                     num_key_value_heads=hidden // 64, vocab_size=vocab, max_position_embeddings=seq)
    split = balanced_layer_split(mc, pp)
    assert len(split) == pp and sum(split) == layers and min(split) >= 1
    kv = hidden
    layer = 2 * hidden * hidden + 2 * hidden * kv + 3 * hidden * 4 * hidden + 2 * hidden * seq
    head = vocab * hidden
    cost = lambda per: max(k * layer + (head if s == pp - 1 else 0) for s, k in enumerate(per))
    even = [layers // pp + (1 if i < layers % pp else 0) for i in range(pp)]
    assert cost(split) <= cost(even)


@settings(max_examples=60, deadline=None, derandomize=True)
@given(cp=st.sampled_from([1, 2, 4, 8]), mult=st.integers(1, 6), layout=st.sampled_from(["contiguous", "zigzag"]))
def test_sequence_layouts_give_every_token_to_exactly_one_rank(cp, mult, layout):
    from picotron_b200.parallel.context_parallel import local_token_positions
    seq = 2 * cp * mult
    parts = [local_token_positions(seq, r, cp, layout) for r in range(cp)]
    assert all(len(p) == seq // cp for p in parts)
    assert sorted(torch.cat(parts).tolist()) == list(range(seq))
    if layout == "zigzag" and cp > 1:                       # causal work (tokens a position attends to) is the same on every rank
        work = [int((p + 1).sum()) for p in parts]
        assert len(set(work)) == 1


@settings(max_examples=80, deadline=None, derandomize=True)
@given(warm=st.integers(0, 20), total=st.integers(1, 200), ratio=st.floats(0.0, 1.0), decay=st.sampled_from(["constant", "linear", "cosine"]),
       step=st.integers(0, 400))
def test_learning_rate_stays_between_its_floor_and_peak_and_never_rises_after_the_warm_up(warm, total, ratio, decay, step):
    from picotron_b200.optim import lr_at
    sched = {"warmup_steps": warm, "decay": decay, "min_lr_ratio": ratio, "total_steps": total}
    lr, nxt = lr_at(step, 1.0, sched), lr_at(step + 1, 1.0, sched)
    assert 0.0 <= lr <= 1.0 + 1e-12                         # a floor of 0 is reached at the end of a linear / cosine decay
    if step >= warm:
        assert nxt <= lr + 1e-12
        if decay != "constant":
            assert lr >= ratio - 1e-12
    else:
        assert lr > 0.0 and nxt >= lr


@settings(max_examples=60, deadline=None, derandomize=True)
@given(n=st.integers(0, 400), seq=st.integers(1, 64))
def test_text_windows_overlap_by_one_token_and_drop_only_an_incomplete_tail(n, seq):
    from picotron_b200.data import group_into_windows
    ids = np.arange(n)
    wins = group_into_windows(ids, seq)
    assert all(len(w) == seq + 1 for w in wins)
    for a, b in zip(wins, wins[1:]):
        assert a[-1] == b[0]                                # the label of a window's last position opens the next window
    assert len(wins) == (max(n - 1, 0) // seq if n >= seq + 1 else 0)


@settings(max_examples=40, deadline=None, derandomize=True)
@given(tp=st.sampled_from([1, 2, 4]), pp=st.sampled_from([1, 2, 4]), cp=st.sampled_from([1, 2]), mbs=st.integers(1, 4),
       sp=st.booleans(), zero1=st.booleans(), dp=st.sampled_from([1, 2, 4]))
def test_memory_plan_is_monotone_in_the_knobs_that_should_shrink_it(tp, pp, cp, mbs, sp, zero1, dp):
    from picotron_b200.config import preset_model_config
    from picotron_b200.utils.memory import plan_memory
    mc = preset_model_config("meta-llama/Llama-2-7b-hf")
    kw = dict(tp=tp, pp=pp, cp=cp, dp=dp, micro_batch_size=mbs, seq_length=4096, grad_acc_steps=8)
    base = plan_memory(mc, **kw)
    assert plan_memory(mc, **{**kw, "micro_batch_size": mbs + 1}).bytes["activations"] > base.bytes["activations"]
    assert plan_memory(mc, **kw, zero1=True).bytes["optimizer"] * (cp * dp) == pytest.approx(base.bytes["optimizer"], rel=1e-6)
    if tp > 1:
        assert plan_memory(mc, **kw, sequence_parallel=True).bytes["activations"] < base.bytes["activations"]
    stage_params = sum(plan_memory(mc, **kw, stage=s).params for s in range(pp))
    assert stage_params * tp == pytest.approx(mc.num_params(), rel=1e-3)          # norm vectors are replicated over tp


@settings(max_examples=40, deadline=None, derandomize=True)
@given(sizes=st.lists(st.integers(1, 700), min_size=1, max_size=14), cap=st.integers(64, 1500), seed=st.integers(0, 10 ** 6))
def test_gradient_buckets_give_every_parameter_a_private_aligned_slice_and_keep_packed_groups_contiguous(sizes, cap, seed):
    import random
    import torch.nn as nn
    from picotron_b200.parallel.bucket import BucketManager
    params = [nn.Parameter(torch.zeros(n)) for n in sizes]
    rng = random.Random(seed)
    groups, i = [], 0
    while i + 1 < len(params):                               # some neighbouring parameters form units one GEMM consumes together
        if rng.random() < 0.4:
            groups.append([params[i], params[i + 1]])
            i += 2
        else:
            i += 1
    bm = BucketManager(params, None, cap, atomic_groups=groups)
    base = bm.flat.data_ptr()
    spans = []
    for p in params:
        off = (p.main_grad.data_ptr() - base) // 4
        assert 0 <= off and off + p.numel() <= bm.flat.numel()
        spans.append((off, off + p.numel()))
    for (a0, a1), (b0, b1) in zip(sorted(spans), sorted(spans)[1:]):
        assert a1 <= b0                                      # no two parameters share an element
    for grp in groups:                                       # a unit is one contiguous region, members back to back
        a, b = grp
        assert (b.main_grad.data_ptr() - a.main_grad.data_ptr()) // 4 == a.numel()
        assert bm.params_to_bucket_location[a][2] == bm.params_to_bucket_location[b][2]
    for bucket in bm.buckets:
        assert (bucket.grad_data.data_ptr() - base) % (64 * 4) == 0               # buckets start on 64-element boundaries
        units = {id(bm._group_of.get(p, [p])[0]) for p in bucket.params}
        assert bucket.grad_data.numel() <= cap or len(units) == 1                  # only a single oversized unit exceeds the cap
    assert sum(len(b.params) for b in bm.buckets) == len(params)
    # writing one parameter's gradient changes nothing else
    params[0].main_grad.fill_(1.0)
    assert float(bm.flat.sum()) == params[0].numel()
