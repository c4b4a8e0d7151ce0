"""Every parallel strategy and both pipeline engines on CPU/Gloo against the single-process oracle."""
import pytest

from dist_utils import run_distributed
import parallel_harness as H


def _run(tp=1, cp=1, pp=1, dp=1, engine="1f1b", grad_acc=2, layers=4):
    world = tp * cp * pp * dp
    res = run_distributed(H.worker, world, tp, cp, pp, dp, engine, grad_acc, layers)
    H.check(res, tp, cp, pp, dp, grad_acc, layers)
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
