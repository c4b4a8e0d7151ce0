"""Every parallel strategy and both pipeline engines on CPU/Gloo against the single-process oracle."""
import pytest

from dist_utils import run_distributed
import parallel_harness as H


def _run(tp=1, cp=1, pp=1, dp=1, engine="1f1b", grad_acc=2, layers=4):
    world = tp * cp * pp * dp
    res = run_distributed(H.worker, world, tp, cp, pp, dp, engine, grad_acc, layers)
    H.check(res, tp, cp, pp, dp, grad_acc, layers)


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


def test_cp2_dp2():
    _run(cp=2, dp=2)


def test_4d_grid_dp2_tp2_pp2_1f1b():
    _run(tp=2, pp=2, dp=2, engine="1f1b", grad_acc=2)


def test_tp2_cp2_pp2_1f1b():
    _run(tp=2, cp=2, pp=2, engine="1f1b", grad_acc=2)
