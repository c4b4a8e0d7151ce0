"""Parallel strategies on real GPUs (bf16, NCCL, CUDA kernels) against the fp32 CPU oracle."""
import pytest
import torch

from dist_utils import run_distributed
import parallel_harness as H

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _run(tp=1, cp=1, pp=1, dp=1, engine="1f1b", grad_acc=2, layers=4, graph=False, cp_layout=None):
    world = tp * cp * pp * dp
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    res = run_distributed(H.worker, world, tp, cp, pp, dp, engine, grad_acc, layers, True, graph, None, cp_layout,
                          backend="nccl")
    H.check(res, tp, cp, pp, dp, grad_acc, layers, gpu=True)


def test_dp2():
    _run(dp=2)


def test_tp2():
    _run(tp=2)


def test_pp2_1f1b():
    _run(pp=2, grad_acc=3)


def test_pp2_afab():
    _run(pp=2, engine="afab", grad_acc=3)


def test_cp2():
    _run(cp=2)


def test_dp2_tp2():
    _run(dp=2, tp=2)


def test_tp2_cp2_pp2():
    _run(tp=2, cp=2, pp=2)


def test_dp2_tp2_pp2():
    _run(dp=2, tp=2, pp=2)


def test_tp2_micro_batches_replayed_from_a_cuda_graph():
    _run(tp=2, grad_acc=3, graph=True)


def test_cp2_micro_batches_replayed_from_a_cuda_graph():
    _run(cp=2, grad_acc=3, graph=True)


def test_dp2_micro_batches_replayed_from_a_cuda_graph():
    _run(dp=2, grad_acc=3, graph=True)


def test_cp2_zigzag_layout():
    _run(cp=2, cp_layout="zigzag")
