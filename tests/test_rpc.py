"""The RPC agent across three processes: sync and async calls with tensors in arguments and
results, remote errors, remote references. CPU here; with CUDA tensors under -m gpu."""
import pytest

import rpc_selftest


def test_rpc_three_processes_cpu(built):
    assert rpc_selftest.run(world=3, use_cuda=False) == [(0, True), (1, True), (2, True)]


@pytest.mark.gpu
def test_rpc_two_processes_cuda(built):
    assert rpc_selftest.run(world=2, use_cuda=True) == [(0, True), (1, True)]
