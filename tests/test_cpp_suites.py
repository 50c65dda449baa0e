"""Runs the C++ test binary suite by suite, so that a failure names the suite in pytest's report.

The C++ tests are where most of the library is exercised (codec golden bytes, transports,
channels, pipes, failure handling with forked peers); this file only dispatches them."""
import subprocess

import pytest

CPU_SUITES = ["Nop.", "Transport.", "TransportShm.", "TransportUv.", "Pipe.", "Context.", "Listener.",
              "Channel.", "Common.", "Faults.", "Plan.", "RoleRing.", "VerbsLoopback.", "VerbsSystem.",
              "TransportIbv.", "CudaGdr.", "CmaMatrix."]
GPU_SUITES = ["Kernel.", "CudaPipe.", "CudaBasic.", "CudaChannel."]


def run(binary, args):
    proc = subprocess.run([binary] + args, capture_output=True, text=True, timeout=1200)
    tail = "\n".join(proc.stdout.splitlines()[-60:]) + "\n" + proc.stderr[-4000:]
    assert proc.returncode == 0, tail
    return proc.stdout


@pytest.mark.parametrize("suite", CPU_SUITES)
def test_cpu_suite(test_binary, suite):
    run(test_binary, [f"--filter={suite}"])


@pytest.mark.gpu
@pytest.mark.parametrize("suite", GPU_SUITES)
def test_gpu_suite(test_binary, suite):
    out = run(test_binary, ["--gpu", f"--filter={suite}"])
    assert "0 failed" in out
