"""Compiles the reference-side programs into baseline/_ref/ against the TensorPipe that PyTorch ships
(headers in torch/include/tensorpipe, code in libtorch_cpu.so / libtorch_cuda.so):
  ref_pipe_bench     ring benchmark harness driven by bench.py --impl reference
  ref_interop        echo peer for the wire-compatibility tests
  ref_pipe_workloads benchmarks/pipe_workloads.cc compiled with -DUSE_REFERENCE (same code, other library)
Usage: python baseline/build_ref.py [name ...]   (default: all). Prints what it built or why not."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)
OUT = os.path.join(HERE, "_ref")

TARGETS = {
    "ref_pipe_bench": (os.path.join(HERE, "ref_pipe_bench.cc"), [], True),
    "ref_interop": (os.path.join(HERE, "ref_interop.cc"), [], False),
    "ref_pipe_workloads": (os.path.join(REPO, "benchmarks", "pipe_workloads.cc"), ["-DUSE_REFERENCE"], True),
}


def build(name):
    """Returns None on success (or when up to date), else a one-line reason."""
    import torch
    src, defines, cuda = TARGETS[name]
    out = os.path.join(OUT, name)
    if os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(src):
        return None
    tdir = os.path.dirname(torch.__file__)
    if not os.path.exists(os.path.join(tdir, "include", "tensorpipe", "tensorpipe.h")):
        return "torch does not ship the TensorPipe headers"
    os.makedirs(OUT, exist_ok=True)
    nv = os.path.join(os.path.dirname(tdir), "nvidia", "cuda_runtime", "lib")
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    cmd = [cxx, "-std=c++17", "-O2", f"-I{tdir}/include", "-I/usr/local/cuda/include", *defines, src, "-o", out,
           f"-L{tdir}/lib", "-ltorch_cpu", "-lc10", f"-Wl,-rpath,{tdir}/lib", "-lpthread"]
    if cuda:
        cmd += ["-ltorch_cuda", "-lc10_cuda", f"-L{nv}", "-l:libcudart.so.12", f"-Wl,-rpath,{nv}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        lines = proc.stderr.strip().splitlines()
        return "does not compile: " + (lines[-1][:200] if lines else "unknown error")
    return None


if __name__ == "__main__":
    for target in (sys.argv[1:] or list(TARGETS)):
        why = build(target)
        print(f"{target}: {'ok' if why is None else why}")
