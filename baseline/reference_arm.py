"""Reference arm of bench.py: runs the reference's own build for the same metric and config.

The reference's source tree cannot be built offline (its third_party submodule directories are empty
and its setup.py insists on clang-6.0; `pip install --no-index` of the tree fails in cmake), so this
arm uses the reference as PyTorch ships it: the TensorPipe public headers under
torch/include/tensorpipe and the compiled library inside libtorch_cpu.so / libtorch_cuda.so.
baseline/ref_pipe_bench.cc is a small harness over that public C++ API (Context, Listener, Pipe;
uv + shm transports; basic, cuda_xth, cuda_ipc, cuda_basic channels with PyTorch's priorities) that
runs the same ring as the native arm. It is compiled on first use into baseline/_ref/. No model,
kernel or engine of this repository is on that path.
"""
import json
import os
import select
import subprocess
import sys
import time

MIXED_SEED = 1  # the seed bench.py gives the native mixed message

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)
BIN = os.path.join(HERE, "_ref", "ref_pipe_bench")


def unavailable(why):
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    sys.exit(0)


def build():
    """Compile the harness against the torch-bundled reference. Returns an error string or None."""
    src = os.path.join(HERE, "ref_pipe_bench.cc")
    if os.path.exists(BIN) and os.path.getmtime(BIN) >= os.path.getmtime(src):
        return None
    # Every rank lands here at once: one compiles (into a temporary name, renamed when complete),
    # the others wait for the lock and then find the binary in place.
    import fcntl
    os.makedirs(os.path.dirname(BIN), exist_ok=True)
    with open(BIN + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.exists(BIN) and os.path.getmtime(BIN) >= os.path.getmtime(src):
                return None
            return _compile(src)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _compile(src):
    import torch
    tdir = os.path.dirname(torch.__file__)
    nv = os.path.join(os.path.dirname(tdir), "nvidia", "cuda_runtime", "lib")
    if not os.path.exists(os.path.join(tdir, "include", "tensorpipe", "tensorpipe.h")):
        return "torch does not ship the TensorPipe headers"
    os.makedirs(os.path.dirname(BIN), exist_ok=True)
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    tmp = f"{BIN}.{os.getpid()}.tmp"
    cmd = [cxx, "-std=c++17", "-O2", f"-I{tdir}/include", "-I/usr/local/cuda/include", src, "-o", tmp,
           f"-L{tdir}/lib", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", f"-Wl,-rpath,{tdir}/lib",
           f"-L{nv}", "-l:libcudart.so.12", f"-Wl,-rpath,{nv}", "-lpthread"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.unlink(tmp)
        return "harness does not compile: " + proc.stderr.strip().splitlines()[-1][:200]
    os.replace(tmp, BIN)
    return None


class Harness:
    def __init__(self, rank, world, device, next_device, base_port, max_bytes, channels="all"):
        self.proc = subprocess.Popen(
            [BIN, "--rank", str(rank), "--world", str(world), "--device", str(device), "--next-device",
             str(next_device), "--base-port", str(base_port), "--max-bytes", str(max_bytes),
             "--channels", channels],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, bufsize=1)

    def readline(self, timeout):
        deadline = time.time() + timeout
        while time.time() < deadline:
            if self.proc.poll() is not None:
                raise RuntimeError("harness exited: " + (self.proc.stderr.read() or "")[-300:].replace("\n", " "))
            r, _, _ = select.select([self.proc.stdout], [], [], 0.5)
            if r:
                line = self.proc.stdout.readline()
                if line:
                    return line.strip()
        raise RuntimeError("harness timed out")

    def send(self, line):
        self.proc.stdin.write(line + "\n")
        self.proc.stdin.flush()

    def command(self, line, timeout=300):
        self.send(line)
        out = self.readline(timeout)
        if not out.startswith("ok"):
            raise RuntimeError("harness said: " + out)
        return out.split()[1:]

    def close(self):
        try:
            self.send("quit")
            self.proc.wait(timeout=20)
        except Exception:
            self.proc.kill()


def main(args, metric):
    err = build()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if err:
        if rank == 0:
            unavailable(err)
        sys.exit(0)

    import torch
    import torch.distributed as dist
    sys.path.insert(0, REPO)
    from bench import ClockSampler, bench_config, messages_per_step, percentile

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def all_ok(ok):
        if world == 1:
            return ok
        t = torch.tensor([1.0 if ok else 0.0], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item() > 0.5)

    base_port = int(os.environ.get("MASTER_PORT", "29500")) + 211
    max_bytes = max(args.bytes, 0 if args.no_sweep else args.max_sweep_bytes)
    failure = None
    h = None
    try:
        h = Harness(rank, world, local_rank, (local_rank + 1) % world if world > 1 else local_rank, base_port, max_bytes)
        if h.readline(120) != "up":
            raise RuntimeError("harness did not come up")
    except Exception as exc:  # noqa: BLE001
        failure = str(exc)
    if not all_ok(failure is None):
        if h:
            h.proc.kill()
        if rank == 0:
            unavailable("reference harness failed to start: " + (failure or "on another rank"))
        sys.exit(0)

    try:
        burst = messages_per_step(args.bytes, args.steps)
        h.command(f"stream {args.bytes} {max(args.warmup, 3) * burst} {args.depth}", timeout=900)
        barrier()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        ms = float(h.command(f"stream {args.bytes} {args.steps * burst} {args.depth}", timeout=1800)[0])
        barrier()
        clocks = sampler.stop() if rank == 0 else None
        ms = max_over_ranks(ms)
        ms_per_step = ms / args.steps
        value = world * burst * args.bytes / (ms_per_step * 1e-3) / 1e9

        sweep = []
        if not args.no_sweep:
            size = 4096
            while size <= args.max_sweep_bytes:
                # The same counts as the native arm: a thousand small messages per measurement.
                iters = 1000 if size <= (1 << 20) else (100 if size <= (64 << 20) else 20)
                h.command(f"stream {size} {max(10, iters // 10)} {args.depth}")
                barrier()
                t = max_over_ranks(float(h.command(f"stream {size} {iters} {args.depth}")[0])) / iters
                barrier()
                sweep.append({"bytes": size, "us_per_msg": round(t * 1e3, 2),
                              "GBps": round(world * size / (t * 1e-3) / 1e9, 2)})
                size *= 2

        barrier()
        h.command("latency 4096 50")
        barrier()
        lat = [float(x) for x in h.command("latency 4096 1000")[1:]]
        barrier()
        latency = None
        if rank == 0 and lat:
            latency = {"bytes": 4096, "p50_us": round(percentile(lat, 0.5), 2),
                       "p99_us": round(percentile(lat, 0.99), 2), "mean_us": round(sum(lat) / len(lat), 2),
                       "hops": world}

        e2e = None
        if not args.no_e2e:
            steps = max(5, min(args.steps, 20))
            h.send(f"e2e {args.bytes} {steps}")
            if h.readline(300) != "ready":
                raise RuntimeError("e2e warm-up failed")
            barrier()
            h.send("go")
            out = h.readline(600)
            if not out.startswith("ok"):
                raise RuntimeError("e2e failed: " + out)
            dt = max_over_ranks(float(out.split()[1])) * 1e-3
            e2e = {"value": round(world * args.bytes * steps / dt / 1e9, 3), "unit": "GB/s", "steps": steps,
                   "h2d_bytes_per_step": args.bytes, "d2h_bytes_per_step": 4,
                   "api": "tensorpipe::Pipe::write / readDescriptor / read (reference C++ API)"}
        # The 64-tensor message with the delivered sizes of the native mixed message, contiguous and
        # unconverted (the reference has neither views nor casts): its layout work is left out. Last
        # and guarded, so that a failure here cannot cost the numbers above.
        mixed = None
        try:
            mixed_steps = 20
            h.command(f"mixed 3 2 {MIXED_SEED}")
            barrier()
            out = h.command(f"mixed {mixed_steps} 2 {MIXED_SEED}")
            barrier()
            mixed_ms = max_over_ranks(float(out[0])) / mixed_steps
            mixed = {"tensors": 64, "bytes_per_msg": int(out[1]), "ms_per_msg": round(mixed_ms, 4),
                     "GBps": round(world * int(out[1]) / (mixed_ms * 1e-3) / 1e9, 2),
                     "note": "contiguous tensors of the delivered sizes; no transposed views, no conversion"}
        except Exception as exc:  # noqa: BLE001
            mixed = {"error": str(exc)}
    except Exception as exc:  # noqa: BLE001
        failure = str(exc)
    ok = all_ok(failure is None)
    h.close()
    if not ok:
        if rank == 0:
            unavailable("reference run failed: " + (failure or "on another rank"))
        sys.exit(0)

    if rank == 0:
        line = {
            "metric": metric, "value": round(value, 3), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
            "reference_build": "TensorPipe as bundled in PyTorch (torch/include/tensorpipe, libtorch_cpu/cuda)",
            "config": bench_config(args, world, burst),
            "data_path": "cuda_xth (same process) / cuda_ipc (other process) / cuda_basic: cudaMemcpyAsync",
            "timed_region_s": round(ms * 1e-3, 4),
            "clocks": clocks, "gpu_launches": 0, "e2e": e2e, "sweep": sweep, "latency": latency,
            "mixed_64_tensor_message": mixed,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
