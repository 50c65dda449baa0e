#!/usr/bin/env python
"""How close the push kernel gets to the copy engines on the NVLink between two GPUs of this box.

One process, two GPUs, one large buffer each way: `cudaMemcpyAsync` device to device (what the
reference's cuda_ipc / cuda_xth channels issue) against the library's push kernel storing into the
peer's memory, in one direction and in both at once. Device-timed with CUDA events; prints one
JSON line. The numbers are the denominators the bandwidth tables of this repository quote next to
the nominal 900 GB/s per direction.

    python benchmarks/link_ceiling.py [--bytes 268435456] [--iters 20] [--only kernel|bulk|plain|copy]
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from tensorpipe_b200 import _C  # noqa: E402


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--bytes", type=int, default=256 << 20)
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--only", default="", help="copy | bulk | plain: run just that variant (one direction)")
    args = p.parse_args()
    if torch.cuda.device_count() < 2:
        raise SystemExit("needs two GPUs")
    n = args.bytes
    a0 = torch.empty(n, dtype=torch.uint8, device="cuda:0")
    b0 = torch.empty(n, dtype=torch.uint8, device="cuda:0")
    a1 = torch.empty(n, dtype=torch.uint8, device="cuda:1")
    b1 = torch.empty(n, dtype=torch.uint8, device="cuda:1")
    b1.copy_(a0)  # enables peer access both ways
    b0.copy_(a1)
    torch.cuda.synchronize(0)
    torch.cuda.synchronize(1)
    s0 = torch.cuda.Stream(device=0)
    s1 = torch.cuda.Stream(device=1)
    w0 = torch.zeros(64, dtype=torch.int32, device="cuda:0")  # flag and arrive counter
    w1 = torch.zeros(64, dtype=torch.int32, device="cuda:1")

    def copy0():
        with torch.cuda.device(0), torch.cuda.stream(s0):
            b1.copy_(a0, non_blocking=True)

    def copy1():
        with torch.cuda.device(1), torch.cuda.stream(s1):
            b0.copy_(a1, non_blocking=True)

    def push(device, src, dst, stream, words, bulk):
        def run():
            with torch.cuda.device(device):
                _C.launch_push([(src.data_ptr(), dst.data_ptr(), n)], stream.cuda_stream, bulk, words.data_ptr(), 1,
                               words.data_ptr() + 64)
        return run

    def timed(fn0, fn1):
        for _ in range(args.warmup):
            fn0()
            if fn1:
                fn1()
        torch.cuda.synchronize(0)
        torch.cuda.synchronize(1)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        with torch.cuda.device(0):
            ev[0].record(s0)
        with torch.cuda.device(1):
            ev[2].record(s1)
        for _ in range(args.iters):
            fn0()
            if fn1:
                fn1()
        with torch.cuda.device(0):
            ev[1].record(s0)
        with torch.cuda.device(1):
            ev[3].record(s1)
        torch.cuda.synchronize(0)
        torch.cuda.synchronize(1)
        ms = ev[0].elapsed_time(ev[1]) / args.iters
        if fn1:
            ms = max(ms, ev[2].elapsed_time(ev[3]) / args.iters)
        return round(n / (ms * 1e-3) / 1e9, 1)

    variants = {
        "copy": (copy0, copy1),
        "bulk": (push(0, a0, b1, s0, w0, True), push(1, a1, b0, s1, w1, True)),
        "plain": (push(0, a0, b1, s0, w0, False), push(1, a1, b0, s1, w1, False)),
    }
    out = {"bytes": n, "iters": args.iters, "unit": "GB/s per direction"}
    for name, (f0, f1) in variants.items():
        if args.only and args.only != name:
            continue
        out[name + "_one_direction"] = timed(f0, None)
        if not args.only:
            out[name + "_both_directions"] = timed(f0, f1)
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
