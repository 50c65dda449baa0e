#!/usr/bin/env python
"""The ring of bench.py with NCCL point-to-point calls in place of pipes: every rank sends one
tensor to the next rank and receives one from the previous rank, `--depth` pairs in flight. The
reference's own pipe benchmark has such an arm behind `USE_NCCL`
(tensorpipe/benchmark/benchmark_pipe.cc:28-51,180-200,429-462); it is context for the pipe numbers,
not a pipe: NCCL needs both ends to agree on every transfer in advance and moves no metadata.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29551 benchmarks/nccl_ring.py [--sizes 4096,1048576,16777216,268435456]

Device-timed with CUDA events, max over ranks; prints one JSON line.
"""
import argparse
import json

import torch
import torch.distributed as dist

from common import Ranks


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="4096,65536,1048576,16777216,268435456")
    ap.add_argument("--depth", type=int, default=2)
    args = ap.parse_args()
    ranks = Ranks()
    if ranks.world < 2:
        raise SystemExit("needs at least two ranks")
    nxt, prv = (ranks.rank + 1) % ranks.world, (ranks.rank - 1) % ranks.world
    rows = []
    for size in [int(x) for x in args.sizes.split(",")]:
        src = torch.empty(size, dtype=torch.uint8, device=ranks.device)
        dst = [torch.empty(size, dtype=torch.uint8, device=ranks.device) for _ in range(args.depth)]
        iters = 200 if size <= (1 << 20) else (50 if size <= (16 << 20) else 20)

        def burst(n):
            for i in range(0, n, args.depth):
                ops = []
                for d in range(args.depth):
                    ops.append(dist.P2POp(dist.isend, src, nxt))
                    ops.append(dist.P2POp(dist.irecv, dst[d], prv))
                for w in dist.batch_isend_irecv(ops):
                    w.wait()

        burst(4 * args.depth)
        ranks.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        burst(iters)
        b.record()
        torch.cuda.synchronize()
        ms = ranks.max(a.elapsed_time(b)) / iters
        rows.append({"bytes": size, "us_per_msg": round(ms * 1e3, 2),
                     "GBps": round(ranks.world * size / (ms * 1e-3) / 1e9, 2)})
        ranks.barrier()
    if ranks.rank == 0:
        print(json.dumps({"benchmark": "nccl_ring", "n_gpus": ranks.world, "depth": args.depth, "sizes": rows}), flush=True)
    ranks.finish()


if __name__ == "__main__":
    main()
