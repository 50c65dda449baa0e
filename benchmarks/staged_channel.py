"""The staged CUDA channel (cuda_basic: device -> pinned host -> wire -> pinned host -> device)
against the reference's channel of the same name, on the same ring as bench.py.

    python benchmarks/staged_channel.py                       # one GPU, two pipe ends in one process
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29531 benchmarks/staged_channel.py      # one process per GPU

Both arms register only the staged channel beside the CPU one, so no device-to-device channel can
be selected. Prints one JSON line with microseconds per message and GB/s per size for each arm.
"""
import argparse
import json
import os
import sys

from common import REPO, Ranks

sys.path.insert(0, os.path.join(REPO, "baseline"))


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--sizes", default="4096,65536,1048576,16777216,268435456")
    p.add_argument("--depth", type=int, default=2)
    p.add_argument("--no-reference", action="store_true")
    args = p.parse_args()
    sizes = [int(x) for x in args.sizes.split(",")]
    ranks = Ranks()
    from tensorpipe_b200 import _C

    def iters_for(size):
        return 200 if size <= (1 << 20) else (40 if size <= (16 << 20) else 10)

    rb = _C.RingBench(device=ranks.local_rank, max_bytes=max(sizes), channel="cuda_basic")
    urls = ranks.gather(f"{rb.listen_url()}|{ranks.local_rank}")
    rb.connect(urls[(ranks.rank + 1) % ranks.world])
    ranks.barrier()
    native = []
    for size in sizes:
        check = rb.run_stream(size, 3, args.depth, True)
        if check.mismatches:
            raise RuntimeError(f"{check.mismatches} bytes differ at {size}")
        ranks.barrier()
        n = iters_for(size)
        ms = ranks.max(rb.run_stream(size, n, args.depth, False).device_ms) / n
        ranks.barrier()
        native.append({"bytes": size, "us_per_msg": round(ms * 1e3, 2),
                       "GBps": round(ranks.world * size / (ms * 1e-3) / 1e9, 3)})
    del rb

    reference = None
    if not args.no_reference:
        import reference_arm
        err = reference_arm.build()
        if err:
            reference = {"unavailable": err}
        else:
            port = int(os.environ.get("MASTER_PORT", "29500")) + 331
            nxt = (ranks.local_rank + 1) % ranks.world if ranks.world > 1 else ranks.local_rank
            h = reference_arm.Harness(ranks.rank, ranks.world, ranks.local_rank, nxt, port, max(sizes), "cuda_basic")
            try:
                if h.readline(120) != "up":
                    raise RuntimeError("harness did not come up")
                reference = []
                for size in sizes:
                    h.command(f"stream {size} 3 {args.depth}")
                    ranks.barrier()
                    n = iters_for(size)
                    ms = ranks.max(float(h.command(f"stream {size} {n} {args.depth}", timeout=900)[0])) / n
                    ranks.barrier()
                    reference.append({"bytes": size, "us_per_msg": round(ms * 1e3, 2),
                                      "GBps": round(ranks.world * size / (ms * 1e-3) / 1e9, 3)})
            finally:
                h.close()
    if ranks.rank == 0:
        print(json.dumps({"benchmark": "staged_channel", "n_gpus": ranks.world, "depth": args.depth,
                          "native_cuda_basic": native, "reference_cuda_basic": reference}), flush=True)
    ranks.finish()


if __name__ == "__main__":
    main()
