#!/usr/bin/env python
"""All-pairs multi-tensor messages: every rank concurrently sends every other rank a message of 64
tensors with mixed dtypes (fp32, bf16, int64), sizes log-uniform from 1 KiB to 16 MiB, a quarter of
them non-contiguous transposed 2-D views (8 to 4096 columns, log-uniform), and the receiver asks for an fp32 -> bf16 conversion on
half of the fp32 tensors. Each message is moved by one fused kernel launch on its sender.
Reports aggregate and per-GPU GB/s (bytes delivered), timed on the device, max over ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29541 benchmarks/all_pairs.py --iters 10
"""
import argparse
import json
import math
import random

from common import Ranks, mesh_pipes, torch


def make_message(seed, device):
    rng = random.Random(seed)
    tensors, casts, delivered = [], {}, 0
    fp32_seen = 0
    for i in range(64):
        dtype = (torch.float32, torch.bfloat16, torch.int64)[i % 3]
        nbytes = int(math.exp(rng.uniform(math.log(1024), math.log(16 << 20))))
        elems = max(64, nbytes // torch.empty((), dtype=dtype).element_size())
        cols = int(math.exp(rng.uniform(math.log(8), math.log(4096)))) if i % 4 == 3 else 64
        rows = max(1, elems // cols)
        if dtype == torch.int64:
            t = torch.randint(-1000, 1000, (cols, rows) if i % 4 == 3 else (rows, cols), dtype=dtype, device=device)
        else:
            t = torch.randn((cols, rows) if i % 4 == 3 else (rows, cols), dtype=dtype, device=device)
        if i % 4 == 3:
            t = t.t()  # a transposed view: [rows, cols] with strides (1, rows)
        out_dtype = dtype
        if dtype == torch.float32:
            if fp32_seen % 2 == 0:
                casts[i] = torch.bfloat16
                out_dtype = torch.bfloat16
            fp32_seen += 1
        delivered += rows * cols * torch.empty((), dtype=out_dtype).element_size()
        tensors.append(t)
    return tensors, casts, delivered


def native(args, r):
    """The same traffic driven from C++ (no Python per tensor): what the channel itself can do."""
    from tensorpipe_b200 import _C
    rb = _C.RingBench(device=r.local_rank, max_bytes=1 << 30)
    urls = r.gather(f"{rb.listen_url()}|{r.local_rank}")
    rb.connect_mesh(urls, r.rank)
    r.barrier()
    rb.run_mixed_mesh(args.warmup, 1234)
    r.barrier()
    res, delivered = rb.run_mixed_mesh(args.iters, 1234)
    r.barrier()
    ms = r.max(res.device_ms) / args.iters
    if r.rank == 0:
        per_gpu_out = delivered * (r.world - 1)
        print(json.dumps({
            "workload": "all_pairs_64_tensor_messages", "impl": "native", "driver": "C++ engine", "n_gpus": r.world,
            "bytes_delivered_per_message": delivered, "messages_per_round": r.world * (r.world - 1),
            "ms_per_round": round(ms, 4),
            "aggregate_GBps": round(per_gpu_out * r.world / (ms * 1e-3) / 1e9, 2),
            "per_gpu_egress_GBps": round(per_gpu_out / (ms * 1e-3) / 1e9, 2),
            "nvlink_roofline_fraction_of_770GBps": round(per_gpu_out / (ms * 1e-3) / 1e9 / 770.0, 3),
            "kernel_launches_per_message": res.kernel_launches / (args.iters * (r.world - 1)),
        }), flush=True)
    del rb
    r.finish()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--python-api", action="store_true",
                    help="drive the messages through the torch-facing Python API instead of the native engine")
    args = ap.parse_args()
    r = Ranks()
    if r.world < 2:
        raise SystemExit("all_pairs needs at least 2 ranks")
    if not args.python_api:
        return native(args, r)
    ctx, listener, pipes = mesh_pipes(r, "ap")
    torch.manual_seed(1234)  # every rank builds the same message, values included
    tensors, casts, delivered = make_message(1234, r.device)
    peers = sorted(pipes)
    devices = r.gather(r.local_rank)
    recv_bufs = {p: [torch.empty(t.shape, dtype=casts.get(i, t.dtype), device=r.device) for i, t in enumerate(tensors)]
                 for p in peers}

    def one_round(check=False):
        sends = [pipes[p].send(tensors, target_devices=[f"cuda:{devices[p]}"] * 64) for p in peers]
        recvs = [pipes[p].recv(cast=casts, out=recv_bufs[p]) for p in peers]
        msgs = [f.result(300) for f in recvs]
        for f in sends:
            f.result(300)
        if check:
            torch.cuda.synchronize()
            for m in msgs:
                for i, (got, sent) in enumerate(zip(m.tensors, tensors)):
                    want = sent.to(casts[i]) if i in casts else sent
                    if not torch.equal(got, want.contiguous()):
                        diff = (got.float() - want.contiguous().float()).abs()
                        raise AssertionError(
                            f"tensor {i} differs: shape {tuple(got.shape)} dtype {got.dtype} cast {i in casts} "
                            f"bad {int((diff > 0).sum())}/{diff.numel()} max {float(diff.max())} "
                            f"got[:4] {got.flatten()[:4].tolist()} want[:4] {want.flatten()[:4].tolist()}")

    one_round(check=True)  # every rank builds the same message, so each can check what it received
    for _ in range(args.warmup):
        one_round()
    r.barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.iters):
        one_round()
    end.record()
    torch.cuda.synchronize()
    ms = r.max(start.elapsed_time(end)) / args.iters
    r.barrier()
    if r.rank == 0:
        per_gpu_out = delivered * (r.world - 1)
        print(json.dumps({
            "workload": "all_pairs_64_tensor_messages", "impl": "native", "n_gpus": r.world,
            "bytes_delivered_per_message": delivered, "messages_per_round": r.world * (r.world - 1),
            "ms_per_round": round(ms, 4),
            "aggregate_GBps": round(per_gpu_out * r.world / (ms * 1e-3) / 1e9, 2),
            "per_gpu_egress_GBps": round(per_gpu_out / (ms * 1e-3) / 1e9, 2),
            "nvlink_roofline_fraction_of_770GBps": round(per_gpu_out / (ms * 1e-3) / 1e9 / 770.0, 3),
            "verified": "first round compared element-wise with torch (views and casts included)",
        }), flush=True)
    for p in pipes.values():
        p.close()
    ctx.join()
    r.finish()


if __name__ == "__main__":
    main()
