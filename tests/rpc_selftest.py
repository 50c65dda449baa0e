"""Worker bodies for the RPC agent's multi-process self-test (importable from spawned children)."""
import os
import sys

import torch


def add(a, b):
    return a + b


def describe(t):
    return {"shape": tuple(t.shape), "sum": float(t.sum()), "device": str(t.device)}


def boom():
    raise ValueError("intended failure")


class Counter:
    def __init__(self, start):
        self.value = start

    def bump(self, by):
        self.value += by
        return self.value


def worker(rank, world, port, use_cuda, results):
    """rank 0 drives calls to every other worker; everybody serves."""
    from datetime import timedelta

    from torch.distributed import TCPStore

    from tensorpipe_b200 import rpc

    try:
        store = TCPStore("127.0.0.1", port, world, rank == 0, timeout=timedelta(seconds=60))
        device = None
        if use_cuda:
            torch.cuda.set_device(rank % torch.cuda.device_count())
            device = f"cuda:{torch.cuda.current_device()}"
        agent = rpc.init_rpc(f"worker{rank}", rank, world, store, device=device)
        ok = True
        if rank == 0:
            for peer in range(1, world):
                name = f"worker{peer}"
                x = torch.arange(10.0)
                y = torch.ones(10)
                if use_cuda:
                    x, y = x.cuda(), y.cuda()
                z = agent.rpc_sync(name, add, args=(x, y))
                ok &= bool(torch.equal(z.cpu(), torch.arange(10.0) + 1))
                info = agent.rpc_sync(name, describe, args=(torch.ones(3, 4),))
                ok &= info["shape"] == (3, 4) and info["sum"] == 12.0
                futs = [agent.rpc_async(name, add, args=(i, i)) for i in range(20)]
                ok &= [f.result(60) for f in futs] == [2 * i for i in range(20)]
                try:
                    agent.rpc_sync(name, boom)
                    ok = False
                except RuntimeError as exc:
                    ok &= "intended failure" in str(exc)
                ref = agent.remote(name, Counter, args=(5,))
                ok &= ref.rpc_sync("bump", 2) == 7 and ref.rpc_sync("bump", 3) == 10
                ok &= ref.to_here().value == 10
            ok &= agent.rpc_sync("worker0", add, args=(1, 2)) == 3  # a call to oneself needs no wire
        results.put((rank, ok))
        agent.shutdown()
    except Exception as exc:  # noqa: BLE001
        results.put((rank, f"{type(exc).__name__}: {exc}"))
        raise


def run(world=3, use_cuda=False, port=None):
    import multiprocessing as mp
    import socket

    if port is None:
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, world, port, use_cuda, results)) for r in range(world)]
    for p in procs:
        p.start()
    out = [results.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(60)
    return sorted(out)


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    print(run(use_cuda="--cuda" in sys.argv))
