"""Shared plumbing of the multi-rank Python benchmarks: rank discovery, barriers, full-mesh pipes."""
import os
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO not in sys.path:
    sys.path.insert(0, REPO)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import tensorpipe_b200 as tpb  # noqa: E402


class Ranks:
    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.device)

    def barrier(self):
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def gather(self, obj):
        if self.world == 1:
            return [obj]
        out = [None] * self.world
        dist.all_gather_object(out, obj)
        return out

    def max(self, x):
        if self.world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def finish(self):
        if self.world > 1:
            dist.barrier()
            dist.destroy_process_group()


def mesh_pipes(ranks: Ranks, name="mesh", pairs=None):
    """One bidirectional pipe per pair of ranks (the lower rank dials). Returns (context, {peer: pipe}).
    `pairs` restricts the mesh, e.g. to neighbours of a pipeline."""
    ctx = tpb.default_context(f"{name}{ranks.rank}")
    listener = ctx.listen(["uv://127.0.0.1", "shm://"])
    urls = ranks.gather(listener.url("uv"))
    wanted = pairs if pairs is not None else [(i, j) for i in range(ranks.world) for j in range(i + 1, ranks.world)]
    mine_in = sorted(i for (i, j) in wanted if j == ranks.rank)
    mine_out = sorted(j for (i, j) in wanted if i == ranks.rank)
    pipes = {}
    accepted = [listener.accept_future() for _ in mine_in]
    for peer in mine_out:
        pipes[peer] = ctx.connect(urls[peer], remote_name=f"{name}{peer}")
        # tell the peer who we are: accepted pipes carry the dialer's context name
    for fut in accepted:
        pipe = fut.result(120)
        peer = int(pipe.remote_name[len(name):])
        pipes[peer] = pipe
    ranks.barrier()
    return ctx, listener, pipes
