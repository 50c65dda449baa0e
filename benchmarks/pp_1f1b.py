#!/usr/bin/env python
"""Pipeline-parallel activation traffic: a GPT-2-medium-shaped model (24 layers, d_model 1024, 16 heads,
random init, bf16) split over N stages (24/N layers each; the headline config is 8 stages of 3 layers),
micro-batch 8 x 1024 tokens, so each forward hands a 16 MiB activation to the next stage and each backward
hands a 16 MiB gradient to the previous one, through pipes. 32 micro-batches per step in a 1F1B schedule,
real forward/backward compute and an SGD step every step. Metric: steps per second.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29551 benchmarks/pp_1f1b.py --steps 5
"""
import argparse
import json
import time

from common import Ranks, mesh_pipes, torch


def build_stage(layers, d_model, heads, device):
    blocks = [torch.nn.TransformerEncoderLayer(d_model, heads, 4 * d_model, dropout=0.0, batch_first=True,
                                               norm_first=True, activation="gelu") for _ in range(layers)]
    return torch.nn.Sequential(*blocks).to(device=device, dtype=torch.bfloat16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--micro-batches", type=int, default=32)
    ap.add_argument("--layers", type=int, default=24)
    args = ap.parse_args()
    r = Ranks()
    S, s = r.world, r.rank
    if S < 2 or args.layers % S:
        raise SystemExit("needs >= 2 stages that divide the layer count")
    torch.manual_seed(1 + s)
    B, T, D = 8, 1024, 1024
    stage = build_stage(args.layers // S, D, 16, r.device)
    opt = torch.optim.SGD(stage.parameters(), lr=1e-4)
    ctx, listener, pipes = mesh_pipes(r, "pp", pairs=[(i, i + 1) for i in range(S - 1)])
    prev_pipe, next_pipe = pipes.get(s - 1), pipes.get(s + 1)
    devices = r.gather(r.local_rank)
    M = args.micro_batches
    depth = min(S, M) + 1
    act_in = [torch.empty(B, T, D, dtype=torch.bfloat16, device=r.device) for _ in range(depth)]
    grad_in = [torch.empty(B, T, D, dtype=torch.bfloat16, device=r.device) for _ in range(depth)]
    data = torch.randn(B, T, D, dtype=torch.bfloat16, device=r.device)  # synthetic input of stage 0

    def step():
        pending_sends = []
        live = {}  # micro-batch -> (input, output)

        def forward(mb):
            if prev_pipe is not None:
                x = prev_pipe.recv(out=[act_in[mb % depth]]).result(300).tensors[0]
                x = x.detach().requires_grad_(True)
            else:
                x = data
            y = stage(x)
            if next_pipe is not None:
                pending_sends.append(next_pipe.send([y.detach()], target_devices=[f"cuda:{devices[s + 1]}"]))
            live[mb] = (x, y)

        def backward(mb):
            x, y = live.pop(mb)
            if next_pipe is not None:
                gy = next_pipe.recv(out=[grad_in[mb % depth]]).result(300).tensors[0]
                y.backward(gy)
            else:
                y.float().pow(2).mean().backward()
            if prev_pipe is not None:
                pending_sends.append(prev_pipe.send([x.grad], target_devices=[f"cuda:{devices[s - 1]}"]))

        warm = min(S - s - 1, M)
        f = b = 0
        for _ in range(warm):
            forward(f)
            f += 1
        while f < M:  # steady state: one forward, one backward
            forward(f)
            f += 1
            backward(b)
            b += 1
        while b < M:
            backward(b)
            b += 1
        for fut in pending_sends:
            fut.result(300)
        opt.step()
        opt.zero_grad(set_to_none=True)

    for _ in range(args.warmup):
        step()
    r.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize()
    dt = r.max(time.perf_counter() - t0)
    r.barrier()
    if r.rank == 0:
        print(json.dumps({
            "workload": "pipeline_1f1b", "impl": "native", "stages": S, "layers_per_stage": args.layers // S,
            "micro_batches": M, "activation_bytes": B * T * D * 2, "steps": args.steps,
            "steps_per_second": round(args.steps / dt, 4), "seconds_per_step": round(dt / args.steps, 4),
            "model": "GPT-2-medium-shaped (d_model 1024, 16 heads, bf16, random init)",
        }), flush=True)
    for p in pipes.values():
        p.close()
    ctx.join()
    r.finish()


if __name__ == "__main__":
    main()
