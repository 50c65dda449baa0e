#!/usr/bin/env python
"""Where the time of one message goes: a timeline of one hop between two GPUs, from the library's
own trace events.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29541 benchmarks/hop_timeline.py [--bytes 4096,16777216] [--laps 300]

Two ranks pass one message round the ring at a time (the latency mode of the ring benchmark) with
tracing on; every stage of a message stamps an event (src/core/pipe_traffic.cc, cuda_p2p.cc,
push.cu) from the steady clock, which the two processes of one host share. For every lap the
events of the sending rank and of the receiving rank are lined up by their order of occurrence,
and the table gives the median (and 90th percentile) time of each stage after the sender's
`Pipe::write`, in microseconds. Prints one markdown table per message size.
"""
import argparse
import json
import os
import sys
import tempfile

from common import Ranks

# (rank role, event name, phase, label)
STAGES = [
    ("send", "pipe.write", "i", "sender: Pipe::write called"),
    ("send", "pipe.announced", "i", "sender: descriptor frame handed to the transport"),
    ("send", "p2p.send.eager", "B", "sender: channel starts an eager push (small messages)"),
    ("recv", "pipe.descriptor", "i", "receiver: descriptor arrived, readDescriptor callback"),
    ("recv", "pipe.read", "i", "receiver: Pipe::read called with the allocation"),
    ("send", "p2p.send.rendezvous", "B", "sender: RecvReady arrived, channel plans the push"),
    ("send", "tpb_push_pack launch", "B", "sender: kernel launch begins"),
    ("send", "tpb_push_pack launch", "E", "sender: kernel launch returned"),
    ("send", "pipe.write.done", "i", "sender: write callback"),
    ("recv", "p2p.recv.complete", "B", "receiver: Launched frame arrived, stream wait being queued"),
    ("recv", "tpb_push_pack launch", "B", "receiver: unpack kernel launch begins (eager only)"),
    ("recv", "tpb_push_pack launch", "E", "receiver: unpack kernel launch returned (eager only)"),
    ("recv", "pipe.read.done", "i", "receiver: read callback (data ordered on its stream)"),
]


def occurrences(events, name, phase):
    return [e["ts"] for e in events if e["name"] == name and e["ph"] == phase]


def percentile(v, q):
    s = sorted(v)
    return s[min(len(s) - 1, int(q * len(s)))]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--bytes", default="4096,16777216")
    ap.add_argument("--laps", type=int, default=300)
    args = ap.parse_args()
    ranks = Ranks()
    if ranks.world != 2:
        raise SystemExit("run with two ranks")
    from tensorpipe_b200 import _C

    sizes = [int(x) for x in args.bytes.split(",")]
    rb = _C.RingBench(device=ranks.local_rank, max_bytes=max(sizes))
    urls = ranks.gather(f"{rb.listen_url()}|{ranks.local_rank}")
    rb.connect(urls[(ranks.rank + 1) % 2])
    tmp = tempfile.mkdtemp(prefix="tpb-timeline-")
    for size in sizes:
        rb.run_latency(size, 50, ranks.rank, 2)
        ranks.barrier()
        path = os.path.join(tmp, f"trace_{size}_r{ranks.rank}.json")
        _C.trace_enable(path)
        lat = rb.run_latency(size, args.laps, ranks.rank, 2)
        ranks.barrier()
        _C.trace_dump()
        _C.trace_disable()
        with open(path) as f:
            events = json.load(f)
        wanted = {name for _, name, _, _ in STAGES}
        mine = [{"name": e["name"], "ph": e["ph"], "ts": e["ts"]} for e in events if e["name"] in wanted]
        both = ranks.gather(mine)
        if ranks.rank != 0:
            continue
        # Rank 0 starts every lap; its outgoing message is received by rank 1.
        by_role = {"send": both[0], "recv": both[1]}
        starts = occurrences(by_role["send"], "pipe.write", "i")
        rows = []
        for role, name, phase, label in STAGES:
            ts = occurrences(by_role[role], name, phase)
            # Each rank both sends and receives once per lap. Pipe and channel events carry their
            # side in their name; kernel launches do not: with eager messages a rank launches twice
            # per lap (rank 0: its push, then the unpack of what comes back; rank 1: the unpack of
            # what it receives, then its own push), with rendezvous once (its push).
            if name == "tpb_push_pack launch":
                if len(ts) == 2 * len(starts):
                    ts = ts[0::2]
                elif role == "recv":
                    continue
            if len(ts) != len(starts) or not ts:
                continue
            deltas = [t - s for t, s in zip(ts, starts)]
            deltas = deltas[len(deltas) // 10:]  # the first laps still warm caches up
            rows.append((label, percentile(deltas, 0.5), percentile(deltas, 0.9)))
        rows.sort(key=lambda r: r[1])
        p50 = percentile(lat, 0.5) if lat else float("nan")
        print(f"\n### {size} bytes, {args.laps} laps, one hop GPU {0} -> GPU {1} "
              f"(lap of two hops: p50 {p50:.1f} us)\n")
        print("| stage | median us after Pipe::write | p90 |")
        print("|---|---|---|")
        for label, med, p90 in rows:
            print(f"| {label} | {med:.1f} | {p90:.1f} |")
        sys.stdout.flush()
    del rb
    ranks.finish()


if __name__ == "__main__":
    main()
