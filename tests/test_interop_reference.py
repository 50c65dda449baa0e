"""Wire-compatibility with the reference library, live: this library's pipes against an echo peer
built only from the TensorPipe that PyTorch ships (baseline/ref_interop.cc), in both directions,
over the uv transport and the basic channel, also with every other CPU backend registered on both
sides (which the two must then agree not to use). This is what validates the from-scratch libnop codec
and the handshake (Packet, Brochure, BrochureAnswer, Descriptor, DescriptorReply) end to end.
Skipped when torch does not ship the TensorPipe headers or the peer cannot be compiled."""
import os
import socket
import subprocess
import threading

import pytest
import torch

import tensorpipe_b200 as tpb

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)
SRC = os.path.join(REPO, "baseline", "ref_interop.cc")
BIN = os.path.join(REPO, "baseline", "_ref", "ref_interop")


def build_peer():
    tdir = os.path.dirname(torch.__file__)
    if not os.path.exists(os.path.join(tdir, "include", "tensorpipe", "tensorpipe.h")):
        pytest.skip("torch does not ship the TensorPipe headers")
    if os.path.exists(BIN) and os.path.getmtime(BIN) >= os.path.getmtime(SRC):
        return BIN
    os.makedirs(os.path.dirname(BIN), exist_ok=True)
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    cmd = [cxx, "-std=c++17", "-O1", f"-I{tdir}/include", SRC, "-o", BIN, f"-L{tdir}/lib", "-ltorch_cpu", "-lc10",
           f"-Wl,-rpath,{tdir}/lib", "-lpthread"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        pytest.skip("reference peer does not compile here: " + proc.stderr[-300:])
    return BIN


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def plain_context(name):
    ctx = tpb.Context(name)
    ctx.register_transport(0, "uv", tpb._C.create_uv_transport())
    ctx.register_channel(0, "basic", tpb._C.create_basic_channel())
    return ctx


def full_context(name):
    """Everything default_context() registers for CPU tensors (shm and uv; basic, cma, xth, mpt_uv):
    only uv and basic are really shared with the reference peer (which registers uv, shm, basic, cma,
    mpt_uv), and the negotiation has to find that out."""
    return tpb.default_context(name, cuda=False, mpt_lanes=3)


@pytest.mark.parametrize("full", [False, True], ids=["uv+basic", "every backend registered"])
def test_our_client_against_reference_server(built, full):
    peer = build_peer()
    port = free_port()
    server = subprocess.Popen([peer, "server", str(port)] + (["full"] if full else []), stdin=subprocess.PIPE,
                              stdout=subprocess.PIPE, text=True)
    try:
        line = server.stdout.readline()
        assert line.startswith("listening"), line
        ctx = full_context("ours") if full else plain_context("ours")
        pipe = ctx.connect(f"uv://127.0.0.1:{port}", remote_name="ref-server")
        for i in range(5):
            tensors = [torch.randn(1000 * (i + 1)), torch.arange(17 + i, dtype=torch.int64)]
            payloads = [bytes([i]) * (10 + i), b""]
            targets = ["cpu:0", None] if i % 2 else None  # with and without the descriptor-reply round trip
            sent = pipe.send(tensors, payloads, f"msg-{i}".encode(), target_devices=targets)
            echo = pipe.recv().result(30)
            sent.result(30)
            assert echo.metadata == f"msg-{i}".encode()
            assert [bytes(p) for p in echo.payloads] == payloads
            assert all(torch.equal(a, b) for a, b in zip(echo.tensors, tensors))
        pipe.close()
        ctx.join()
    finally:
        server.stdin.close()
        server.wait(timeout=20)


@pytest.mark.parametrize("full", [False, True], ids=["uv+basic", "every backend registered"])
def test_reference_client_against_our_server(built, full):
    peer = build_peer()
    ctx = full_context("ours") if full else plain_context("ours")
    listener = ctx.listen(["uv://127.0.0.1", "shm://"] if full else ["uv://127.0.0.1"])
    stop = threading.Event()

    def serve(pipe):
        def loop():
            while not stop.is_set():
                try:
                    msg = pipe.recv().result(30)
                except Exception:
                    return
                pipe.send(msg.tensors, [bytes(p) for p in msg.payloads], msg.metadata,
                          payload_metadata=msg.payload_metadata, tensor_metadata=msg.tensor_metadata).result(30)
        threading.Thread(target=loop, daemon=True).start()

    listener.accept(lambda err, pipe: serve(pipe) if not err else None)
    addr = listener.url("uv").split("://")[1]
    out = subprocess.run([peer, "client", addr, "6"] + (["full"] if full else []), capture_output=True, text=True,
                         timeout=120)
    stop.set()
    assert out.returncode == 0 and out.stdout.strip() == "ok 6", out.stdout + out.stderr
    ctx.join()
