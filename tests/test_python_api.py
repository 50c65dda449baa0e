"""Python API tests: torch-tensor messages over CPU channels here, CUDA channels under -m gpu.
(The reference's only Python test is a CPU read/write, tensorpipe/test/python/tensorpipe.py:14-83.)"""
import threading

import pytest
import torch

import tensorpipe_b200 as tpb


def connected_pair(**kw):
    a = tpb.default_context("a", **kw)
    b = tpb.default_context("b", **kw)
    listener = a.listen(["uv://127.0.0.1", "shm://"])
    fut = listener.accept_future()
    out_pipe = b.connect(listener.url("uv"), remote_name="a")
    in_pipe = fut.result(30)
    return a, b, listener, out_pipe, in_pipe


def test_cpu_message_round_trip(built):
    a, b, listener, out_pipe, in_pipe = connected_pair(cuda=False)
    x = torch.randn(1000, 10)
    y = torch.arange(12).reshape(3, 4).t()  # non-contiguous: made contiguous on the way
    sent = out_pipe.send([x, y], payloads=[b"hello", bytearray(b"xyz")], metadata=b"meta")
    msg = in_pipe.recv().result(30)
    sent.result(30)
    assert msg.metadata == b"meta"
    assert [bytes(p) for p in msg.payloads] == [b"hello", b"xyz"]
    assert torch.equal(msg.tensors[0], x) and torch.equal(msg.tensors[1], y)
    assert in_pipe.remote_name == "b" and out_pipe.remote_name == "a"
    stats = a.stats()
    assert stats["messages_read"] == 1 and stats["tensor_bytes_received"] == x.numel() * 4 + 12 * 8
    a.join()
    b.join()


def test_callbacks_are_ordered_and_errors_reach_python(built):
    a, b, listener, out_pipe, in_pipe = connected_pair(cuda=False)
    order = []
    done = threading.Event()
    n = 20
    for i in range(n):
        def cb(err, i=i):
            order.append((i, err))
            if len(order) == n:
                done.set()
        out_pipe.write(tpb.Message([torch.full((100,), float(i))]), cb)
    for i in range(n):
        msg = in_pipe.recv().result(30)
        assert float(msg.tensors[0][0]) == float(i)
    assert done.wait(30)
    assert order == [(i, "") for i in range(n)]
    # After close every pending callback fires with an error string.
    fut = in_pipe.recv()
    in_pipe.close()
    with pytest.raises(RuntimeError):
        fut.result(30)
    a.join()
    b.join()


def test_deadlines_and_trace_from_python(built, tmp_path):
    from tensorpipe_b200 import _C
    trace_file = str(tmp_path / "trace.json")
    _C.trace_enable(trace_file)
    a, b, listener, out_pipe, in_pipe = connected_pair(cuda=False)
    in_pipe.set_timeouts(descriptor=0.3)
    sent = out_pipe.send([torch.ones(8)])
    assert torch.equal(in_pipe.recv().result(30).tensors[0], torch.ones(8))  # in time: unaffected
    sent.result(30)
    late = in_pipe.recv()  # nothing is ever sent again
    with pytest.raises(RuntimeError, match="timeout"):
        late.result(30)
    _C.trace_disable()
    assert _C.trace_dump()
    import json
    events = json.load(open(trace_file))
    assert {"pipe.write", "pipe.read.done"} <= {e["name"] for e in events}
    a.join()
    b.join()


def test_mpt_lanes_carry_tensors(built):
    a = tpb.Context("a")
    b = tpb.Context("b")
    for ctx in (a, b):
        ctx.register_transport(0, "uv", tpb._C.create_uv_transport())
        ctx.register_channel(0, "mpt_uv", tpb._C.create_mpt_channel(3))
    listener = a.listen(["uv://127.0.0.1"])
    fut = listener.accept_future()
    out_pipe = b.connect(listener.url("uv"))
    in_pipe = fut.result(30)
    x = torch.randn(1_000_003)
    sent = out_pipe.send([x])
    msg = in_pipe.recv().result(30)
    sent.result(30)
    assert torch.equal(msg.tensors[0], x)
    assert a.stats()["bytes_per_channel"] == {"mpt_uv": x.numel() * 4}
    a.join()
    b.join()


@pytest.mark.gpu
def test_cuda_tensors_views_and_casts(built):
    a, b, listener, out_pipe, in_pipe = connected_pair()
    x = torch.randn(513, 257, device="cuda")
    y = torch.randn(100, 64, device="cuda", dtype=torch.bfloat16).t()
    z = torch.arange(1000, device="cuda")
    sent = out_pipe.send([x, y, z], payloads=[b"p"], target_devices=["cuda:0"] * 3)
    msg = in_pipe.recv(cast={0: torch.bfloat16}).result(30)
    sent.result(30)
    torch.cuda.synchronize()
    assert torch.equal(msg.tensors[0], x.to(torch.bfloat16))
    assert torch.equal(msg.tensors[1], y)
    assert torch.equal(msg.tensors[2], z)
    assert a.stats()["bytes_per_channel"].get("cuda_p2p", 0) > 0
    assert tpb.kernel_launch_count() > 0
    a.join()
    b.join()


@pytest.mark.gpu
def test_recv_is_ordered_on_the_callers_stream_and_device(built):
    """recv() allocates on the device and orders on the stream that are current on the CALLER's
    thread, not on the library thread that sees the descriptor: work queued on that side stream
    right after the future resolves must see the data, with no synchronisation in between."""
    last = torch.cuda.device_count() - 1  # the second GPU where there is one
    a, b, listener, out_pipe, in_pipe = connected_pair()
    side = torch.cuda.Stream(device=last)
    n = 8 << 20
    for round_ in range(3):
        x = torch.full((n,), float(round_ + 1), device="cuda:0")
        torch.cuda.synchronize(0)
        with torch.cuda.device(last), torch.cuda.stream(side):
            incoming = in_pipe.recv()
            sent = out_pipe.send([x], target_devices=[f"cuda:{last}"])
            msg = incoming.result(30)
            sent.result(30)
            t = msg.tensors[0]
            assert t.device.index == last
            total = t.sum()  # queued on `side`, behind the wait the library put there
        side.synchronize()
        assert float(total) == float(n * (round_ + 1))
    # explicit output tensors on the side stream work the same way
    out = torch.zeros(n, device=f"cuda:{last}")
    x = torch.full((n,), 7.0, device="cuda:0")
    torch.cuda.synchronize()
    with torch.cuda.device(last), torch.cuda.stream(side):
        incoming = in_pipe.recv(out=[out])
        sent = out_pipe.send([x], target_devices=[f"cuda:{last}"])
        incoming.result(30)
        sent.result(30)
        total = out.sum()
    side.synchronize()
    assert float(total) == float(n * 7)
    a.join()
    b.join()


@pytest.mark.gpu
def test_smoke_entry_point(built):
    import __graft_entry__
    __graft_entry__.smoke()


def test_tensor_metadata_fast_path_agrees_with_json(built):
    import json
    from tensorpipe_b200.core import _parse_tensor_metadata
    for dtype, shape in [("float32", [1000, 10]), ("bfloat16", []), ("int64", [7]), ("uint8", [2, 3, 4, 5])]:
        ours = ('{"dtype": "%s", "shape": %s}' % (dtype, shape)).encode()  # what the sender writes
        assert _parse_tensor_metadata(ours) == (dtype, shape)
        assert _parse_tensor_metadata(json.dumps({"shape": shape, "dtype": dtype}).encode()) == (dtype, shape)
    for foreign in [b"", b"a place", b"\xff\xfe", b'{"dtype": "float32"}', b'{"dtype": "x", "shape": [1, "a"]}',
                    b'[1, 2]', b'{"dtype": 3, "shape": [1]}']:
        got = _parse_tensor_metadata(foreign)
        assert got is None or got == ("x", [1, "a"])


def test_trace_from_the_environment_is_written_at_exit(built, tmp_path):
    import json
    import os
    import subprocess
    import sys
    pattern = str(tmp_path / "trace.%p.json")
    code = (
        "import torch, tensorpipe_b200 as tpb\n"
        "a = tpb.default_context('a', cuda=False); b = tpb.default_context('b', cuda=False)\n"
        "l = a.listen(['uv://127.0.0.1']); f = l.accept_future()\n"
        "o = b.connect(l.url('uv')); i = f.result(30)\n"
        "s = o.send([torch.ones(4)]); i.recv().result(30); s.result(30)\n"
        "a.join(); b.join()\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = {**os.environ, "TPB_TRACE": pattern, "PYTHONPATH": root}
    proc = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0, proc.stderr[-2000:]
    files = [p for p in os.listdir(tmp_path) if p.startswith("trace.") and p.endswith(".json")]
    assert len(files) == 1 and "%p" not in files[0]  # the process id took the place of %p
    names = {e["name"] for e in json.load(open(tmp_path / files[0]))}
    assert {"pipe.write", "pipe.write.done", "pipe.readDescriptor", "pipe.read", "pipe.read.done"} <= names


def test_a_program_that_never_joins_exits_cleanly(built):
    """Contexts left open, a receive still pending: the interpreter's exit joins them (the pending
    future gets its error while Python can still run the callback) instead of dying in a library
    thread's destructor."""
    import os
    import subprocess
    import sys
    code = (
        "import torch, tensorpipe_b200 as tpb\n"
        "a = tpb.default_context('a', cuda=False); b = tpb.default_context('b', cuda=False)\n"
        "l = a.listen(['uv://127.0.0.1', 'shm://']); f = l.accept_future()\n"
        "o = b.connect(l.url('uv')); i = f.result(30)\n"
        "s = o.send([torch.ones(4)]); i.recv().result(30); s.result(30)\n"
        "pending = i.recv()\n"
        "pending.add_done_callback(lambda fut: print('pending ended with', type(fut.exception()).__name__, flush=True))\n"
        "print('leaving', flush=True)\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = {**os.environ, "PYTHONPATH": root}
    proc = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0, (proc.returncode, proc.stderr[-2000:])
    assert "leaving" in proc.stdout and "pending ended with RuntimeError" in proc.stdout, proc.stdout
    assert "terminate" not in proc.stderr


def test_objects_with_tensors_inside(built):
    from tensorpipe_b200 import rpc
    a, b, listener, out_pipe, in_pipe = connected_pair(cuda=False)
    obj = {"step": 7, "weights": [torch.arange(6.0).reshape(2, 3), torch.ones(4, dtype=torch.int64)],
           "nested": ("text", {"t": torch.full((3,), 2.5)})}
    sent = rpc.send_object(out_pipe, obj)
    got = rpc.recv_object(in_pipe).result(30)
    sent.result(30)
    assert got["step"] == 7 and got["nested"][0] == "text"
    assert torch.equal(got["weights"][0], obj["weights"][0]) and torch.equal(got["weights"][1], obj["weights"][1])
    assert torch.equal(got["nested"][1]["t"], torch.full((3,), 2.5))
    a.join()
    b.join()
