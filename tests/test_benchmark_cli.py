"""The two-process ping-pong CLI with the reference's flags (tensorpipe/benchmark/benchmark_pipe.cc):
a listener and a connector started as separate processes finish, verify their data and report
percentiles."""
import os
import socket
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "build", "bin", "benchmark_pipe")


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("transport,channel,address", [
    ("uv", "basic", None),
    ("shm", "cma", "shm://tpb-cli-test-{pid}"),
    ("uv", "mpt_uv", None),
])
def test_listen_and_connect_processes_complete(built, transport, channel, address):
    if address is None:
        address = f"uv://127.0.0.1:{free_port()}"
    address = address.format(pid=os.getpid())
    common = ["--transport", transport, "--channel", channel, "--address", address, "--num-round-trips", "50",
              "--num-payloads", "2", "--payload-size", "1000", "--num-tensors", "3", "--tensor-size", "100000",
              "--metadata-size", "32"]
    server = subprocess.Popen([BIN, "--mode", "listen"] + common, stderr=subprocess.PIPE, text=True)
    try:
        # The listener prints its URL once it accepts connections.
        line = server.stderr.readline()
        assert "listening on" in line, line
        client = subprocess.run([BIN, "--mode", "connect"] + common, stderr=subprocess.PIPE, text=True, timeout=120)
        assert client.returncode == 0, client.stderr
        assert "p50" in client.stderr and "# ping-pong" in client.stderr
        fields = client.stderr.strip().splitlines()[-1].split()
        assert fields[0] == "cpu" and int(fields[1]) == 32 + 2 * 1000 + 3 * 100000 and int(fields[2]) == 50
        assert server.wait(timeout=60) == 0, server.stderr.read()
    finally:
        if server.poll() is None:
            server.kill()


def test_bad_flags_are_refused(built):
    out = subprocess.run([BIN, "--mode", "sideways", "--address", "uv://127.0.0.1:1", "--num-round-trips", "1"],
                         stderr=subprocess.PIPE, text=True)
    assert out.returncode == 2 and "--mode must be listen or connect" in out.stderr


WORKLOADS = os.path.join(ROOT, "build", "bin", "pipe_workloads")


@pytest.mark.parametrize("args,key", [
    (["--workload", "cpu_pingpong", "--transport", "shm", "--channel", "cma", "--iters", "120"], "rtt_p50_us"),
    (["--workload", "cpu_pingpong", "--transport", "uv", "--channel", "mpt", "--iters", "60"], "rtt_p50_us"),
    (["--workload", "cpu_small", "--transport", "shm", "--iters", "2000"], "rtt_p50_us"),
    (["--workload", "cpu_stream", "--transport", "uv", "--bytes", "4096", "--iters", "5000"], "us_per_message"),
    (["--workload", "pipe_setup", "--transport", "shm", "--channel", "basic", "--iters", "20"],
     "connect_to_first_answer_p50_us"),
    (["--workload", "transport_pingpong", "--transport", "shm", "--iters", "2000"], "rtt_p50_us"),
])
def test_cpu_workloads_run_and_verify_their_data(built, args, key):
    """The CPU workloads that are compiled against both libraries: each forks its peers, checks
    its own data (a mismatch or a callback out of order makes it exit non-zero) and prints one
    JSON line."""
    import json
    out = subprocess.run([WORKLOADS] + args, capture_output=True, text=True, timeout=180)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "native" and "error" not in line and line[key] > 0
