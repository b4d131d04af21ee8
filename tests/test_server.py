"""End-to-end checks of the batching server with its CPU stand-in model (no GPU): protocol,
fragmentation, cancellation, limits, back-pressure, several workers.  Cases follow the reference's
server/tests/test_e2e.py:29-101 and server/tests/test_protocol.py:10-45."""
import asyncio
import json
import socket
import struct
import subprocess
import time

import pytest

from tinyinfer_b200.server import binary, loadgen, protocol


def expected_tokens(prompt, count):
    """The CPU stand-in: next = (last + cached_length + 1) mod 50257 (reference model.hpp:70-75)."""
    out, last, length = [], prompt[-1], len(prompt)
    for _ in range(count):
        nxt = (last + length + 1) % 50257
        out.append(nxt)
        last, length = nxt, length + 1
    return out


class Server:
    def __init__(self, *flags):
        from tinyinfer_b200 import build
        build.build()
        with socket.socket() as probe:
            probe.bind(("127.0.0.1", 0))
            self.port = probe.getsockname()[1]
        self.proc = subprocess.Popen([str(binary()), "--model", "cpu", "--port", str(self.port), *map(str, flags)],
                                     stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
        line = self.proc.stdout.readline()
        self.ready = json.loads(line)
        assert self.ready["ready"] is True and self.ready["port"] == self.port

    def connect(self):
        sock = socket.create_connection(("127.0.0.1", self.port), timeout=10)
        sock.settimeout(10)
        return sock

    def close(self):
        self.proc.terminate()
        try:
            _, err = self.proc.communicate(timeout=10)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            _, err = self.proc.communicate()
        return err

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.close()


def collect(sock, finals):
    """Reads frames until `finals` FINAL responses arrived; returns (firsts, finals) keyed by id."""
    first, final = {}, {}
    while len(final) < finals:
        reply = protocol.recv_response(sock)
        (first if reply["kind"] == protocol.FIRST else final)[reply["id"]] = reply
    return first, final


def test_protocol_layout_and_limits():
    frame = protocol.request(7, [1, 2, 3], 4)
    assert struct.unpack("!I", frame[:4])[0] == 20 + 12 and frame[4:8] == b"\x00\x01\x00\x01"
    assert protocol.cancellation(9)[4:] == protocol.REQUEST.pack(1, 2, 9, 0, 0)
    for bad in (lambda: protocol.request(0, [1], 1), lambda: protocol.request(1, [], 1), lambda: protocol.request(1, [50257], 1),
                lambda: protocol.request(1, [1] * 1000, 25), lambda: protocol.request(1, [True], 1), lambda: protocol.cancellation(2 ** 64)):
        with pytest.raises(ValueError):
            bad()
    body = protocol.RESPONSE.pack(1, protocol.FINAL, 5, 0, 2, 64, 0, 1, 2, 3, 4) + struct.pack("!2I", 10, 11)
    assert protocol.decode_response(body)["tokens"] == [10, 11]
    with pytest.raises(ValueError):
        protocol.decode_response(protocol.RESPONSE.pack(1, protocol.FINAL, 5, 0, 0, 65, 0, 0, 0, 0, 0))
    with pytest.raises(ValueError):
        protocol.decode_response(protocol.RESPONSE.pack(1, protocol.FIRST, 5, 0, 0, 1, 0, 0, 0, 0, 0))


def test_workload_is_deterministic_and_bounded():
    a, b = loadgen.workload(4, 50.0, 200), loadgen.workload(4, 50.0, 200)
    assert a == b and a != loadgen.workload(4, 60.0, 200)
    assert all(8 <= len(p) <= 900 and 1 <= n <= 256 and len(p) + n <= 1024 for _, _, p, n in a)
    assert all(x[0] < y[0] for x, y in zip(a, a[1:])) and [x[1] for x in a] == list(range(1, 201))
    assert loadgen.percentile([10, 0, 20], 50) == 10 and loadgen.percentile([0, 10], 95) == 9.5
    for bad in ([], [float("nan")], [-1.0]):
        with pytest.raises(ValueError):
            loadgen.percentile(bad, 50)


def test_generate_fragmented_and_coalesced_frames():
    with Server("--max-batch", 4, "--max-wait-us", 2000, "--send-chunk-bytes", 7) as server:
        sock = server.connect()
        prompts = {1: ([3, 4, 5], 3), 2: ([9], 2), 3: ([100, 200], 1)}
        stream = b"".join(protocol.request(i, p, n) for i, (p, n) in prompts.items())
        for byte in stream[:25]:                       # byte by byte, then the rest in one piece
            sock.sendall(bytes([byte]))
        sock.sendall(stream[25:])
        first, final = collect(sock, 3)
        for i, (p, n) in prompts.items():
            want = expected_tokens(p, n)
            assert final[i]["status"] == 0 and final[i]["tokens"] == want and first[i]["tokens"] == want[:1]
            assert 1 <= final[i]["batch_size"] <= 4
        assert expected_tokens([3, 4, 5], 3) == [9, 14, 20]
        sock.close()


def test_invalid_frames_close_only_that_connection():
    with Server() as server:
        good = server.connect()
        for payload in (struct.pack("!I", 5), struct.pack("!I", 10 ** 6), protocol.request(1, [1], 1)[:4] + b"\x00\x02" + protocol.request(1, [1], 1)[6:]):
            bad = server.connect()
            bad.sendall(payload)
            assert bad.recv(16) == b""                  # closed without a reply
            bad.close()
        dup = server.connect()
        dup.sendall(protocol.request(5, [1], 1) + protocol.request(5, [2], 1))
        seen = b""
        while True:
            piece = dup.recv(4096)
            if not piece:
                break
            seen += piece
        dup.close()
        good.sendall(protocol.request(1, [7, 8], 2))
        _, final = collect(good, 1)
        assert final[1]["tokens"] == expected_tokens([7, 8], 2)
        good.close()


def test_cancellation_and_id_reuse_across_connections():
    with Server("--max-batch", 1, "--max-wait-us", 0, "--max-new-tokens", 1000) as server:
        sock = server.connect()
        sock.sendall(protocol.request(1, [5], 1000) + protocol.request(2, [6], 1000) + protocol.cancellation(2) + protocol.cancellation(77))
        _, final = collect(sock, 2)
        assert final[2]["status"] == 3 and final[2]["tokens"] == []
        assert final[1]["status"] in (0, 3)
        other = server.connect()
        other.sendall(protocol.request(1, [5, 6], 2))     # the same id on another connection is a new request
        _, again = collect(other, 1)
        assert again[1]["tokens"] == expected_tokens([5, 6], 2)
        sock.close(); other.close()


def test_overload_reply_and_output_backpressure():
    with Server("--max-pending", 1, "--per-connection", 1, "--max-batch", 1, "--max-wait-us", 200000) as server:
        sock = server.connect()
        sock.sendall(protocol.request(1, [1], 4) + protocol.request(2, [1], 4))
        _, final = collect(sock, 2)
        assert final[2]["status"] == 2 and final[1]["status"] == 0
        sock.close()
    with Server("--max-output-bytes", 64) as server:      # one FIRST frame (64 bytes) fits, FIRST + FINAL do not
        sock = server.connect()
        sock.sendall(protocol.request(1, [1], 8))
        data = b""
        while True:
            piece = sock.recv(4096)
            if not piece:
                break
            data += piece
        assert len(data) <= 64
        sock.close()


def test_several_workers_share_the_load_and_loadgen_runs():
    with Server("--devices", "0,1,2", "--max-batch", 8, "--max-wait-us", 500, "--max-new-tokens", 256, "--max-pending", 512,
                "--max-connections", 600) as server:
        assert server.ready["devices"] == [0, 1, 2]
        summary = asyncio.run(loadgen.run("127.0.0.1", server.port, rate=400.0, count=120, seed=4, outstanding=256, timeout=30))
        assert summary["completed"] == 120 and summary["failed"] == 0 and summary["tokens_per_s"] > 0
        assert summary["per_output_token_ms"]["p50"] >= 0 and summary["generated_tokens"] == sum(n for _, _, _, n in loadgen.workload(4, 400.0, 120))
        sock = server.connect()
        items = loadgen.workload(4, 400.0, 6)
        sock.sendall(b"".join(protocol.request(i, p, n) for _, i, p, n in items))
        _, final = collect(sock, 6)
        for _, i, p, n in items:
            assert final[i]["tokens"] == expected_tokens(p, n)
        sock.close()
    err = server.close()


@pytest.mark.parametrize("group", [1, 3, 4])
def test_grouped_admission_serves_every_request(group):
    """`--admit-batch n`: a busy worker waits for n free slots (or for as many as there are requests waiting) before it
    admits; whatever n, every request is served with the tokens the model function gives."""
    with Server("--max-batch", 4, "--admit-batch", group, "--max-wait-us", 200, "--max-new-tokens", 64, "--max-pending", 512) as server:
        sock = server.connect()
        items = loadgen.workload(4, 400.0, 23)
        sock.sendall(b"".join(protocol.request(i, p, min(n, 64)) for _, i, p, n in items))
        _, final = collect(sock, 23)
        for _, i, p, n in items:
            assert final[i]["status"] == 0 and final[i]["tokens"] == expected_tokens(p, min(n, 64))
        sock.close()
    server.close()


def test_a_device_listed_twice_carries_two_replicas():
    """`--devices 0,0`: two workers (own model context each) on one device, both serving."""
    with Server("--devices", "0,0", "--max-batch", 2, "--max-wait-us", 500, "--max-new-tokens", 64, "--max-pending", 512) as server:
        assert server.ready["devices"] == [0, 0]
        sock = server.connect()
        items = loadgen.workload(4, 400.0, 12)
        sock.sendall(b"".join(protocol.request(i, p, min(n, 64)) for _, i, p, n in items))
        _, final = collect(sock, 12)
        for _, i, p, n in items:
            assert final[i]["status"] == 0 and final[i]["tokens"] == expected_tokens(p, min(n, 64))
        sock.close()
    server.close()


@pytest.mark.parametrize("sanitizer", [[], ["-fsanitize=thread"]], ids=["plain", "tsan"])
def test_mpsc_queue_with_real_threads(tmp_path, sanitizer):
    from tinyinfer_b200.build import SRC
    exe = tmp_path / "mpsc_check"
    source = str(__import__("pathlib").Path(__file__).with_name("mpsc_check.cpp"))
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-pthread", *sanitizer, f"-I{SRC / 'server'}", source, "-o", str(exe)],
                           capture_output=True, text=True)
    if build.returncode and sanitizer:
        pytest.skip("thread sanitizer runtime unavailable: " + build.stderr[-200:])
    assert build.returncode == 0, build.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    if sanitizer and "FATAL: ThreadSanitizer" in run.stderr:
        pytest.skip("thread sanitizer cannot run in this environment")
    assert run.returncode == 0 and run.stdout.strip() == "ok", run.stdout + run.stderr


def test_a_failing_worker_answers_internal_and_the_other_worker_keeps_serving():
    """Reference behaviour for a failed native call (server/src/main.cpp:151-156): everything outstanding on that worker
    and everything it receives later is answered `internal`, the process stays up.  With several workers the router
    then prefers the healthy ones.  The failure is injected on the host (test hook --fail-after-steps)."""
    with Server("--devices", "0,1", "--max-batch", 4, "--fail-worker", 0, "--fail-after-steps", 3) as server:
        sock = server.connect()
        prompts = {i: [100 + i, 200 + i, 300 + i] for i in range(1, 9)}
        for i, prompt in prompts.items():
            sock.sendall(protocol.request(i, prompt, 6))
        _, final = collect(sock, len(prompts))
        failed = sorted(i for i, r in final.items() if r["status"] == protocol.INTERNAL)
        served = sorted(i for i, r in final.items() if r["status"] == protocol.OK)
        assert failed and served and len(failed) + len(served) == len(prompts)
        for i in served:
            assert final[i]["tokens"] == expected_tokens(prompts[i], 6)
        for i in failed:
            assert final[i]["tokens"] == []
        # later requests: the healthy worker serves them all
        for i in range(20, 30):
            sock.sendall(protocol.request(i, [i, i + 1], 4))
        _, later = collect(sock, 10)
        assert all(r["status"] == protocol.OK and r["tokens"] == expected_tokens([i, i + 1], 4) for i, r in later.items())
        sock.close()
        err = server.close()
    assert "model_poisoned: device 0" in err


def test_a_single_failing_worker_answers_internal_from_then_on():
    with Server("--max-batch", 2, "--fail-after-steps", 2) as server:
        sock = server.connect()
        sock.sendall(protocol.request(1, [5, 6, 7], 8))
        _, final = collect(sock, 1)
        assert final[1]["status"] == protocol.INTERNAL
        sock.sendall(protocol.request(2, [9], 2))
        _, final = collect(sock, 1)
        assert final[2]["status"] == protocol.INTERNAL and final[2]["tokens"] == []
        sock.close()
