"""Native batching server on a GPU: tokens over the socket equal direct NativeModel.greedy tokens
(the reference's socket gate, server/tests/native_correctness.py:417-494)."""
import json
import socket
import subprocess

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def test_socket_tokens_equal_direct_greedy(tmp_path_factory):
    from tinyinfer_b200 import artifact
    from tinyinfer_b200.runtime import NativeModel
    from tinyinfer_b200.server import binary, protocol
    manifest = artifact.write_synthetic(tmp_path_factory.mktemp("srv_art"), seed=0)
    rng = np.random.default_rng(11)
    cases = [(rng.integers(0, 50257, n).tolist(), m) for n, m in ((33, 6), (5, 9), (120, 3), (17, 1), (64, 12))]
    with NativeModel(None, manifest, max_batch=8, cache_slots=8, capacity=256) as model:
        want = [model.greedy([p], m, slots=[0])["tokens"][0] if not model.reset(0) else None for p, m in cases]
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    proc = subprocess.Popen([str(binary()), "--model", "native", "--manifest", str(manifest), "--port", str(port), "--max-batch", "8",
                             "--capacity", "256", "--max-wait-us", "20000", "--devices", "0"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        ready = json.loads(proc.stdout.readline())
        assert ready["ready"] and ready["model"] == "native"
        sock = socket.create_connection(("127.0.0.1", port), timeout=60)
        sock.settimeout(60)
        # all at once (batched, admitted together), then the same requests again in reverse (slot reuse, continuous admission)
        for round_ids in (range(1, 6), range(10, 5, -1)):
            ids = list(round_ids)
            order = list(range(5)) if ids[0] == 1 else list(range(4, -1, -1))
            sock.sendall(b"".join(protocol.request(i, cases[c][0], cases[c][1]) for i, c in zip(ids, order)))
            final, first = {}, {}
            while len(final) < 5:
                reply = protocol.recv_response(sock)
                (first if reply["kind"] == protocol.FIRST else final)[reply["id"]] = reply
            for i, c in zip(ids, order):
                assert final[i]["status"] == 0 and final[i]["tokens"] == want[c], (i, c)
                assert first[i]["tokens"] == want[c][:1]
            assert max(f["batch_size"] for f in final.values()) >= 2
        sock.close()
    finally:
        proc.terminate()
        _, err = proc.communicate(timeout=60)
    trace = [json.loads(line) for line in err.splitlines() if line.startswith("{")]
    assert trace and trace[-1]["native_trace_status"] == 0 and trace[-1]["gemm_int8"] > 0 and trace[-1]["attention"] > 0
