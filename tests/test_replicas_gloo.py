"""World-size-2 gloo run of the replica bookkeeping used by the multi-GPU benchmark."""
import os
import socket

import pytest

torch = pytest.importorskip("torch")


def _worker(rank, world, port, out):
    import torch.distributed as dist
    from tinyinfer_b200 import replicas
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mine = replicas.shard(range(10), rank, world)
    dist.barrier()
    units, seconds, rate = replicas.job_throughput(len(mine) * 100, 1.0 + rank, dist)
    out.put((rank, mine, units, seconds, rate))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_agree_on_shards_and_job_throughput():
    import torch.multiprocessing as mp
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results[0][1] == [0, 2, 4, 6, 8] and results[1][1] == [1, 3, 5, 7, 9]
    for _, _, units, seconds, rate in results:
        assert units == 1000 and seconds == 2.0 and rate == 500.0       # sum of units, slowest rank's time


def test_single_process_passthrough():
    from tinyinfer_b200 import replicas
    assert replicas.job_throughput(64, 0.5) == (64, 0.5, 128.0)
    with pytest.raises(ValueError):
        replicas.shard([1], 2, 2)


def _server_worker(rank, world, port, out):
    import sys
    from pathlib import Path
    import torch.distributed as dist
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    import bench
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    record = bench.server_record(None, dist, rank, world, None, "cpu", 300, 3000.0)
    out.put((rank, record))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_share_one_server_and_one_request_stream():
    """The multi-GPU serving measurement of bench.py on CPU: rank 0 starts one server with two workers (the protocol
    stand-in model), both ranks play half of the request stream, the totals are summed on rank 0."""
    import torch.multiprocessing as mp
    from tinyinfer_b200 import build
    from tinyinfer_b200.server import loadgen
    build.build()
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_server_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(out.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results[1] is None                                   # only rank 0 holds the merged record
    record = results[0]
    expected_tokens = sum(new for _, _, _, new in loadgen.workload(4, 3000.0, 300))
    assert record["completed"] == 300 and record["generated_tokens"] == expected_tokens
    assert record["gpus"] == 2 and record["load_generators"] == 2 and record["tokens_per_s"] > 0
    assert record["per_output_token_ms"]["p99"] >= record["per_output_token_ms"]["p50"] >= 0
