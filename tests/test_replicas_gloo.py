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
