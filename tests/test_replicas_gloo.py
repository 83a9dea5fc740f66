"""The N > 1 host logic on CPU: two gloo ranks, batch sharding and the slowest-rank throughput rule."""
import os
import socket

import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

from darknet_b200 import replicas  # noqa: E402


def test_shard_batch_covers_every_image_once():
    assert replicas.shard_batch(256, 8) == [(32 * r, 32) for r in range(8)]
    assert replicas.shard_batch(10, 4) == [(0, 3), (3, 3), (6, 2), (8, 2)]
    assert replicas.shard_batch(2, 4) == [(0, 1), (1, 1), (2, 0), (2, 0)]
    assert replicas.shard_batch(0, 2) == [(0, 0), (0, 0)]
    with pytest.raises(ValueError):
        replicas.shard_batch(4, 0)


def test_single_process_is_identity():
    assert replicas.max_over_ranks(3.5) == 3.5
    assert replicas.aggregate_images_per_s(100, 50.0) == pytest.approx(2000.0)


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank: int, world: int, port: int, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        first, count = replicas.shard_batch(7, world)[rank]
        ms = 10.0 if rank == 0 else 25.0                       # rank 1 is the slow one
        slowest = replicas.max_over_ranks(ms)
        total = replicas.aggregate_images_per_s(count, ms)
        dist.barrier()
        out.put((rank, first, count, slowest, total))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_report_the_slowest_rank_time():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [(r[1], r[2]) for r in results] == [(0, 4), (4, 3)]
    for r in results:
        assert r[3] == 25.0
        assert r[4] == pytest.approx(7 / 0.025)
