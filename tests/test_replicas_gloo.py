"""The multi-rank host logic (sharding, barrier, max-over-ranks timing) on two CPU processes over gloo."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total, q):
    sys.path.insert(0, str(ROOT))
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from sofie_b200 import replicas
    rep = replicas.init_from_env("gloo")
    begin, end = replicas.shard_range(total, rep.rank, rep.world)
    replicas.barrier(rep)
    slowest = replicas.max_over_ranks(rep, 10.0 + rank)          # rank r "took" 10+r ms
    units = replicas.sum_over_ranks(rep, float(end - begin))
    q.put((rank, begin, end, slowest, units, rep.is_root))
    replicas.shutdown(rep)


@pytest.mark.parametrize("total", [512, 7])
def test_two_replicas_share_the_batch_and_report_the_slowest(total):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, total, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, b0, e0, slow0, units0, root0), (r1, b1, e1, slow1, units1, root1) = out
    assert (b0, e1) == (0, total) and e0 == b1 and abs((e0 - b0) - (e1 - b1)) <= 1   # contiguous, balanced cover
    assert slow0 == slow1 == 11.0                                                     # the slower rank's time everywhere
    assert units0 == units1 == float(total)
    assert root0 and not root1


def test_shard_range_properties():
    from sofie_b200.replicas import shard_range
    for total in (0, 1, 5, 512, 1001):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 4, 4)
