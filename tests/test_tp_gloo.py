"""Host logic of the column split (shards, handle exchange, destination table) on two CPU processes over gloo."""
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


def _worker(rank, world, port, n_total, q):
    sys.path.insert(0, str(ROOT))
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from sofie_b200 import replicas, tp
    rep = replicas.init_from_env("gloo")
    n0, n = tp.column_shard(n_total, rank, world)
    # stand-ins for exported handles: each rank "exports" two buffers whose addresses encode (rank, buffer)
    handles = tp.exchange([bytes([rank, b]) for b in range(2)])
    opened = [[None if r == rank else 1_000_000 * (h[0] + 1) + 1000 * h[1] for h in handles[r]] for r in range(world)]
    table = tp.PeerTable(opened, rank, n0 * 2)
    q.put((rank, n0, n, [table.peers(t) for t in range(3)]))
    replicas.shutdown(rep)


def test_two_ranks_exchange_handles_and_aim_at_their_own_columns():
    world, port, n_total = 2, _free_port(), 2048 + 64
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_total, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (_, a0, an, peers0), (_, b0, bn, peers1) = out
    assert a0 == 0 and b0 == an and an + bn == n_total and an % 64 == 0 and bn % 64 == 0 and abs(an - bn) <= 64
    # rank 0 stores into rank 1's buffers (base 2_000_000) at its own column offset 0; the calls alternate the buffers
    assert peers0 == [[2_000_000], [2_001_000], [2_000_000]]
    assert peers1 == [[1_000_000 + 2 * b0], [1_001_000 + 2 * b0], [1_000_000 + 2 * b0]]


def test_column_shards_are_whole_groups_of_64():
    from sofie_b200.tp import column_shard
    for n_total in (64, 512, 2048, 8192 + 64):
        for world in (1, 2, 3, 8):
            spans = [column_shard(n_total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and sum(n for _, n in spans) == n_total
            assert all(spans[i][0] + spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert all(n % 64 == 0 for _, n in spans) and max(n for _, n in spans) - min(n for _, n in spans) <= 64
    with pytest.raises(ValueError):
        column_shard(100, 0, 2)
