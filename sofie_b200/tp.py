"""Tensor-parallel column split of one large Gemm: contraction and all-gather in one kernel.

The reference runs one Session per device (core/src/RModel_ALPAKA.cxx:1123-1132) and never splits an operator; this is
the optional next step after replicas for a Gemm whose weight should not be held whole by every GPU.  Rank r keeps the
rows [n0, n0 + n) of the K-major weight W[N, K] (the columns of Y = A · Wᵀ), computes Y[:, n0:n0+n] with the tcgen05
kernel, and the kernel's epilogue stores every finished row segment into the full-width result of EVERY rank
(sofie_b200_gemm_enqueue_peers: one bulk tensor store per destination, plain peer stores over NVLink, no multicast).
When all ranks' kernels are done each rank holds the whole Y; what remains of the collective is one barrier.

One process per GPU; the other ranks' results are reached through CUDA IPC (sofie_b200_peer_export / _open), the
handles travel through torch.distributed (any backend).  The results come from torch's caching allocator, which must
hand out cudaMalloc memory (its default; `expandable_segments` blocks cannot be exported).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.distributed as dist

from . import lib as L
from .ops import Context, GemmPlan
from .replicas import shard_range

MAX_PEERS = 7   # sofie_b200_gemm_enqueue_peers: n_peers 0..7
QUANTUM = 64   # columns: the epilogue stores whole row segments (128 bytes of bf16), so a shard is whole groups of 64 columns


def column_shard(n_total: int, rank: int, world: int, quantum: int = QUANTUM) -> tuple[int, int]:
    """(first column, columns) of `rank`: contiguous whole quanta, sizes differing by at most one quantum."""
    if n_total % quantum:
        raise ValueError(f"{n_total} columns are not whole groups of {quantum}")
    q0, q1 = shard_range(n_total // quantum, rank, world)
    return q0 * quantum, (q1 - q0) * quantum


def exchange(mine, group=None) -> list:
    """Every rank's `mine` (any picklable object), in rank order."""
    world = dist.get_world_size(group)
    out = [None] * world
    dist.all_gather_object(out, mine, group=group)
    return out


class PeerTable:
    """Where this rank's columns start inside every OTHER rank's result buffers.

    `opened[r][b]` is the device pointer (valid in this process) to buffer b of rank r, None for this rank itself."""

    def __init__(self, opened: Sequence[Sequence[Optional[int]]], rank: int, column_offset_bytes: int):
        self.rank = rank
        self.buffers = len(opened[rank]) if opened else 0
        self._ptrs = []
        for b in range(self.buffers):
            self._ptrs.append([opened[r][b] + column_offset_bytes for r in range(len(opened)) if r != rank])

    def peers(self, turn: int) -> list[int]:
        """Destinations of call number `turn`: the calls walk round the buffers, so that a rank may still be reading the
        previous call's result while the others already write the next one."""
        return self._ptrs[turn % self.buffers]


class ColumnParallelGemm:
    """Y[M, n_total] = epilogue(A[M, K] · W[n_total, K]ᵀ) with W split by rows (Y's columns) over the ranks of `group`.

    __call__(a, w_shard, epilogue) takes this rank's weight rows and an epilogue whose column vectors (col_scale, bias)
    are this rank's slices; it returns this rank's full-width result, valid on return.  Results rotate over `buffers`
    (>= 2) tensors owned by the object: the one returned stays untouched until `buffers - 1` further calls have been
    made, and work that reads it must be enqueued on `ctx`'s stream (the next call waits for that stream before the
    ranks meet)."""

    def __init__(self, ctx: Context, M: int, n_total: int, K: int, ab_dtype, y_dtype, group=None, buffers: int = 2,
                 wide_stores: bool = True):
        if buffers < 2:
            raise ValueError("at least two result buffers")
        self.ctx, self.group = ctx, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > MAX_PEERS + 1:
            raise ValueError(f"at most {MAX_PEERS + 1} ranks")
        self.n0, self.n = column_shard(n_total, self.rank, self.world)
        if self.n == 0:
            raise ValueError("fewer groups of 64 columns than ranks")
        dev = torch.device("cuda", ctx.device)
        self.results = [torch.empty((M, n_total), dtype=y_dtype, device=dev) for _ in range(buffers)]
        self._ys = self.results[0].element_size()
        # 128-byte row segments: NVLink carries them at 700 GB/s, scattered 64-byte ones at about 410 GB/s
        self.plan = GemmPlan(ctx, M, self.n, K, ab_dtype, y_dtype, trans_b=True, ldy=n_total,
                             flags=L.GEMM_WIDE_STORES if wide_stores else 0)
        handles = exchange([ctx.peer_export(t) for t in self.results], group)
        self._opened = [[None if r == self.rank else ctx.peer_open(h) for h in handles[r]] for r in range(self.world)]
        self._table = PeerTable(self._opened, self.rank, self.n0 * self._ys)
        self._turn = 0
        dist.barrier(group)   # nobody stores before every rank has its buffers

    def enqueue(self, a: torch.Tensor, w_shard: torch.Tensor, epilogue: Optional[L.Epilogue] = None) -> torch.Tensor:
        """Only the kernel; the result is complete after finish()."""
        y = self.results[self._turn % len(self.results)]
        self.plan.enqueue_peers(a, w_shard, y.data_ptr() + self.n0 * self._ys, self._table.peers(self._turn), epilogue)
        self._turn += 1
        return y

    def finish(self) -> None:
        """Waits for this rank's kernel (its stores into the peers included), then for every other rank's."""
        self.ctx.sync()
        dist.barrier(self.group)

    def __call__(self, a, w_shard, epilogue=None) -> torch.Tensor:
        y = self.enqueue(a, w_shard, epilogue)
        self.finish()
        return y

    def close(self) -> None:
        if getattr(self, "_opened", None):
            self.ctx.sync()
            dist.barrier(self.group)   # no rank closes a mapping while another still stores through its own
            for row in self._opened:
                for p in row:
                    if p is not None:
                        self.ctx.peer_close(p)
            self._opened = None
            self.plan.close()
            dist.barrier(self.group)   # ... and the owners free only after everybody has closed
            self.results = []

