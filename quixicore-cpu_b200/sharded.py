"""Row (output-channel) sharding of a packed weight matrix over the ranks of one node.

Every output element depends on one weight row and one activation row, so the weights
shard by rows with no reduction crossing a shard (the reference partitions rows over its
threads in the same way, src/threading/thread_pool.cpp:22-29). Rank r keeps the
contiguous row range ``shard_rows(n, world, r)`` of the canonical ``[n][k/32]`` block
array, activations are replicated, and the output slices are exchanged with one
all-gather (semantics of ``all_gather`` in kernels/collectives/collectives_ref.cpp:26-37).

The compute step is injected: on GPUs it is ``PackedWeights.qgemm_dev`` of this package;
the CPU tests run the same host logic over gloo with a stand-in compute function.
"""

from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

TILE = 128  # prepared panels are tiles of 128 rows: keep shard boundaries on tiles


def shard_rows(n: int, world: int, rank: int, align: int = TILE) -> Tuple[int, int]:
    """(first row, row count) of rank's shard: contiguous, in rank order, covering [0, n).
    Boundaries fall on multiples of `align` where n allows it."""
    if world < 1 or not 0 <= rank < world or n < 1:
        raise ValueError("bad shard request")
    units = (n + align - 1) // align
    begin = min(n, (units * rank // world) * align)
    end = min(n, (units * (rank + 1) // world) * align)
    return begin, end - begin


class ShardedLinear:
    """y[m, n] = x[m, k] . dequant(W)^T with W's rows sharded over the process group.

    compute(x [m, k], out) fills this rank's slice: `out` is a [m, rows_local] view whose
    row stride (out.stride(0)) may exceed rows_local. forward() returns the full y on every
    rank.
    """

    def __init__(self, n: int, k: int, compute: Callable[[torch.Tensor, torch.Tensor], None],
                 group: Optional[dist.ProcessGroup] = None, device: str = "cpu"):
        self.n, self.k = n, k
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.begin, self.rows = shard_rows(n, self.world, self.rank)
        self.ranges = [shard_rows(n, self.world, r) for r in range(self.world)]
        self.max_rows = max(rows for _, rows in self.ranges)
        self.uniform = all(rows == self.max_rows for _, rows in self.ranges)
        self.compute = compute
        self.device = device

    def forward(self, x: torch.Tensor, y: Optional[torch.Tensor] = None) -> torch.Tensor:
        m = x.shape[0]
        if y is None:
            y = torch.empty((m, self.n), dtype=torch.float32, device=self.device)
        if self.world == 1:
            self.compute(x, y)
            return y
        if m == 1 and self.uniform:
            # contiguous slices: compute in place and gather straight into y
            local = y[0, self.begin:self.begin + self.rows]
            self.compute(x, local.view(1, self.rows))
            dist.all_gather_into_tensor(y.view(-1), local, group=self.group)
            return y
        # strided or uneven slices: gather [world][m][max_rows], then place the columns
        local = torch.zeros((m, self.max_rows), dtype=torch.float32, device=self.device)
        self.compute(x, local[:, :self.rows])
        gathered = torch.empty((self.world, m, self.max_rows), dtype=torch.float32,
                               device=self.device)
        dist.all_gather_into_tensor(gathered.view(self.world * m, self.max_rows), local,
                                    group=self.group)
        for r, (begin, rows) in enumerate(self.ranges):
            y[:, begin:begin + rows] = gathered[r, :, :rows]
        return y


class PushAllGather:
    """Row-sharded decode with the all-gather fused into the GEMV kernel (peer stores over
    NVLink instead of a collective call): one instance per rank, built collectively.

    Each rank allocates a result buffer [2][world][m][rows] and a peer-mappable inbox of the
    same shape (8-byte cells) through the C library, the 64-byte inbox handles travel through
    the process group (all_gather_object), and every rank maps the others'. step() enqueues
    the GEMV and the receive of all other slices and returns the device address of the
    step's [world][m][rows] results.
    """

    def __init__(self, qx, rows_per_rank: int, max_m: int = 1,
                 group: Optional[dist.ProcessGroup] = None):
        self.qx = qx
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.rows, self.max_m = rows_per_rank, max_m
        result_bytes = 2 * self.world * max_m * rows_per_rank * 4
        self.results, _ = qx.peer_alloc(result_bytes)
        self.inbox, inbox_handle = qx.peer_alloc(qx.push_inbox_bytes(self.world, max_m, rows_per_rank))
        handles = [None] * self.world
        dist.all_gather_object(handles, inbox_handle, group=group)
        plan = qx.PushPlan()
        plan.world, plan.rank, plan.rows_per_rank = self.world, self.rank, rows_per_rank
        plan.results_local, plan.inbox_local = self.results, self.inbox
        for r, handle in enumerate(handles):
            if r != self.rank:
                plan.inbox_peer[r] = qx.peer_open(handle)
        self.plan = plan
        self.steps = 0
        dist.barrier(group=group)  # every rank has mapped every inbox before anyone pushes

    def step(self, weights, x, m: int = 1) -> int:
        if m != self.max_m:
            raise ValueError("the buffers are laid out for max_m rows per step")
        self.steps += 1
        self.qx.check(self.qx.qgemm_push_dev(weights, x, m, self.plan, self.steps),
                      "qx_qgemm_prepacked_push_dev")
        return self.qx.allgather_wait_dev(self.plan, m, self.steps)
