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


class ShardedPrefill:
    """Y[m, n] = X[m, k] . dequant(W)^T for prefill batches with W's rows sharded over the
    process group (uniform shards), the exchange overlapped with the compute.

    The activation rows are cut into chunks of `chunk_rows`. For chunk c the injected
    compute(x_chunk [mc, k], out [mc, rows_local]) fills this rank's slice (on GPUs
    ``PackedWeights.qgemm_bf16_dev``, the tensor-core GEMM); as soon as it is enqueued, the
    all-gather of that chunk runs on a second stream while the GEMM of chunk c + 1 runs on
    the first. The gathered result keeps the layout the exchange produces,
    ``[chunk][rank][row in chunk][row of the rank's shard]`` -- no pass over the output to
    re-order it; ``assemble`` copies it into a dense [m, n] matrix where a caller wants one.
    """

    def __init__(self, n: int, k: int, compute: Callable[[torch.Tensor, torch.Tensor], None],
                 chunk_rows: int = 256, group: Optional[dist.ProcessGroup] = None,
                 device: str = "cpu"):
        self.n, self.k, self.chunk = n, k, chunk_rows
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.begin, self.rows = shard_rows(n, self.world, self.rank)
        if any(shard_rows(n, self.world, r)[1] != self.rows for r in range(self.world)):
            raise ValueError("ShardedPrefill needs shards of equal size")
        self.compute = compute
        self.device = device
        self.side = torch.cuda.Stream() if str(device).startswith("cuda") else None
        self.local = self.gathered = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        m = x.shape[0]
        if m % self.chunk:
            raise ValueError("the batch must be a multiple of the chunk size")
        chunks = m // self.chunk
        if self.gathered is None or self.gathered.shape[0] != chunks:
            self.local = torch.empty((chunks, self.chunk, self.rows), dtype=torch.float32,
                                     device=self.device)
            self.gathered = torch.empty((chunks, self.world, self.chunk, self.rows),
                                        dtype=torch.float32, device=self.device)
        for c in range(chunks):
            self.compute(x[c * self.chunk:(c + 1) * self.chunk], self.local[c])
            if self.world == 1:
                self.gathered[c, 0].copy_(self.local[c])
            elif self.side is None:
                dist.all_gather_into_tensor(self.gathered[c].view(-1), self.local[c].view(-1),
                                            group=self.group)
            else:
                done = torch.cuda.Event()
                done.record()
                self.side.wait_event(done)
                with torch.cuda.stream(self.side):
                    dist.all_gather_into_tensor(self.gathered[c].view(-1), self.local[c].view(-1),
                                                group=self.group)
        if self.side is not None and self.world > 1:
            torch.cuda.current_stream().wait_stream(self.side)
        return self.gathered

    def assemble(self, gathered: torch.Tensor) -> torch.Tensor:
        """Dense [m, n] copy of a forward() result."""
        chunks = gathered.shape[0]
        return gathered.permute(0, 2, 1, 3).reshape(chunks * self.chunk, self.world * self.rows)
