"""Host logic of the row-sharded path, world_size 2 over gloo on CPU. The compute step is
a stand-in (the CPU oracle) so that only the partitioning and the all-gather are under
test here; the GPU tests check that the CUDA kernels give shard-independent bits."""

import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    sharded = entry._load_file("qx_sharded", os.path.join(entry.PKG_DIR, "sharded.py"))
    wl = entry._load_file("qx_wl", os.path.join(entry.PKG_DIR, "workloads.py"))
    oracle = entry.load_oracle()
    return sharded, wl, oracle


def test_shard_rows_cover_and_align():
    sharded, _, _ = _load()
    for n in (1, 127, 128, 129, 4096, 14336, 28672, 28673):
        for world in (1, 2, 4, 8):
            ranges = [sharded.shard_rows(n, world, r) for r in range(world)]
            assert ranges[0][0] == 0 and sum(c for _, c in ranges) == n
            for (b0, c0), (b1, _) in zip(ranges, ranges[1:]):
                assert b0 + c0 == b1
            assert all(b % 128 == 0 for b, _ in ranges)
    assert [sharded.shard_rows(28672, 8, r)[1] for r in range(8)] == [3584] * 8
    with pytest.raises(ValueError):
        sharded.shard_rows(10, 2, 2)


def _worker(rank, world, port, fmt, n, k, m, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sharded, wl, oracle = _load()
    orc = oracle.Oracle()
    packed = wl.packed_blocks(fmt, n, k, 0.002, 0.04, seed=17)
    x = wl.activations_f32(m, k, seed=17)
    block_bytes = 34 if fmt == 0 else 18
    begin, rows = sharded.shard_rows(n, world, rank)
    shard = packed.reshape(n, -1)[begin:begin + rows].copy().reshape(-1)
    assert shard.size == rows * (k // 32) * block_bytes

    def compute(xt, out):
        _, y = orc.qgemm(fmt, shard, xt.numpy(), xt.shape[0], rows, k)
        out.copy_(torch.from_numpy(y))

    layer = sharded.ShardedLinear(n, k, compute)
    y = layer.forward(torch.from_numpy(x))
    np.save(os.path.join(out_dir, f"y{rank}.npy"), y.numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("case", [(1, 512, 256, 1), (0, 384, 128, 3), (1, 300, 64, 1)])
def test_two_rank_gather_matches_unsharded(tmp_path, case):
    fmt, n, k, m = case
    port = 29500 + (os.getpid() + n) % 2000
    mp.spawn(_worker, args=(2, port, fmt, n, k, m, str(tmp_path)), nprocs=2, join=True)
    _, wl, oracle = _load()
    packed = wl.packed_blocks(fmt, n, k, 0.002, 0.04, seed=17)
    x = wl.activations_f32(m, k, seed=17)
    _, want = oracle.Oracle().qgemm(fmt, packed, x, m, n, k)
    for rank in range(2):
        got = np.load(os.path.join(str(tmp_path), f"y{rank}.npy"))
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"rank {rank}"


def _prefill_worker(rank, world, port, n, k, m, chunk, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sharded, wl, oracle = _load()
    orc = oracle.Oracle()
    packed = wl.packed_blocks(1, n, k, 0.002, 0.04, seed=19)
    x = wl.activations_f32(m, k, seed=19)
    begin, rows = sharded.shard_rows(n, world, rank)
    shard = packed.reshape(n, -1)[begin:begin + rows].copy().reshape(-1)

    def compute(xt, out):
        _, y = orc.qgemm(1, shard, np.ascontiguousarray(xt.numpy()), xt.shape[0], rows, k)
        out.copy_(torch.from_numpy(y))

    layer = sharded.ShardedPrefill(n, k, compute, chunk_rows=chunk)
    gathered = layer.forward(torch.from_numpy(x))
    assert tuple(gathered.shape) == (m // chunk, world, chunk, rows)
    np.save(os.path.join(out_dir, f"p{rank}.npy"), layer.assemble(gathered).numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_chunked_prefill_matches_unsharded(tmp_path):
    """The M-chunked exchange of the sharded prefill: layout [chunk][rank][row][shard row],
    assembled result equal to the unsharded product on both ranks."""
    n, k, m, chunk = 256, 128, 12, 4
    port = 29500 + (os.getpid() + 777) % 2000
    mp.spawn(_prefill_worker, args=(2, port, n, k, m, chunk, str(tmp_path)), nprocs=2, join=True)
    sharded, wl, oracle = _load()
    packed = wl.packed_blocks(1, n, k, 0.002, 0.04, seed=19)
    x = wl.activations_f32(m, k, seed=19)
    _, want = oracle.Oracle().qgemm(1, packed, x, m, n, k)
    for rank in range(2):
        got = np.load(os.path.join(str(tmp_path), f"p{rank}.npy"))
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"rank {rank}"
    with pytest.raises(ValueError):
        sharded.ShardedPrefill(n, k, lambda a, b: None, chunk_rows=5).forward(torch.zeros((12, k)))
