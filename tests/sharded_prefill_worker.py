"""Worker of test_sharded_push_gpu.py::test_sharded_prefill_two_gpus: one process per GPU
(torchrun). Every rank prepares its row shard of a q4_0 matrix and runs the prefill GEMM
(bf16 activations) chunk by chunk with the all-gather of a chunk overlapping the GEMM of
the next one; the assembled result must equal the unsharded GEMM of the same weights
computed locally bit for bit (no reduction crosses a shard, chunks are whole token tiles)."""

import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    qx = entry.load_package()
    wl = entry._load_file("wl", os.path.join(entry.PKG_DIR, "workloads.py"))
    sharded = entry._load_file(entry.PKG_NAME + ".sharded", os.path.join(entry.PKG_DIR, "sharded.py"))
    n, k, m, chunk = 512 * world, 1024, 768, 256
    packed = wl.packed_blocks(qx.Q4_0, n, k, 0.002, 0.04, seed=23)
    xb = torch.from_numpy(wl.to_bf16_bits(wl.activations_f32(m, k, seed=23)).view(np.int16)).cuda()
    full = qx.PackedWeights()
    qx.check(full.prepare(qx.Q4_0, packed, n, k), "prepare full")
    want = torch.zeros((m, n), device="cuda")
    qx.check(full.qgemm_bf16_dev(xb, want, m), "unsharded prefill GEMM")
    begin, rows = sharded.shard_rows(n, world, rank)
    shard = qx.PackedWeights()
    qx.check(shard.prepare(qx.Q4_0, packed, n, k, begin, rows), "prepare shard")

    def compute(x_chunk, out):
        qx.check(shard.qgemm_bf16_dev(x_chunk, out, x_chunk.shape[0]), "sharded prefill GEMM")

    layer = sharded.ShardedPrefill(n, k, compute, chunk_rows=chunk, device="cuda")
    for attempt in range(3):
        got = layer.assemble(layer.forward(xb))
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int32), want.view(torch.int32)), f"rank {rank} attempt {attempt}"
    assert qx.lib.qx_check_device_errors() == 0
    dist.barrier()
    if rank == 0:
        print("sharded prefill ok")
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
