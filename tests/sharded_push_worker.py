"""Worker of test_sharded_push_gpu.py: one process per GPU (torchrun). Every rank prepares
its row shard, runs the GEMV with the fused all-gather for several steps (eager, then
replayed from a CUDA graph) and compares the gathered result with the unsharded GEMV of the
same weights computed locally: bit-identical, since no reduction crosses a shard."""

import ctypes
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def device_to_host(ptr: int, count: int) -> np.ndarray:
    out = torch.empty(count, dtype=torch.float32, device="cuda")
    cudart = ctypes.CDLL("libcudart.so.12")
    cudart.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    assert cudart.cudaMemcpy(out.data_ptr(), ptr, count * 4, 3) == 0  # device to device
    return out.cpu().numpy()


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    qx = entry.load_package()
    wl = entry._load_file("wl", os.path.join(entry.PKG_DIR, "workloads.py"))
    sharded = entry._load_file(entry.PKG_NAME + ".sharded", os.path.join(entry.PKG_DIR, "sharded.py"))
    for fmt, (lo, hi) in ((1, (0.002, 0.04)), (0, (0.001, 0.02))):
        n, k = 512 * world, 2048
        packed = wl.packed_blocks(fmt, n, k, lo, hi, seed=11)
        full = qx.PackedWeights()
        qx.check(full.prepare(fmt, packed, n, k), "prepare full")
        shard = qx.PackedWeights()
        rows = n // world
        qx.check(shard.prepare(fmt, packed, n, k, rank * rows, rows), "prepare shard")
        gather = sharded.PushAllGather(qx, rows, 1)
        xs = [torch.from_numpy(wl.activations_f32(1, k, seed=s)).cuda() for s in range(4)]
        want = []
        for x in xs:
            y = torch.zeros(n, device="cuda")
            qx.check(full.qgemm_dev(x, y, 1, n), "full gemv")
            want.append(y)
        torch.cuda.synchronize()
        for s, x in enumerate(xs):  # eager steps
            ptr = gather.step(shard, x, 1)
            torch.cuda.synchronize()
            got = device_to_host(ptr, n)
            assert np.array_equal(got.view(np.uint32), want[s].cpu().numpy().view(np.uint32)), \
                f"rank {rank} fmt {fmt} step {s}: gathered result differs from the unsharded GEMV"
        dist.barrier()
        # the same two steps replayed from a CUDA graph (step numbers live on the device)
        graph = torch.cuda.CUDAGraph()
        ptrs = []
        with torch.cuda.graph(graph):
            for x in xs[:2]:
                ptrs.append(gather.step(shard, x, 1))
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        for s in range(2):
            got = device_to_host(ptrs[s], n)
            assert np.array_equal(got.view(np.uint32), want[s].cpu().numpy().view(np.uint32)), \
                f"rank {rank} fmt {fmt} graph step {s}"
        # Many steps with nothing between them but the stream order, a different activation
        # vector per step, and one rank held back on the host now and then: every step's
        # full gathered result (all ranks' slices) is copied aside on the stream and compared
        # afterwards. A wait that returned early, or a rank overwriting a buffer a peer
        # still reads, shows up as a stale or mixed slice.
        import time
        for m in (1, 4):
            steps = 24
            gather_m = gather if m == 1 else sharded.PushAllGather(qx, rows, m)
            xs_m = [torch.from_numpy(wl.activations_f32(m, k, seed=100 + s)).cuda() for s in range(steps)]
            wants = []
            for x in xs_m:
                y = torch.zeros((m, n), device="cuda")
                qx.check(full.qgemm_dev(x, y, m, n), "full gemm")
                wants.append(y)
            history = torch.zeros((steps, world, m, rows), device="cuda")
            cudart = ctypes.CDLL("libcudart.so.12")
            cudart.cudaMemcpyAsync.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t,
                                               ctypes.c_int, ctypes.c_void_p]
            torch.cuda.synchronize()
            dist.barrier()
            stream = torch.cuda.current_stream().cuda_stream
            for s in range(steps):
                if s % 5 == rank % 5 and s > 0:
                    time.sleep(0.002)  # this rank falls behind on the host
                ptr = gather_m.step(shard, xs_m[s], m)
                assert cudart.cudaMemcpyAsync(history[s].data_ptr(), ptr, world * m * rows * 4, 3, stream) == 0
            torch.cuda.synchronize()
            for s in range(steps):
                for r in range(world):
                    want_slice = wants[s][:, r * rows:(r + 1) * rows].contiguous()
                    assert torch.equal(history[s, r].view(torch.int32), want_slice.view(torch.int32)), \
                        f"rank {rank} fmt {fmt} m {m}: unsynchronised step {s}, slice of rank {r} differs"
            dist.barrier()
        # A long captured chain with nothing but the two kernels of every step in it: with
        # programmatic dependent launch the kernels of several steps are resident at once
        # (small grids leave room), among them receive kernels of steps two apart, which
        # poll the same cells. Each must take only the cells of its own step.
        chain = torch.cuda.CUDAGraph()
        chain_ptrs = []
        with torch.cuda.graph(chain):
            for s in range(200):
                chain_ptrs.append(gather.step(shard, xs[s % 2], 1))
        dist.barrier()
        for _ in range(3):
            chain.replay()
        torch.cuda.synchronize()
        for s in (198, 199):
            got = device_to_host(chain_ptrs[s], n)
            assert np.array_equal(got.view(np.uint32), want[s % 2].cpu().numpy().view(np.uint32)), \
                f"rank {rank} fmt {fmt}: step {s} of the long chain"
        assert qx.lib.qx_check_device_errors() == qx.OK, f"rank {rank}: {qx.last_error()}"
        dist.barrier()
        status, _ = qx.qgemv(fmt, packed[: 32 * (k // 32) * (18 if fmt == 1 else 34)],
                             wl.activations_f32(1, k)[0], 32, k)  # host call: reports device errors
        assert status == qx.OK, qx.last_error()
        dist.barrier()
    if rank == 0:
        print("sharded push ok", flush=True)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
