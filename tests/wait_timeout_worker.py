"""Worker of test_device_gpu.py: makes a bounded device-side wait run out (on purpose, in
the safe form: the kernel returns by itself) and checks how the host learns of it.

A two-rank push plan is built on ONE GPU whose "peer" buffers are local allocations, and
the receive of a step's slices is enqueued although no GEMV ever pushed one. With
QX_B200_WAIT_LIMIT_MS=5 in the environment the wait kernel gives up after 5 ms, leaves role
code 31 in the device's error word and returns; nothing faults, traps or hangs."""

import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def main() -> int:
    assert os.environ.get("QX_B200_WAIT_LIMIT_MS") == "5"
    torch.cuda.set_device(0)
    qx = entry.load_package()
    wl = entry._load_file("wl", os.path.join(entry.PKG_DIR, "workloads.py"))
    orc = entry.load_oracle().Oracle()
    fmt, n, k = 0, 256, 1024
    packed = wl.packed_blocks(fmt, n, k, 0.001, 0.02, seed=3)
    x = wl.activations_f32(1, k, seed=3)
    _, want = orc.qgemm(fmt, packed, x, 1, n, k)

    def gemv_ok():
        status, y = qx.qgemv(fmt, packed, x[0].copy(), n, k)
        return status, (status == qx.OK and
                        bool(np.all(np.abs(y - want[0]) <= 1e-4 + 1e-5 * np.abs(want[0]))))

    status, ok = gemv_ok()  # creates the device context; nothing pending
    assert status == qx.OK and ok, qx.last_error()

    rows = 128
    plan = qx.PushPlan()
    plan.world, plan.rank, plan.rows_per_rank = 2, 0, rows
    plan.results_local, _ = qx.peer_alloc(2 * 2 * rows * 4)
    plan.inbox_local, _ = qx.peer_alloc(qx.push_inbox_bytes(2, 1, rows))
    plan.inbox_peer[1], _ = qx.peer_alloc(qx.push_inbox_bytes(2, 1, rows))  # stand-in for rank 1's inbox

    for round_ in range(2):
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        qx.allgather_wait_dev(plan, 1, round_ + 1)  # nobody produces this step
        t1.record()
        torch.cuda.synchronize()                     # returns: the kernel gave up by itself
        waited_ms = t0.elapsed_time(t1)
        assert 4.0 <= waited_ms < 500.0, waited_ms
        if round_ == 0:
            # a `_dev` caller polls the error word
            assert qx.lib.qx_check_device_errors() == qx.DEVICE_ERROR
            assert "role code 31" in qx.last_error(), qx.last_error()
            assert qx.lib.qx_check_device_errors() == qx.OK  # reported once, then clear
        else:
            # a host-pointer caller gets it from its next call (whose own result is suspect)
            status, _ = gemv_ok()
            assert status == qx.DEVICE_ERROR and "role code 31" in qx.last_error(), qx.last_error()
        status, ok = gemv_ok()                       # the context stays usable and correct
        assert status == qx.OK and ok, qx.last_error()
    print("wait timeout ok", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
