"""Row-sharded decode with the all-gather fused into the GEMV kernel, on two GPUs of one
node (skipped where fewer are visible): gathered results are bit-identical to the unsharded
GEMV, eagerly and replayed from a CUDA graph. The host logic of row sharding itself is
covered on CPU by test_sharded_cpu.py."""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_push_allgather_two_gpus():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29533",
           os.path.join(ROOT, "tests", "sharded_push_worker.py")]
    done = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-4000:]
    assert "sharded push ok" in done.stdout


def test_sharded_prefill_two_gpus():
    """Prefill GEMM with row-sharded weights, M-chunked all-gather overlapped with the GEMM
    (NCCL on a second stream): bit-identical to the unsharded GEMM on every rank."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29535",
           os.path.join(ROOT, "tests", "sharded_prefill_worker.py")]
    done = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-4000:]
    assert "sharded prefill ok" in done.stdout
