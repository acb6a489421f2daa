"""W8A32 GEMM and the q8_0 / q4_0 authoring kernels (pack / unpack)."""

import numpy as np
import pytest

from conftest import assert_bit_equal, assert_close_f32_path

pytestmark = pytest.mark.gpu
Q8_0, Q4_0 = 0, 1


def _close_w8a32(got, ref):
    # the stated bound of the f32 paths, 1e-4 absolute + 1e-5 relative per element, which is
    # tighter than the reference's own test bound wherever |ref| > 5
    # (3e-5 * max(1, |ref|), tests/correctness/test_w8a32_gemm.cpp:16-17); both must hold
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    return np.all(np.abs(got - ref) <= np.minimum(1e-4 + 1e-5 * np.abs(ref),
                                                  3e-5 * np.maximum(1.0, np.abs(ref))))


def test_w8a32_reference_ladder(qx, orc, golden, gold_inputs):
    for k in gold_inputs.W8A32_KS:
        w, scales, x = gold_inputs.w8a32_inputs(5, 5, k)
        status, y = qx.qgemm_w8a32(w, scales, x, 5, 5, k)
        assert status == qx.OK, qx.last_error()
        _, ref = orc.qgemm_w8a32(w, scales, x, 5, 5, k)
        assert _close_w8a32(y, ref), f"K={k} vs sequential f32"
        assert _close_w8a32(y, golden["default"][f"w8a32_5x5x{k}_y"]), f"K={k} vs reference"


@pytest.mark.parametrize("shape", [(4, 1024, 1408), (16, 4096, 4096), (3, 77, 1000), (64, 96, 333),
                                   (1, 5000, 48), (33, 4736, 528), (7, 9, 15)])
def test_w8a32_bench_shapes(qx, orc, wl, shape):
    # shapes of the reference benchmark (benchmarks/cases/colibri_ops.cpp:466-478) + ragged
    m, n, k = shape
    rng = np.random.Generator(np.random.Philox(key=[m, n + k]))
    w = rng.integers(-127, 128, (n, k), dtype=np.int8)
    ws = rng.uniform(0.001, 0.01, n).astype(np.float32)
    x = rng.standard_normal((m, k), dtype=np.float32)
    status, y = qx.qgemm_w8a32(w, ws, x, m, n, k)
    assert status == qx.OK, qx.last_error()
    y64 = orc.qgemm_w8a32_f64(w, ws, x, m, n, k)
    _, ref = orc.qgemm_w8a32(w, ws, x, m, n, k, avx512_order=True)
    # against the reference's f32 path (its AVX-512 summation order) at the stated bound, and
    # against float64 not worse than 2x the reference's own f32 error
    assert_close_f32_path(y, ref, f"w8a32 {shape} vs reference f32")
    assert np.abs(y - y64).max() <= max(2 * np.abs(ref - y64).max(), 1e-5 * np.abs(y64).max())
    assert _close_w8a32(y, y64)


@pytest.mark.parametrize("fmt", [Q8_0, Q4_0])
def test_pack_unpack_bit_exact(qx, orc, wl, fmt):
    for n, k in [(1, 32), (3, 64), (33, 512), (129, 2048)]:
        values = wl.xorshift_uniform(0xC0FFEE ^ (n * 131 + k), n * k)
        w = values.reshape(n, k).copy()
        w[0, :32] *= 1e-3 / max(1.0, np.abs(w[0, :32]).max())  # fp16-subnormal scale block
        if n > 1:
            w[1, :32] = 0.0  # all-zero block: d = 0, inverse 0
        status, packed = qx.qgemv_pack(fmt, w, n, k)
        assert status == qx.OK, qx.last_error()
        _, want = orc.pack(fmt, w, n, k)
        assert np.array_equal(packed, want), f"pack fmt {fmt} {n}x{k}"
        status, dq = qx.qgemv_unpack(fmt, packed, n, k)
        assert status == qx.OK
        _, want_dq = orc.unpack(fmt, packed, n, k)
        assert_bit_equal(dq, want_dq, "unpack")


def test_pack_rejects_non_finite(qx):
    # tests/correctness/test_qgemv.cpp:124-140
    bad = np.ones((1, 32), np.float32)
    bad[0, 7] = np.nan
    assert qx.qgemv_pack(Q8_0, bad, 1, 32)[0] == qx.INVALID_ARGUMENT
    assert qx.qgemv_pack(Q4_0, bad, 1, 32)[0] == qx.INVALID_ARGUMENT
    bad[0, 7] = np.inf
    assert qx.qgemv_pack(Q8_0, bad, 1, 32)[0] == qx.INVALID_ARGUMENT


def test_device_query(qx):
    info = qx.device_info()
    assert info["sm_major"] == 10 and info["sm_count"] >= 100
    assert info["peer_access_mask"] & (1 << info["device"])
    # NVLink discovery: consistent with the peer mask; one visible GPU has no NVLink peers
    assert info["nvlink_peer_mask"] & ~info["peer_access_mask"] == 0
    assert info["nvlink_peers"] == bin(info["nvlink_peer_mask"]).count("1")
    if info["visible_devices"] == 1:
        assert info["nvlink_peers"] == 0 and info["nvlink_uniform"] == 0
    else:
        assert info["nvlink_peers"] >= 1  # the GPUs of one B200 node sit on one NVSwitch fabric
        for peer in range(min(16, info["visible_devices"])):
            if info["nvlink_peer_mask"] & (1 << peer):
                assert info["peer_performance_rank"][peer] >= 0
