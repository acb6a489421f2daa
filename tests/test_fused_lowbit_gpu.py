"""The callers either side of the GEMV, through the C ABI against the oracle:
the activation-quantising GEMV (qgemv_w8a8), the fused decode projections (up + gate,
up + gate + activation, q + k + v), the int8 activation quantiser and the compact int4 rows
(f32 GEMM, W4A8, authoring). Integer work is compared bit for bit, f32 paths at
1e-4 + 1e-5 * |ref|."""

import numpy as np
import pytest

from conftest import assert_bit_equal, assert_close_f32_path

pytestmark = pytest.mark.gpu
Q8_0, Q4_0 = 0, 1
DIST = {Q8_0: (0.001, 0.02), Q4_0: (0.002, 0.04)}


@pytest.mark.parametrize("fmt", [Q8_0, Q4_0])
def test_qgemv_w8a8_matches_oracle(qx, orc, wl, fmt):
    for n, k in [(40, 1024), (1, 32), (129, 2080), (4096, 4096), (300, 96)]:
        packed = wl.packed_blocks(fmt, n, k, *DIST[fmt], seed=n + k)
        x = wl.activations_f32(1, k, seed=k)[0].copy()
        if k >= 96:
            x[32:64] = 0.0           # an all-zero block: scale 0, inverse 0
            x[64] = 3.0e4            # a block dominated by one value
        status, y = qx.qgemv_w8a8(fmt, packed, x, n, k)
        assert status == qx.OK, qx.last_error()
        _, ref = orc.qgemv_w8a8(fmt, packed, x, n, k)
        assert_close_f32_path(y, ref, f"qgemv_w8a8 fmt {fmt} {n}x{k}")
    assert qx.lib.qx_check_device_errors() == qx.OK


@pytest.mark.parametrize("fmt", [Q8_0, Q4_0])
def test_fused_projections_match_oracle(qx, orc, wl, fmt):
    for n, k, kv in [(40, 1024, 24), (4096, 4096, 1024), (130, 2080, 5)]:
        up_w = wl.packed_blocks(fmt, n, k, *DIST[fmt], seed=1)
        gate_w = wl.packed_blocks(fmt, n, k, *DIST[fmt], seed=2)
        wk = wl.packed_blocks(fmt, kv, k, *DIST[fmt], seed=3)
        wv = wl.packed_blocks(fmt, kv, k, *DIST[fmt], seed=4)
        x = wl.activations_f32(1, k, seed=5)[0].copy()
        _, up_ref = orc.qgemv(fmt, up_w, x, n, k, 0)
        _, gate_ref = orc.qgemv(fmt, gate_w, x, n, k, 0)
        status, up, gate = qx.qgemv_up_gate(fmt, up_w, gate_w, x, n, k)
        assert status == qx.OK, qx.last_error()
        assert_close_f32_path(up, up_ref, "up")
        assert_close_f32_path(gate, gate_ref, "gate")
        # the fused launch gives the bits of the separate GEMVs
        assert_bit_equal(up, qx.qgemv(fmt, up_w, x, n, k)[1], "fused up == single GEMV")
        assert_bit_equal(gate, qx.qgemv(fmt, gate_w, x, n, k)[1], "fused gate == single GEMV")
        for gelu in (True, False):
            # act(gate) * up multiplies the (in-tolerance) differences of the two projections
            # by the other factor, so the activation step is held to the bound on ITS inputs:
            # the projections this library computed (checked above)
            status, act = qx.qgemv_up_gate_activation(fmt, up_w, gate_w, x, n, k, gelu)
            assert status == qx.OK, qx.last_error()
            assert_close_f32_path(act, orc.gate_activation(up, gate, gelu), f"activation {gelu}")
        status, q, k_out, v_out = qx.qgemv_qkv(fmt, up_w, wk, wv, x, n, kv, k)
        assert status == qx.OK, qx.last_error()
        assert_close_f32_path(q, up_ref, "q")
        assert_close_f32_path(k_out, orc.qgemv(fmt, wk, x, kv, k, 0)[1], "k")
        assert_close_f32_path(v_out, orc.qgemv(fmt, wv, x, kv, k, 0)[1], "v")


def test_fused_handle_device_entry(qx, orc, wl):
    import torch
    fmt, n, k, m = Q4_0, 1536, 4096, 3
    parts = [wl.packed_blocks(fmt, n, k, *DIST[fmt], seed=s) for s in (7, 8)]
    fused = qx.PackedWeights()
    assert fused.prepare_fused(fmt, parts, [n, n], k) == qx.OK, qx.last_error()
    info = fused.info()
    assert info["rows"] == 2 * n and info["prepared_bytes"] == info["contract_bytes"]
    x = wl.activations_f32(m, k, seed=9)
    xd = torch.from_numpy(x).cuda()
    outs = [torch.full((m, n), -3.0, device="cuda") for _ in range(2)]
    assert fused.qgemm_fused_dev(xd, outs, m) == qx.OK, qx.last_error()
    torch.cuda.synchronize()
    for part, out in zip(parts, outs):
        _, ref = orc.qgemm(fmt, part, x, m, n, k)
        assert_close_f32_path(out.cpu().numpy(), ref, "fused device entry")
    out = torch.zeros(n, device="cuda")
    scratch = torch.zeros(2 * n, device="cuda")
    assert fused.up_gate_activation_dev(xd[0], out, scratch, True) == qx.OK, qx.last_error()
    torch.cuda.synchronize()
    up_ref = orc.qgemv(fmt, parts[0], x[0].copy(), n, k, 0)[1]
    gate_ref = orc.qgemv(fmt, parts[1], x[0].copy(), n, k, 0)[1]
    both = scratch.cpu().numpy()
    assert_close_f32_path(both[:n], up_ref, "up (scratch)")
    assert_close_f32_path(both[n:], gate_ref, "gate (scratch)")
    assert_close_f32_path(out.cpu().numpy(), orc.gate_activation(both[:n].copy(), both[n:].copy(), True),
                          "act dev")


def test_quantize_int8_bit_exact(qx, orc, wl):
    for rows, dim, group in [(5, 192, 0), (5, 192, 32), (3, 4096, 128), (1, 33, 0), (2, 64, 1)]:
        x = wl.activations_f32(rows, dim, seed=rows + dim)
        x[0, : min(dim, 32)] = 0.0
        if dim > 40:
            x[-1, 40] = 1e-30
        status, codes, scales = qx.quantize_int8(x, rows, dim, group)
        assert status == qx.OK, qx.last_error()
        _, c_ref, s_ref = orc.quantize_int8(x, rows, dim, group)
        assert np.array_equal(codes, c_ref), (rows, dim, group)
        assert_bit_equal(scales, s_ref, "quantize_int8 scales")


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (1, 4096, 4096), (4, 1024, 1408), (9, 65, 33), (3, 300, 2050),
                                   (16, 512, 1024)])
def test_lowbit_w8a8_bit_exact(qx, orc, m, n, k):
    """tests/correctness/test_lowbit_w8a8.cpp:53-72 demands exact equality."""
    rng = np.random.Generator(np.random.Philox(key=[m * 1000 + n, k]))
    w = (rng.integers(-1000, 1001, (n, k)).astype(np.float32) / np.float32(1000.0)) * np.float32(0.2)
    x = rng.integers(-2000, 2001, (m, k)).astype(np.float32) / np.float32(500.0)
    status, packed, scales = qx.lowbit_pack(qx.LOWBIT_INT4_ROW, w, n, k)
    assert status == qx.OK, qx.last_error()
    _, p_ref, s_ref = orc.lowbit_pack(2, w, n, k, 0)
    assert np.array_equal(packed, p_ref)
    assert_bit_equal(scales, s_ref, "lowbit_pack scales")
    status, y = qx.lowbit_gemm_w8a8(packed, scales.reshape(-1).copy(), x, m, n, k)
    assert status == qx.OK, qx.last_error()
    _, ref = orc.lowbit_gemm_w8a8(p_ref, s_ref.reshape(-1).copy(), x, m, n, k)
    assert_bit_equal(y, ref, f"lowbit_gemm_w8a8 {m}x{n}x{k}")


@pytest.mark.parametrize("fmt,group,m,n,k", [(2, 0, 3, 19, 200), (3, 64, 2, 17, 256), (2, 0, 4, 9, 33),
                                             (3, 128, 4, 1024, 1408), (2, 0, 16, 4096, 4096),
                                             (3, 48, 2, 33, 200)])
def test_lowbit_gemm_int4(qx, orc, fmt, group, m, n, k):
    rng = np.random.Generator(np.random.Philox(key=[fmt * 100 + k, n]))
    w = (rng.integers(-1000, 1001, (n, k)).astype(np.float32) / np.float32(1000.0)) * np.float32(0.2)
    x = rng.standard_normal((m, k), dtype=np.float32)
    status, packed, scales = qx.lowbit_pack(fmt, w, n, k, group)
    assert status == qx.OK, qx.last_error()
    _, p_ref, s_ref = orc.lowbit_pack(fmt, w, n, k, group)
    assert np.array_equal(packed, p_ref)
    assert_bit_equal(scales, s_ref, "scales")
    status, dq = qx.lowbit_unpack(fmt, packed, scales, n, k, group)
    assert status == qx.OK
    assert_bit_equal(dq, orc.lowbit_unpack(fmt, p_ref, s_ref, n, k, group)[1], "unpack")
    status, y = qx.lowbit_gemm(fmt, packed, scales, x, m, n, k, group)
    assert status == qx.OK, qx.last_error()
    _, ref = orc.lowbit_gemm(fmt, p_ref, s_ref, x, m, n, k, group)
    _, exact = orc.lowbit_gemm_f64(fmt, p_ref, s_ref, x, m, n, k, group)
    assert_close_f32_path(y, exact, "lowbit_gemm vs exact")
    slack = 1e-4 + 1e-5 * np.abs(ref) + np.abs(ref.astype(np.float64) - exact)
    assert np.all(np.abs(y.astype(np.float64) - ref) <= slack), "lowbit_gemm vs reference order"
    assert qx.lowbit_gemm(qx.LOWBIT_INT2_ROW, packed, scales, x, m, n, k, 0)[0] in (
        qx.UNSUPPORTED_FORMAT, qx.INVALID_SHAPE)
