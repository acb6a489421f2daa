"""The oracle is pinned here: bit-for-bit against the golden vectors produced by the
unmodified reference, and against the reference library itself when it is built."""

import numpy as np
import pytest

from conftest import assert_bit_equal

Q8_0, Q4_0 = 0, 1


def test_fp16_conversion_golden(orc, golden):
    g = golden["default"]
    table = np.array([orc.fp16_to_fp32(h) for h in range(65536)], np.float32).view(np.uint32)
    assert np.array_equal(table, g["fp16_all_to_f32"])
    for value, want in zip(g["fp16_values"], g["fp16_bits"]):
        assert orc.fp32_to_fp16(float(value)) == int(want), value
    for value, want in zip(g["fp16_values"], g["bf16_bits"]):
        assert orc.float_to_bf16(float(value)) == int(want), value
    # known answers of tests/correctness/test_qgemv.cpp:79-97
    assert orc.fp32_to_fp16(2.0 ** -14) == 0x0400
    assert orc.fp32_to_fp16(2.0 ** -15) == 0x0200
    assert orc.fp32_to_fp16(2.0 ** -24) == 0x0001
    assert orc.fp32_to_fp16(2.0 ** -25) == 0x0000
    assert orc.fp32_to_fp16(-(2.0 ** -24)) == 0x8001
    for v in (1.0, 0.5, 0.0, 65504.0):
        assert orc.fp16_to_fp32(orc.fp32_to_fp16(v)) == v


def test_validation_statuses(orc):
    # tests/correctness/test_qgemv.cpp:99-122
    assert orc.qgemv_packed_size(Q8_0, 4, 33)[0] == 1
    assert orc.qgemv_packed_size(Q8_0, 0, 32)[0] == 1
    assert orc.qgemv_packed_size(Q8_0, 1, 32, want_size=False)[0] == 3
    assert orc.qgemv_packed_size(Q8_0, 1 << 62, 128)[0] == 1
    assert orc.qgemv_packed_size(7, 4, 64)[0] == 2
    assert orc.qgemv_packed_size(Q8_0, 4, 64) == (0, 4 * 2 * 34)
    assert orc.qgemv_packed_size(Q4_0, 4, 64) == (0, 4 * 2 * 18)
    assert orc.lib.qxo_qgemv(Q8_0, None, None, None, 4, 33, 0) == 1
    x = np.zeros(32, np.float32)
    assert orc.lib.qxo_qgemv(Q8_0, None, x.ctypes.data, x.ctypes.data, 1, 32, 0) == 3
    bad = np.ones((1, 32), np.float32)
    bad[0, 7] = np.nan
    assert orc.pack(Q8_0, bad, 1, 32)[0] == 3
    assert orc.pack(Q4_0, bad, 1, 32)[0] == 3
    bad[0, 7] = np.inf
    assert orc.pack(Q8_0, bad, 1, 32)[0] == 3


def _ladder_inputs(wl, gold_inputs, n, k, seed):
    values = wl.xorshift_uniform(seed, n * k + k)
    return values[:n * k].reshape(n, k).copy(), values[n * k:].copy()


def test_q8_0_ladder_golden(orc, wl, golden, gold_inputs):
    g = golden["default"]
    for n, k in gold_inputs.Q8_LADDER:
        w, x = _ladder_inputs(wl, gold_inputs, n, k, (0x9E3779B9 ^ (n * 131 + k)) & 0xFFFFFFFF)
        status, packed = orc.pack(Q8_0, w, n, k)
        assert status == 0
        tag = f"q8_{n}x{k}"
        assert gold_inputs.sha(packed) == str(g[tag + "_packed_sha"])
        _, dq = orc.unpack(Q8_0, packed, n, k)
        assert gold_inputs.sha(dq) == str(g[tag + "_unpacked_sha"])
        _, y = orc.qgemv(Q8_0, packed, x, n, k)
        assert_bit_equal(y, g[tag + "_y"], tag)
        # the reference's own acceptance bound against float64 (test_qgemv.cpp:297)
        _, y64 = orc.qgemm_f64(Q8_0, packed, x.reshape(1, k), 1, n, k)
        assert np.all(np.abs(y - y64[0]) <= 1e-5 + 1e-4 * np.abs(y64[0]))


def test_q4_0_golden_both_variants(orc, wl, golden, gold_inputs):
    n, k = 33, 512
    w, x = _ladder_inputs(wl, gold_inputs, n, k, 0xD1B54A32)
    status, packed = orc.pack(Q4_0, w, n, k)
    assert status == 0
    assert np.array_equal(packed, golden["default"]["q4_33x512_packed"])
    _, dq = orc.unpack(Q4_0, packed, n, k)
    assert gold_inputs.sha(dq) == str(golden["default"]["q4_33x512_unpacked_sha"])
    assert str(golden["default"]["variant_qgemv_q4_0"]) == "avx2"
    assert str(golden["forced_ref"]["variant_qgemv_q4_0"]) == "q4_0_ref"
    _, y_avx2 = orc.qgemv(Q4_0, packed, x, n, k, q4_variant=1)
    assert_bit_equal(y_avx2, golden["default"]["q4_33x512_y"], "q4_0 avx2 order")
    _, y_ref = orc.qgemv(Q4_0, packed, x, n, k, q4_variant=0)
    assert_bit_equal(y_ref, golden["forced_ref"]["q4_33x512_y"], "q4_0 portable order")


def test_subnormal_scale_block(orc, golden):
    # tests/correctness/test_qgemv.cpp:199-216
    w = np.full((1, 32), 1e-3, np.float32)
    _, packed = orc.pack(Q8_0, w, 1, 32)
    assert np.array_equal(packed, golden["default"]["q8_subnormal_packed"])
    _, dq = orc.unpack(Q8_0, packed, 1, 32)
    assert dq[0, 0] != 0.0 and abs(dq[0, 0] - 1e-3) < 1e-5
    _, y = orc.qgemv(Q8_0, packed, np.ones(32, np.float32), 1, 32)
    assert_bit_equal(y, golden["default"]["q8_subnormal_y"])
    assert abs(y[0] - 32.0 * dq[0, 0]) < 1e-6


def test_bench_distribution_golden(orc, wl, golden, gold_inputs):
    for fmt, name, lo, hi in ((Q8_0, "q8", 0.001, 0.02), (Q4_0, "q4", 0.002, 0.04)):
        n, k, m = 48, 4096, 3
        packed = wl.packed_blocks(fmt, n, k, lo, hi, seed=21)
        x = wl.activations_f32(m, k, seed=21)
        tag = f"{name}_bench_{m}x{n}x{k}"
        assert gold_inputs.sha(packed) == str(golden["default"][tag + "_packed_sha"])
        _, y = orc.qgemm(fmt, packed, x, m, n, k, q4_variant=1)
        assert_bit_equal(y, golden["default"][tag + "_y"], tag)
        _, y = orc.qgemm(fmt, packed, x, m, n, k, q4_variant=0)
        assert_bit_equal(y, golden["forced_ref"][tag + "_y"], tag + " portable")


def test_int8_gemm_golden(orc, golden, gold_inputs):
    for which in ("default", "forced_ref"):
        g = golden[which]
        for m, n, k in gold_inputs.INT8_SHAPES:
            w, x, ws, xs, row_sum, zp = gold_inputs.int8_inputs(m, n, k)
            status, y, acc = orc.int8_gemm(w, x, ws, xs, m, n, k)
            assert status == 0
            assert_bit_equal(y, g[f"int8_{m}x{n}x{k}_y"], f"int8 {m}x{n}x{k} {which}")
            assert np.array_equal(acc, x.astype(np.int64) @ w.astype(np.int64).T)
            _, y, _ = orc.int8_gemm(w, x, ws, xs, m, n, k, row_sum, zp, True)
            assert_bit_equal(y, g[f"int8_{m}x{n}x{k}_y_azp"], f"int8 azp {m}x{n}x{k} {which}")
    # hand case of tests/correctness/test_sibling_entrypoints.cpp:270-280:
    # dots 2-2-3+3=0 and -4-1+0+2=-3 -> [0, -3*0.25*2]
    w8 = np.array([[1, 2, -1, 3], [-2, 1, 0, 2]], np.int8)
    x8 = np.array([[2, -1, 3, 1]], np.int8)
    _, y, acc = orc.int8_gemm(w8, x8, np.array([0.5, 0.25], np.float32),
                              np.array([2.0], np.float32), 1, 2, 4)
    assert acc.tolist() == [[0, -3]] and y.tolist() == [[0.0, -1.5]]
    assert_bit_equal(y, golden["default"]["int8_hand_y"])


def test_int8_gemm_statuses(orc):
    w = np.zeros((2, 4), np.int8)
    x = np.zeros((1, 4), np.int8)
    ws = np.ones(2, np.float32)
    xs = np.ones(1, np.float32)
    assert orc.int8_gemm(w, x, ws, xs, 0, 2, 4)[0] == 1
    assert orc.int8_gemm(w, x, ws, xs, 1, 2, 4, asymmetric=True)[0] == 3
    ws[1] = np.inf
    assert orc.int8_gemm(w, x, ws, xs, 1, 2, 4)[0] == 3


def test_w8a32_golden(orc, golden, gold_inputs):
    for k in gold_inputs.W8A32_KS:
        w, scales, x = gold_inputs.w8a32_inputs(5, 5, k)
        _, y = orc.qgemm_w8a32(w, scales, x, 5, 5, k)
        assert_bit_equal(y, golden["forced_ref"][f"w8a32_5x5x{k}_y"], f"w8a32 ref K={k}")
        _, y = orc.qgemm_w8a32(w, scales, x, 5, 5, k, avx512_order=True)
        assert_bit_equal(y, golden["default"][f"w8a32_5x5x{k}_y"], f"w8a32 avx512 K={k}")


def test_panel_layout_golden(orc, wl, golden):
    for fmt, name, lo, hi in ((Q8_0, "q8", 0.001, 0.02), (Q4_0, "q4", 0.002, 0.04)):
        rows, cols = 6, 96
        packed = wl.packed_blocks(fmt, rows, cols, lo, hi, seed=5)
        status, panel = orc.build_panel(fmt, packed, rows, cols, 4)
        assert status == 0
        assert np.array_equal(panel, golden["default"][f"panel_{name}_6x96_tile4"])
        # m >= 64 takes the reference's panel kernels, whose per-row arithmetic is the
        # portable GEMV order (kernels/quantization/qgemm_panel.cpp:83-170)
        x = wl.activations_f32(70, cols, seed=5)
        _, y = orc.qgemm(fmt, packed, x, 70, rows, cols, q4_variant=0)
        assert_bit_equal(y, golden["default"][f"prepacked_{name}_70x6x96_y"], f"panel gemm {name}")


def test_oracle_matches_live_reference(orc, ref, wl):
    """Where the reference library is built, compare on fresh seeded inputs too."""
    variants = ref.variants()
    for fmt, lo, hi in ((Q8_0, 0.001, 0.02), (Q4_0, 0.002, 0.04)):
        n, k, m = 40, 2048, 2
        packed = wl.packed_blocks(fmt, n, k, lo, hi, seed=33)
        x = wl.activations_f32(m, k, seed=33)
        _, y_ref = ref.qgemm(fmt, packed, x, m, n, k)
        variant = 1 if (fmt == Q4_0 and variants["qgemv_q4_0"] == "avx2") else 0
        _, y = orc.qgemm(fmt, packed, x, m, n, k, q4_variant=variant)
        assert_bit_equal(y, y_ref, f"live fmt={fmt}")
    w, x, ws, xs = wl.w8a8_inputs(7, 33, 4096, seed=3)
    _, y_ref = ref.qgemm_w8a8(w, x, ws, xs, 7, 33, 4096)
    _, y, _ = orc.int8_gemm(w, x, ws, xs, 7, 33, 4096)
    assert_bit_equal(y, y_ref, "live w8a8")
