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


# ---- callers either side of the GEMV: activation-quantising GEMV, fused decode projections,
# ---- int8 activation quantiser, compact int4 rows ----------------------------------------

def _fused_inputs(wl, fmt, lo, hi):
    n, k, kv = 40, 1024, 24
    up_w = wl.packed_blocks(fmt, n, k, lo, hi, seed=31)
    gate_w = wl.packed_blocks(fmt, n, k, lo, hi, seed=32)
    wk = wl.packed_blocks(fmt, kv, k, lo, hi, seed=33)
    wv = wl.packed_blocks(fmt, kv, k, lo, hi, seed=34)
    x = wl.activations_f32(1, k, seed=31)[0].copy()
    return n, k, kv, up_w, gate_w, wk, wv, x


@pytest.mark.parametrize("fmt,name,lo,hi", [(Q8_0, "q8", 0.001, 0.02), (Q4_0, "q4", 0.002, 0.04)])
def test_w8a8_and_fused_projections_golden(orc, wl, golden, fmt, name, lo, hi):
    """The portable kernels of the reference (forced-ref fixtures) bit for bit; the runtime
    dispatched ones (default fixtures) within the f32 tolerance where their summation order
    differs."""
    n, k, kv, up_w, gate_w, wk, wv, x = _fused_inputs(wl, fmt, lo, hi)
    g_ref, g_def = golden["forced_ref"], golden["default"]
    status, y = orc.qgemv_w8a8(fmt, up_w, x, n, k)
    assert status == 0
    assert_bit_equal(y, g_ref[f"w8a8_{name}_{n}x{k}_y"], "qgemv_w8a8 vs reference (ref variant)")
    assert np.allclose(y, g_def[f"w8a8_{name}_{n}x{k}_y"], rtol=1e-5, atol=1e-4)
    _, up = orc.qgemv(fmt, up_w, x, n, k, 0)
    _, gate = orc.qgemv(fmt, gate_w, x, n, k, 0)
    for g in (g_ref, g_def):  # the fused entry points have one (portable) kernel on x86
        assert_bit_equal(up, g[f"upgate_{name}_{n}x{k}_up"], "up")
        assert_bit_equal(gate, g[f"upgate_{name}_{n}x{k}_gate"], "gate")
        for gelu in (1, 0):
            assert_bit_equal(orc.gate_activation(up, gate, bool(gelu)),
                             g[f"upgate_{name}_{n}x{k}_act{gelu}"], f"activation gelu={gelu}")
        assert_bit_equal(orc.qgemv(fmt, wk, x, kv, k, 0)[1], g[f"qkv_{name}_k"], "qkv k")
        assert_bit_equal(orc.qgemv(fmt, wv, x, kv, k, 0)[1], g[f"qkv_{name}_v"], "qkv v")
        assert_bit_equal(up, g[f"qkv_{name}_q"], "qkv q")
    # non-finite activations are rejected (src/dispatch/qgemv_w8a8.cpp:141-145)
    bad = x.copy()
    bad[5] = np.inf
    assert orc.qgemv_w8a8(fmt, up_w, bad, n, k)[0] == 3


def test_quantize_int8_golden(orc, wl, golden):
    x = wl.activations_f32(5, 192, seed=41)
    x[1] = 0.0
    x[2, 7] = 1e-30
    for name in ("default", "forced_ref"):
        for group in (0, 32, 64):
            status, codes, scales = orc.quantize_int8(x, 5, 192, group)
            assert status == 0
            assert np.array_equal(codes, golden[name][f"quant_int8_g{group}_codes"])
            assert_bit_equal(scales, golden[name][f"quant_int8_g{group}_scales"], "scales")
    assert orc.quantize_int8(x, 5, 192, 50)[0] == 1       # group does not divide dim
    bad = x.copy()
    bad[0, 0] = np.nan
    assert orc.quantize_int8(bad, 5, 192, 0)[0] == 3


def _lowbit_case(fmt, n, k, m):
    rng = np.random.Generator(np.random.Philox(key=[fmt * 100 + k, 7]))
    w = (rng.integers(-1000, 1001, (n, k)).astype(np.float32) / np.float32(1000.0)) * np.float32(0.2)
    x = rng.integers(-2000, 2001, (m, k)).astype(np.float32) / np.float32(500.0)
    return w, x


@pytest.mark.parametrize("fmt,group,n,k,m", [(2, 0, 19, 200, 3), (3, 64, 17, 256, 2), (2, 0, 9, 33, 4)])
def test_lowbit_int4_golden(orc, golden, fmt, group, n, k, m):
    import hashlib
    w, x = _lowbit_case(fmt, n, k, m)
    tag = f"lowbit_f{fmt}_{m}x{n}x{k}"
    for name in ("default", "forced_ref"):
        g = golden[name]
        status, packed, scales = orc.lowbit_pack(fmt, w, n, k, group)
        assert status == 0
        assert np.array_equal(packed, g[tag + "_packed"])
        assert_bit_equal(scales, g[tag + "_scales"], "scales")
        _, dq = orc.lowbit_unpack(fmt, packed, scales, n, k, group)
        assert hashlib.sha256(np.ascontiguousarray(dq).tobytes()).hexdigest() == str(g[tag + "_unpacked_sha"])
        _, y = orc.lowbit_gemm(fmt, packed, scales, x, m, n, k, group)
        # the f32 GEMM runs an AVX-512 variant on the generating host (another summation
        # order): tolerance; the W4A8 route is exact integers and two multiplies: bits
        assert np.allclose(y, g[tag + "_y"], rtol=1e-5, atol=1e-4), str(g["lowbit_variant"])
        if fmt == 2:
            _, y8 = orc.lowbit_gemm_w8a8(packed, scales.reshape(-1), x, m, n, k)
            assert_bit_equal(y8, g[tag + "_y_w8a8"], "lowbit_gemm_w8a8")


def test_new_entry_points_against_live_reference(orc, ref, wl):
    if not hasattr(ref.lib, "qxref_qgemv_w8a8"):
        pytest.skip("reference library built before these entry points were added")
    for fmt, lo, hi in ((Q8_0, 0.001, 0.02), (Q4_0, 0.002, 0.04)):
        n, k = 130, 2048
        w = wl.packed_blocks(fmt, n, k, lo, hi, seed=51)
        x = wl.activations_f32(1, k, seed=52)[0].copy()
        a, b = orc.qgemv_w8a8(fmt, w, x, n, k)[1], ref.qgemv_w8a8(fmt, w, x, n, k)[1]
        assert np.allclose(a, b, rtol=1e-5, atol=1e-4)
    x = wl.activations_f32(7, 4096, seed=53)
    for group in (0, 128):
        _, c1, s1 = orc.quantize_int8(x, 7, 4096, group)
        _, c2, s2 = ref.quantize_int8(x, 7, 4096, group)
        assert np.array_equal(c1, c2)
        assert_bit_equal(s1, s2, "quantize_int8 scales")
    w, xx = _lowbit_case(2, 65, 1408, 4)
    _, packed, scales = orc.lowbit_pack(2, w, 65, 1408, 0)
    _, p2, s2 = ref.lowbit_pack(2, w, 65, 1408, 0)
    assert np.array_equal(packed, p2)
    assert_bit_equal(scales, s2, "lowbit scales")
    assert_bit_equal(orc.lowbit_gemm_w8a8(packed, scales.reshape(-1), xx, 4, 65, 1408)[1],
                     ref.lowbit_gemm_w8a8(packed, scales.reshape(-1), xx, 4, 65, 1408)[1], "W4A8")
    assert np.allclose(orc.lowbit_gemm(2, packed, scales, xx, 4, 65, 1408)[1],
                       ref.lowbit_gemm(2, packed, scales, xx, 4, 65, 1408)[1], rtol=1e-5, atol=1e-4)
