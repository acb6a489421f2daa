"""The C-ABI library loads without a GPU, exports every symbol include/qx_b200.h declares,
answers the validation-only calls exactly like the reference, and fails loudly (no CPU
fallback) when asked to compute without a device."""

import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "qx_b200.h")).read()
    return sorted(set(re.findall(r"QX_API[^;(]*?\b(qx_[a-z0-9_]+)\s*\(", text)))


def test_exports_every_declared_symbol(qx):
    names = declared_symbols()
    assert len(names) >= 28, names
    for name in names:
        assert hasattr(qx.lib, name), f"{name} is declared in qx_b200.h but not exported"


def test_packed_size_and_validation_order(qx):
    # tests/correctness/test_qgemv.cpp:99-122 of the reference
    assert qx.qgemv_packed_size(qx.Q8_0, 4, 33)[0] == qx.INVALID_SHAPE
    assert qx.qgemv_packed_size(qx.Q8_0, 0, 32)[0] == qx.INVALID_SHAPE
    assert qx.qgemv_packed_size(qx.Q8_0, 1, 32, want_size=False)[0] == qx.INVALID_ARGUMENT
    assert qx.qgemv_packed_size(qx.Q8_0, 1 << 62, 128)[0] == qx.INVALID_SHAPE
    assert qx.qgemv_packed_size(9, 4, 64)[0] == qx.UNSUPPORTED_FORMAT
    assert qx.qgemv_packed_size(qx.Q8_0, 4, 64) == (qx.OK, 4 * 2 * 34)
    assert qx.qgemv_packed_size(qx.Q4_0, 4, 64) == (qx.OK, 4 * 2 * 18)
    # a null pointer with a bad shape reports the shape (checked first)
    assert qx.lib.qx_qgemv(qx.Q8_0, None, None, None, 4, 33) == qx.INVALID_SHAPE
    x = np.zeros(32, np.float32)
    assert qx.lib.qx_qgemv(qx.Q8_0, None, x.ctypes.data, x.ctypes.data, 1, 32) == qx.INVALID_ARGUMENT
    assert qx.lib.qx_qgemm(qx.Q8_0, None, None, None, 0, 4, 32) == qx.INVALID_SHAPE
    assert qx.lib.qx_qgemm(qx.Q8_0, None, None, None, 1, 4, 32) == qx.INVALID_ARGUMENT


def test_int8_and_w8a32_validation_order(qx):
    w = np.zeros((2, 4), np.int8)
    x = np.zeros((1, 4), np.int8)
    ws = np.ones(2, np.float32)
    xs = np.ones(1, np.float32)
    # src/dispatch/int8_gemm.cpp:72-85: shape, then pointers, then finite scales
    assert qx.int8_gemm(w, x, ws, xs, 0, 2, 4)[0] == qx.INVALID_SHAPE
    assert qx.lib.qx_int8_gemm(None, None, None, None, None, None, None, 1, 2, 4, 0) == qx.INVALID_ARGUMENT
    assert qx.lib.qx_int8_gemm(w.ctypes.data, x.ctypes.data, ws.ctypes.data, xs.ctypes.data, None,
                               None, ws.ctypes.data, 1, 2, 4, 1) == qx.INVALID_ARGUMENT
    ws_bad = ws.copy()
    ws_bad[1] = np.nan
    assert qx.int8_gemm(w, x, ws_bad, xs, 1, 2, 4)[0] == qx.INVALID_ARGUMENT
    xf = np.zeros((1, 4), np.float32)
    assert qx.qgemm_w8a32(w, ws, xf, 0, 2, 4)[0] == qx.INVALID_SHAPE
    assert qx.qgemm_w8a32(w, ws_bad, xf, 1, 2, 4)[0] == qx.INVALID_ARGUMENT


def test_w8a8_fused_and_lowbit_validation_order(qx):
    """Checks the reference makes before it touches any data, in its order
    (src/dispatch/qgemv_w8a8.cpp:131-146; kernels/quantization/qgemv_fused_ref.cpp:195-210,
    288-300; kernels/quantization/lowbit_ref.cpp:203-222, 258-272, 366-380;
    src/dispatch/lowbit_w8a8.cpp:68-80; quantization_ref.cpp:143-147)."""
    x = np.zeros(64, np.float32)
    y = np.zeros(4, np.float32)
    packed = np.zeros(4 * 2 * 34, np.uint8)
    P = lambda a: a.ctypes.data  # noqa: E731
    assert qx.lib.qx_qgemv_w8a8(qx.Q8_0, None, None, None, 4, 33) == qx.INVALID_SHAPE
    assert qx.lib.qx_qgemv_w8a8(11, P(packed), P(x), P(y), 4, 64) == qx.UNSUPPORTED_FORMAT
    assert qx.lib.qx_qgemv_w8a8(qx.Q8_0, P(packed), None, P(y), 4, 64) == qx.INVALID_ARGUMENT
    bad = x.copy()
    bad[3] = np.inf
    assert qx.lib.qx_qgemv_w8a8(qx.Q8_0, P(packed), P(bad), P(y), 4, 64) == qx.INVALID_ARGUMENT
    size = C.c_longlong(0)
    assert qx.lib.qx_qgemv_w8a8_packed_size(qx.Q4_0, 4, 64, C.byref(size)) == qx.OK and size.value == 4 * 2 * 18
    assert qx.lib.qx_qgemv_w8a8_packed_size(qx.Q4_0, 4, 64, None) == qx.INVALID_ARGUMENT
    assert qx.lib.qx_qgemv_w8a8_variant(3).decode() == "unsupported"
    # fused projections: shape, then pointers, then format / layout
    assert qx.lib.qx_qgemv_up_gate(qx.Q8_0, None, None, None, None, None, 0, 64) == qx.INVALID_SHAPE
    assert qx.lib.qx_qgemv_up_gate(qx.Q8_0, P(packed), None, P(x), P(y), P(y), 4, 64) == qx.INVALID_ARGUMENT
    assert qx.lib.qx_qgemv_up_gate(9, P(packed), P(packed), P(x), P(y), P(y), 4, 64) == qx.UNSUPPORTED_FORMAT
    assert qx.lib.qx_qgemv_up_gate(qx.Q8_0, P(packed), P(packed), P(x), P(y), P(y), 4, 65) == qx.INVALID_SHAPE
    assert qx.lib.qx_qgemv_up_gate_activation(qx.Q8_0, P(packed), P(packed), P(x), None, 4, 64, 1) == qx.INVALID_ARGUMENT
    assert qx.lib.qx_qgemv_qkv(qx.Q8_0, None, None, None, None, None, None, None, 4, 0, 64) == qx.INVALID_SHAPE
    assert qx.lib.qx_qgemv_qkv(qx.Q8_0, P(packed), P(packed), None, P(x), P(y), P(y), P(y), 4, 4, 64) == qx.INVALID_ARGUMENT
    # compact int4 rows
    assert qx.lowbit_packed_size(qx.LOWBIT_INT4_ROW, 3, 33) == (qx.OK, 3 * 17, 3)
    assert qx.lowbit_packed_size(qx.LOWBIT_INT4_GROUP, 3, 130, 64) == (qx.OK, 3 * 65, 9)
    assert qx.lowbit_packed_size(qx.LOWBIT_INT2_ROW, 2, 9) == (qx.OK, 2 * 3, 2)
    assert qx.lowbit_packed_size(qx.LOWBIT_INT3_GROUP64, 2, 65) == (qx.OK, 2 * 48, 4)
    assert qx.lowbit_packed_size(qx.LOWBIT_INT4_GROUP, 3, 130, 0)[0] == qx.INVALID_SHAPE
    assert qx.lowbit_packed_size(7, 3, 130, 0)[0] == qx.INVALID_SHAPE
    assert qx.lib.qx_lowbit_packed_size(qx.LOWBIT_INT4_ROW, 3, 33, 0, None, None) == qx.INVALID_ARGUMENT
    w4 = np.zeros(3 * 17, np.uint8)
    s4 = np.ones(3, np.float32)
    xf = np.zeros((2, 33), np.float32)
    yf = np.zeros((2, 3), np.float32)
    assert qx.lib.qx_lowbit_gemm(qx.LOWBIT_INT4_ROW, P(w4), P(s4), P(xf), P(yf), 2, 0, 33, 0) == qx.INVALID_SHAPE
    assert qx.lib.qx_lowbit_gemm(qx.LOWBIT_INT4_ROW, None, P(s4), P(xf), P(yf), 2, 3, 33, 0) == qx.INVALID_ARGUMENT
    s_bad = s4.copy()
    s_bad[1] = np.nan
    assert qx.lib.qx_lowbit_gemm(qx.LOWBIT_INT4_ROW, P(w4), P(s_bad), P(xf), P(yf), 2, 3, 33, 0) == qx.INVALID_ARGUMENT
    assert qx.lib.qx_lowbit_gemm(qx.LOWBIT_INT4_ROW, P(w4), P(s4), None, P(yf), 2, 3, 33, 0) == qx.INVALID_ARGUMENT
    assert qx.lib.qx_lowbit_gemm_w8a8(P(w4), P(s4), P(xf), P(yf), 2, 3, 0) == qx.INVALID_SHAPE
    assert qx.lib.qx_lowbit_gemm_w8a8(None, P(s4), P(xf), P(yf), 2, 3, 33) == qx.INVALID_ARGUMENT
    x_bad = xf.copy()
    x_bad[1, 2] = np.nan
    assert qx.lib.qx_lowbit_gemm_w8a8(P(w4), P(s4), P(x_bad), P(yf), 2, 3, 33) == qx.INVALID_ARGUMENT
    codes = np.zeros((2, 33), np.int8)
    sc = np.zeros(2, np.float32)
    assert qx.lib.qx_quantize_int8(P(xf), P(codes), P(sc), 2, 33, 16) == qx.INVALID_SHAPE
    assert qx.lib.qx_quantize_int8(None, P(codes), P(sc), 2, 33, 0) == qx.INVALID_ARGUMENT
    assert qx.lib.qx_quantize_int8(P(x_bad), P(codes), P(sc), 2, 33, 0) == qx.INVALID_ARGUMENT


def test_variant_names_and_threads(qx):
    v = qx.variants()
    assert v["qgemv_q8_0"].startswith("sm100a") and v["qgemv_q4_0"].startswith("sm100a")
    assert v["int8_gemm"].startswith("sm100a") and v["qgemm_w8a32"].startswith("sm100a")
    assert qx.lib.qx_qgemv_variant(17).decode() == "unsupported"
    qx.lib.qx_set_num_threads(0)
    assert qx.lib.qx_num_threads() == 1  # clamps like the reference (threading.h:6-8)
    qx.lib.qx_set_num_threads(8)
    assert qx.lib.qx_num_threads() == 8
    qx.lib.qx_set_num_threads(1)


def test_no_cpu_fallback_without_device(qx):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; the loud-failure path is for GPU-less hosts")
    w = np.zeros((2, 32), np.int8)
    x = np.zeros((1, 32), np.int8)
    status, _ = qx.qgemm_w8a8(w, x, np.ones(2, np.float32), np.ones(1, np.float32), 1, 2, 32)
    assert status == qx.DEVICE_ERROR
    assert "no CUDA device" in qx.last_error()
    packed = np.zeros(34, np.uint8)
    status, _ = qx.qgemv(qx.Q8_0, packed, np.zeros(32, np.float32), 1, 32)
    assert status == qx.DEVICE_ERROR


def test_product_sources_do_not_touch_the_oracle():
    """Nothing under the package or include/ may import, link or call oracle/."""
    pkg = os.path.join(ROOT, "quixicore-cpu_b200")
    for folder, _, files in os.walk(pkg):
        if os.path.basename(folder) == "build":
            continue
        for name in files:
            if name.endswith((".py", ".cu", ".cuh", ".h", ".hpp")):
                text = open(os.path.join(folder, name)).read()
                assert "qxo_" not in text and "qxref_" not in text and "libqx_oracle" not in text, name
                assert not re.search(r"^\s*(import|from)\s+oracle\b", text, re.M), name
