"""TEST INFRASTRUCTURE ONLY: ctypes bindings of the two CPU checkers.

``Oracle`` binds ``oracle/libqx_oracle.so`` (the plain-C restatement in
``qx_oracle.c``); ``Reference`` binds ``oracle/_ref/libqx_ref.so`` (the unmodified
QuixiCore-CPU library built by ``oracle/Makefile``) when that file exists. Only the
tests, the smoke check and the CPU-baseline legs of the benchmark import this module;
the product package never does.
"""

from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libqx_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libqx_ref.so")

Q8_0, Q4_0 = 0, 1
BLOCK_BYTES = {Q8_0: 34, Q4_0: 18}
OK, INVALID_SHAPE, UNSUPPORTED_FORMAT, INVALID_ARGUMENT, OUT_OF_MEMORY = range(5)

_ll = C.c_longlong
_vp = C.c_void_p


def reference_root() -> str:
    """Where the reference project's sources are looked for: $QX_REFERENCE_ROOT, else a
    checkout named `reference` beside this repository."""
    return os.environ.get("QX_REFERENCE_ROOT") or os.path.join(
        os.path.dirname(os.path.dirname(HERE)), "reference")


def build(reference_root: str | None = None) -> None:
    """Compile the C restatement, and the reference library when its sources exist."""
    reference_root = reference_root or globals()["reference_root"]()
    subprocess.check_call(["make", "-s", "-C", HERE, "oracle"])
    if os.path.isdir(reference_root):
        subprocess.check_call(
            ["make", "-s", "-j8", "-C", HERE, "ref", f"REF={reference_root}"])


def _ptr(array):
    if array is None:
        return None
    assert array.flags["C_CONTIGUOUS"]
    return array.ctypes.data_as(_vp)


def packed_size(fmt: int, n: int, k: int) -> int:
    return n * (k // 32) * BLOCK_BYTES[fmt]


# storage element types of FloatStorageType (f16 / bf16 travel as their 16-bit patterns)
STORAGE_DTYPES = {0: np.float32, 1: np.uint16, 2: np.uint16}


class CanonicalTensor:
    """The fields of a CanonicalQuantTensor the projections read."""

    def __init__(self, layout, scale_mode, rows, columns, group_size, data, scales, zeros=None,
                 group_index=None, act_order=None):
        self.layout, self.scale_mode = layout, scale_mode
        self.rows, self.columns, self.group_size = rows, columns, group_size
        self.data = np.ascontiguousarray(data, np.uint8).reshape(-1)
        self.scales = np.ascontiguousarray(scales, np.float32).reshape(-1)
        self.zeros = None if zeros is None else np.ascontiguousarray(zeros, np.float32).reshape(-1)
        self.group_index = None if group_index is None else np.ascontiguousarray(group_index, np.int32)
        self.act_order = None if act_order is None else np.ascontiguousarray(act_order, np.int32)

    def extras(self):
        """(zeros, count, group_index, count, act_order, count) as ctypes arguments"""
        def pair(a):
            return (_ptr(a), 0 if a is None else a.size)
        return pair(self.zeros) + pair(self.group_index) + pair(self.act_order)

    @property
    def plain(self):
        return self.zeros is None and self.group_index is None and self.act_order is None


class Oracle:
    """Plain-C restatement (qx_oracle.c)."""

    def __init__(self, path: str = ORACLE_SO):
        if not os.path.exists(path):
            build()
        self.lib = L = C.CDLL(path)
        L.qxo_fp16_to_fp32.restype = C.c_float
        L.qxo_fp16_to_fp32.argtypes = [C.c_uint16]
        L.qxo_fp32_to_fp16.restype = C.c_uint16
        L.qxo_fp32_to_fp16.argtypes = [C.c_float]
        L.qxo_float_to_bf16.restype = C.c_uint16
        L.qxo_float_to_bf16.argtypes = [C.c_float]
        L.qxo_bf16_to_float.restype = C.c_float
        L.qxo_bf16_to_float.argtypes = [C.c_uint16]
        L.qxo_qgemv_packed_size.argtypes = [C.c_int, _ll, _ll, C.POINTER(C.c_size_t)]
        L.qxo_qgemv_pack.argtypes = [C.c_int, _vp, _ll, _ll, _vp]
        L.qxo_qgemv_unpack.argtypes = [C.c_int, _vp, _ll, _ll, _vp]
        L.qxo_qgemv.argtypes = [C.c_int, _vp, _vp, _vp, _ll, _ll, C.c_int]
        L.qxo_qgemm.argtypes = [C.c_int, _vp, _vp, _vp, _ll, _ll, _ll, C.c_int]
        L.qxo_qgemm_f64.argtypes = [C.c_int, _vp, _vp, _vp, _ll, _ll, _ll]
        L.qxo_int8_gemm.argtypes = [_vp] * 8 + [_ll, _ll, _ll, C.c_int]
        L.qxo_qgemm_w8a32.argtypes = [_vp] * 4 + [_ll, _ll, _ll]
        L.qxo_qgemm_w8a32_avx512_order.argtypes = [_vp] * 4 + [_ll, _ll, _ll]
        L.qxo_qgemm_w8a32_f64.argtypes = [_vp] * 4 + [_ll, _ll, _ll]
        L.qxo_qgemm_w8a32_f64.restype = None
        L.qxo_panel_bytes.restype = _ll
        L.qxo_panel_bytes.argtypes = [C.c_int, _ll, _ll, _ll]
        L.qxo_build_panel.argtypes = [C.c_int, _vp, _ll, _ll, _ll, _vp]
        L.qxo_qgemv_w8a8.argtypes = [C.c_int, _vp, _vp, _vp, _ll, _ll, _vp, _vp]
        L.qxo_gate_activation.argtypes = [_vp, _vp, _vp, _ll, C.c_int]
        L.qxo_gate_activation.restype = None
        L.qxo_quantize_int8.argtypes = [_vp, _vp, _vp, _ll, _ll, _ll]
        L.qxo_lowbit_pack.argtypes = [C.c_int, _vp, _vp, _vp, _ll, _ll, _ll]
        L.qxo_lowbit_unpack.argtypes = [C.c_int, _vp, _vp, _vp, _ll, _ll, _ll]
        L.qxo_lowbit_gemm.argtypes = [C.c_int, _vp, _vp, _vp, _vp, _ll, _ll, _ll, _ll]
        L.qxo_lowbit_gemm_f64.argtypes = [C.c_int, _vp, _vp, _vp, _vp, _ll, _ll, _ll, _ll]
        L.qxo_lowbit_gemm_w8a8.argtypes = [_vp, _vp, _vp, _vp, _ll, _ll, _ll, _vp, _vp]
        L.qxo_quantize_canonical.argtypes = [C.c_int, _vp, _ll, _ll, _ll, _vp, _vp,
                                             C.POINTER(C.c_int), C.POINTER(_ll)]
        L.qxo_canonical_gemm.argtypes = [C.c_int, C.c_int, _ll, _ll, _ll, _vp, C.c_size_t, _vp,
                                         C.c_size_t, _vp, C.c_int, _ll, _vp, _vp, C.c_int, _ll,
                                         _ll, C.c_int]
        L.qxo_canonical_gemm_ex.argtypes = [C.c_int, C.c_int, _ll, _ll, _ll, _vp, C.c_size_t, _vp,
                                            C.c_size_t, _vp, C.c_size_t, _vp, C.c_size_t, _vp,
                                            C.c_size_t, _vp, C.c_int, _ll, _vp, _vp, C.c_int, _ll,
                                            _ll, C.c_int]
        L.qxo_canonical_gemm_ex_f64.argtypes = [C.c_int, _ll, _ll, _ll, _vp, _vp, _vp, _vp, _vp, _vp,
                                                C.c_int, _vp, _ll]
        L.qxo_canonical_gemm_f64.argtypes = [C.c_int, _ll, _ll, _ll, _vp, _vp, _vp, C.c_int, _vp, _ll]
        L.qxo_import_smoothquant_row_sums.argtypes = [_vp, C.c_size_t, _vp, C.c_size_t, _vp,
                                                      C.c_size_t, _vp, C.c_size_t, _ll, _ll, _vp]

    # scalar conversions
    def fp16_to_fp32(self, h):
        return self.lib.qxo_fp16_to_fp32(h)

    def fp32_to_fp16(self, v):
        return self.lib.qxo_fp32_to_fp16(v)

    def float_to_bf16(self, v):
        return self.lib.qxo_float_to_bf16(v)

    def bf16_to_float(self, h):
        return self.lib.qxo_bf16_to_float(h)

    def qgemv_packed_size(self, fmt, n, k, want_size=True):
        size = C.c_size_t(0)
        status = self.lib.qxo_qgemv_packed_size(
            fmt, n, k, C.byref(size) if want_size else None)
        return status, size.value

    def pack(self, fmt, weights, n, k):
        packed = np.zeros(packed_size(fmt, n, k), np.uint8)
        status = self.lib.qxo_qgemv_pack(fmt, _ptr(weights), n, k, _ptr(packed))
        return status, packed

    def unpack(self, fmt, packed, n, k):
        out = np.zeros((n, k), np.float32)
        status = self.lib.qxo_qgemv_unpack(fmt, _ptr(packed), n, k, _ptr(out))
        return status, out

    def qgemv(self, fmt, packed, x, n, k, q4_variant=0):
        y = np.zeros(n, np.float32)
        status = self.lib.qxo_qgemv(fmt, _ptr(packed), _ptr(x), _ptr(y), n, k, q4_variant)
        return status, y

    def qgemm(self, fmt, packed, x, m, n, k, q4_variant=0):
        y = np.zeros((m, n), np.float32)
        status = self.lib.qxo_qgemm(fmt, _ptr(packed), _ptr(x), _ptr(y), m, n, k, q4_variant)
        return status, y

    def qgemm_f64(self, fmt, packed, x, m, n, k):
        y = np.zeros((m, n), np.float64)
        status = self.lib.qxo_qgemm_f64(fmt, _ptr(packed), _ptr(x), _ptr(y), m, n, k)
        return status, y

    def int8_gemm(self, w, x, ws, xs, m, n, k, row_sum=None, zp=None, asymmetric=False):
        y = np.zeros((m, n), np.float32)
        acc = np.zeros((m, n), np.int64)
        status = self.lib.qxo_int8_gemm(_ptr(w), _ptr(x), _ptr(ws), _ptr(xs), _ptr(row_sum),
                                        _ptr(zp), _ptr(y), _ptr(acc), m, n, k,
                                        1 if asymmetric else 0)
        return status, y, acc

    def qgemm_w8a32(self, w, ws, x, m, n, k, avx512_order=False):
        y = np.zeros((m, n), np.float32)
        fn = self.lib.qxo_qgemm_w8a32_avx512_order if avx512_order else self.lib.qxo_qgemm_w8a32
        status = fn(_ptr(w), _ptr(ws), _ptr(x), _ptr(y), m, n, k)
        return status, y

    def qgemm_w8a32_f64(self, w, ws, x, m, n, k):
        y = np.zeros((m, n), np.float64)
        self.lib.qxo_qgemm_w8a32_f64(_ptr(w), _ptr(ws), _ptr(x), _ptr(y), m, n, k)
        return y

    # ---- callers either side of the GEMV
    def qgemv_w8a8(self, fmt, packed, x, n, k):
        y = np.zeros(n, np.float32)
        codes, scales = np.zeros(max(k, 1), np.int8), np.zeros(max(k // 32, 1), np.float32)
        status = self.lib.qxo_qgemv_w8a8(fmt, _ptr(packed), _ptr(x), _ptr(y), n, k, _ptr(codes),
                                         _ptr(scales))
        return status, y

    def gate_activation(self, up, gate, gelu_tanh=True):
        out = np.zeros_like(up)
        self.lib.qxo_gate_activation(_ptr(up), _ptr(gate), _ptr(out), up.size, 1 if gelu_tanh else 0)
        return out

    def quantize_int8(self, x, rows, dim, group_size=0):
        groups = dim // (group_size or dim)
        codes, scales = np.zeros((rows, dim), np.int8), np.zeros((rows, groups), np.float32)
        status = self.lib.qxo_quantize_int8(_ptr(x), _ptr(codes), _ptr(scales), rows, dim, group_size)
        return status, codes, scales

    def lowbit_pack(self, fmt, weights, rows, dim, group_size=0):
        groups = 1 if fmt == 2 else -(-dim // group_size)
        packed = np.zeros(rows * ((dim + 1) // 2), np.uint8)
        scales = np.zeros((rows, groups), np.float32)
        status = self.lib.qxo_lowbit_pack(fmt, _ptr(weights), _ptr(packed), _ptr(scales), rows, dim,
                                          group_size)
        return status, packed, scales

    def lowbit_unpack(self, fmt, packed, scales, rows, dim, group_size=0):
        out = np.zeros((rows, dim), np.float32)
        status = self.lib.qxo_lowbit_unpack(fmt, _ptr(packed), _ptr(scales), _ptr(out), rows, dim,
                                            group_size)
        return status, out

    def lowbit_gemm(self, fmt, packed, scales, x, m, n, k, group_size=0):
        y = np.zeros((m, n), np.float32)
        status = self.lib.qxo_lowbit_gemm(fmt, _ptr(packed), _ptr(scales), _ptr(x), _ptr(y), m, n, k,
                                          group_size)
        return status, y

    def lowbit_gemm_f64(self, fmt, packed, scales, x, m, n, k, group_size=0):
        y = np.zeros((m, n), np.float64)
        status = self.lib.qxo_lowbit_gemm_f64(fmt, _ptr(packed), _ptr(scales), _ptr(x), _ptr(y), m, n,
                                              k, group_size)
        return status, y

    def lowbit_gemm_w8a8(self, packed, scales, x, m, n, k):
        y = np.zeros((m, n), np.float32)
        codes, act = np.zeros(m * k, np.int8), np.zeros(m, np.float32)
        status = self.lib.qxo_lowbit_gemm_w8a8(_ptr(packed), _ptr(scales), _ptr(x), _ptr(y), m, n, k,
                                               _ptr(codes), _ptr(act))
        return status, y

    def build_panel(self, fmt, packed, rows, cols, tile):
        size = self.lib.qxo_panel_bytes(fmt, rows, cols, tile)
        panel = np.full(max(size, 1), 0xAB, np.uint8)
        status = self.lib.qxo_build_panel(fmt, _ptr(packed), rows, cols, tile, _ptr(panel))
        return status, panel[:max(size, 0)]


    # ---- canonical prepared projections (kInt8Symmetric = 2, kInt4Symmetric = 0)
    def quantize_canonical(self, layout, values, rows, columns, group_size=0):
        """-> status, CanonicalTensor"""
        data = np.zeros(rows * columns // (1 if layout == 2 else 2), np.uint8)
        groups = columns // (group_size or columns)
        scales = np.zeros(rows * groups, np.float32)
        mode, stored = C.c_int(0), _ll(0)
        status = self.lib.qxo_quantize_canonical(layout, _ptr(values), rows, columns, group_size,
                                                 _ptr(data), _ptr(scales), C.byref(mode),
                                                 C.byref(stored))
        return status, CanonicalTensor(layout, mode.value, rows, columns, stored.value, data, scales)

    def canonical_gemm(self, t, x, x_type, m, bias=None, y_type=0, activation=0,
                       x_count=None, y_count=None):
        y = np.zeros(max(m, 1) * t.rows, STORAGE_DTYPES.get(y_type, np.float32))
        x_count = m * t.columns if x_count is None else x_count
        y_count = m * t.rows if y_count is None else y_count
        if t.plain and t.layout != 1:
            status = self.lib.qxo_canonical_gemm(
                t.layout, t.scale_mode, t.rows, t.columns, t.group_size, _ptr(t.data), t.data.size,
                _ptr(t.scales), t.scales.size, _ptr(x), x_type, x_count, _ptr(bias), _ptr(y),
                y_type, y_count, m, activation)
        else:
            status = self.lib.qxo_canonical_gemm_ex(
                t.layout, t.scale_mode, t.rows, t.columns, t.group_size, _ptr(t.data), t.data.size,
                _ptr(t.scales), t.scales.size, *t.extras(), _ptr(x), x_type, x_count, _ptr(bias),
                _ptr(y), y_type, y_count, m, activation)
        return status, y.reshape(max(m, 1), t.rows)

    def canonical_gemm_f64(self, t, x, x_type, m):
        y = np.zeros((m, t.rows), np.float64)
        self.lib.qxo_canonical_gemm_ex_f64(t.layout, t.rows, t.columns, t.scales.size // t.rows,
                                           _ptr(t.data), _ptr(t.scales), _ptr(t.zeros),
                                           _ptr(t.group_index), _ptr(t.act_order), _ptr(x), x_type,
                                           _ptr(y), m)
        return y

    def import_smoothquant_row_sums(self, weights, weight_scales, activation_scales, rows, columns,
                                    row_sums=None):
        out = np.zeros(rows, np.int32)
        status = self.lib.qxo_import_smoothquant_row_sums(
            _ptr(weights), weights.size, _ptr(weight_scales), weight_scales.size,
            _ptr(activation_scales), activation_scales.size, _ptr(row_sums),
            0 if row_sums is None else row_sums.size, rows, columns, _ptr(out))
        return status, out


class Reference:
    """The unmodified reference library behind oracle/ref_shim.cpp."""

    @staticmethod
    def available(path: str = REF_SO) -> bool:
        return os.path.exists(path)

    def __init__(self, path: str = REF_SO):
        self.lib = L = C.CDLL(path)
        L.qxref_qgemv_packed_size.argtypes = [C.c_int, _ll, _ll, C.POINTER(C.c_size_t)]
        L.qxref_qgemv_pack.argtypes = [C.c_int, _vp, _ll, _ll, _vp]
        L.qxref_qgemv_unpack.argtypes = [C.c_int, _vp, _ll, _ll, _vp]
        L.qxref_qgemv.argtypes = [C.c_int, _vp, _vp, _vp, _ll, _ll]
        L.qxref_qgemm.argtypes = [C.c_int, _vp, _vp, _vp, _ll, _ll, _ll]
        L.qxref_int8_gemm.argtypes = [_vp] * 7 + [_ll, _ll, _ll, C.c_int]
        L.qxref_qgemm_w8a8.argtypes = [_vp] * 5 + [_ll, _ll, _ll]
        L.qxref_qgemm_w8a32.argtypes = [_vp] * 4 + [_ll, _ll, _ll]
        L.qxref_quantize_canonical.argtypes = [C.c_int, _vp, _ll, _ll, _ll, _vp, C.c_size_t, _vp,
                                               C.c_size_t, C.POINTER(C.c_size_t),
                                               C.POINTER(C.c_size_t), C.POINTER(C.c_int),
                                               C.POINTER(_ll)]
        L.qxref_canonical_validate.argtypes = [C.c_int, C.c_int, _ll, _ll, _ll, _vp, C.c_size_t,
                                               _vp, C.c_size_t]
        L.qxref_canonical_gemm.argtypes = [C.c_int, C.c_int, _ll, _ll, _ll, _vp, C.c_size_t, _vp,
                                           C.c_size_t, _vp, C.c_int, _ll, _vp, _vp, C.c_int, _ll,
                                           _ll, C.c_int]
        L.qxref_canonical_gemm_ex.argtypes = [C.c_int, C.c_int, _ll, _ll, _ll, _vp, C.c_size_t, _vp,
                                              C.c_size_t, _vp, C.c_size_t, _vp, C.c_size_t, _vp,
                                              C.c_size_t, _vp, C.c_int, _ll, _vp, _vp, C.c_int, _ll,
                                              _ll, C.c_int]
        L.qxref_import_awq_u4.argtypes = [_vp, C.c_size_t, _vp, C.c_size_t, _vp, C.c_size_t, _ll, _ll,
                                          _ll, _vp, _vp, _vp, _vp]
        L.qxref_import_gptq_u4.argtypes = [_vp, C.c_size_t, _vp, C.c_size_t, _vp, C.c_size_t, _vp,
                                           C.c_size_t, _vp, C.c_size_t, _ll, _ll, _ll, C.c_int,
                                           C.c_int, _vp, _vp, _vp, _vp]
        L.qxref_import_smoothquant.argtypes = [_vp, C.c_size_t, _vp, C.c_size_t, _vp, C.c_size_t,
                                               _vp, C.c_size_t, _vp, C.c_size_t, _ll, _ll, _vp, _vp,
                                               _vp, C.POINTER(C.c_int), C.POINTER(C.c_int),
                                               C.POINTER(_ll)]
        L.qxref_packed_create.argtypes = [C.c_int, _vp, _ll, _ll, C.c_int, C.POINTER(_vp)]
        L.qxref_packed_destroy.argtypes = [_vp]
        L.qxref_packed_destroy.restype = None
        L.qxref_packed_info.argtypes = [_vp, C.POINTER(_ll)]
        L.qxref_packed_info.restype = None
        L.qxref_packed_panel.argtypes = [_vp]
        L.qxref_packed_panel.restype = _vp
        L.qxref_qgemm_prepacked.argtypes = [_vp, _vp, _vp, _ll]
        L.qxref_set_num_threads.argtypes = [C.c_int]
        L.qxref_set_num_threads.restype = None
        L.qxref_qgemv_variant.restype = C.c_char_p
        L.qxref_qgemv_variant.argtypes = [C.c_int]
        L.qxref_int8_gemm_variant.restype = C.c_char_p
        L.qxref_qgemm_w8a32_variant.restype = C.c_char_p
        L.qxref_fp16_to_fp32.restype = C.c_float
        L.qxref_fp16_to_fp32.argtypes = [C.c_uint16]
        L.qxref_fp32_to_fp16.restype = C.c_uint16
        L.qxref_fp32_to_fp16.argtypes = [C.c_float]
        L.qxref_float_to_bf16.restype = C.c_uint16
        L.qxref_float_to_bf16.argtypes = [C.c_float]
        L.qxref_bf16_to_float.restype = C.c_float
        L.qxref_bf16_to_float.argtypes = [C.c_uint16]
        # a library built before these entry points were added lacks them: rebuild it
        if hasattr(L, "qxref_qgemv_w8a8"):
            L.qxref_qgemv_w8a8.argtypes = [C.c_int, _vp, _vp, _vp, _ll, _ll]
            L.qxref_qgemv_w8a8_variant.restype = C.c_char_p
            L.qxref_qgemv_w8a8_variant.argtypes = [C.c_int]
            L.qxref_qgemv_up_gate.argtypes = [C.c_int, _vp, _vp, _vp, _vp, _vp, _ll, _ll]
            L.qxref_qgemv_up_gate_activation.argtypes = [C.c_int, _vp, _vp, _vp, _vp, _ll, _ll, C.c_int]
            L.qxref_qgemv_qkv.argtypes = [C.c_int] + [_vp] * 7 + [_ll, _ll, _ll]
            L.qxref_quantize_int8.argtypes = [_vp, _vp, _vp, _ll, _ll, _ll]
            L.qxref_lowbit_packed_size.argtypes = [C.c_int, _ll, _ll, _ll, C.POINTER(C.c_size_t),
                                                   C.POINTER(C.c_size_t)]
            L.qxref_lowbit_pack.argtypes = [C.c_int, _vp, _vp, _vp, _ll, _ll, _ll]
            L.qxref_lowbit_unpack.argtypes = [C.c_int, _vp, _vp, _vp, _ll, _ll, _ll]
            L.qxref_lowbit_gemm.argtypes = [C.c_int, _vp, _vp, _vp, _vp, _ll, _ll, _ll, _ll]
            L.qxref_lowbit_gemm_w8a8.argtypes = [_vp, _vp, _vp, _vp, _ll, _ll, _ll]
            L.qxref_lowbit_gemm_w8a8_variant.restype = C.c_char_p
            L.qxref_lowbit_gemm_variant.restype = C.c_char_p
            L.qxref_lowbit_gemm_variant.argtypes = [C.c_int]

    # ---- callers either side of the GEMV
    def qgemv_w8a8(self, fmt, packed, x, n, k):
        y = np.zeros(n, np.float32)
        return self.lib.qxref_qgemv_w8a8(fmt, _ptr(packed), _ptr(x), _ptr(y), n, k), y

    def up_gate(self, fmt, up_w, gate_w, x, n, k):
        up, gate = np.zeros(n, np.float32), np.zeros(n, np.float32)
        status = self.lib.qxref_qgemv_up_gate(fmt, _ptr(up_w), _ptr(gate_w), _ptr(x), _ptr(up),
                                              _ptr(gate), n, k)
        return status, up, gate

    def up_gate_activation(self, fmt, up_w, gate_w, x, n, k, gelu_tanh=True):
        out = np.zeros(n, np.float32)
        status = self.lib.qxref_qgemv_up_gate_activation(fmt, _ptr(up_w), _ptr(gate_w), _ptr(x),
                                                         _ptr(out), n, k, 1 if gelu_tanh else 0)
        return status, out

    def qkv(self, fmt, wq, wk, wv, x, query_dim, kv_dim, input_dim):
        q, k_out, v_out = (np.zeros(query_dim, np.float32), np.zeros(kv_dim, np.float32),
                           np.zeros(kv_dim, np.float32))
        status = self.lib.qxref_qgemv_qkv(fmt, _ptr(wq), _ptr(wk), _ptr(wv), _ptr(x), _ptr(q),
                                          _ptr(k_out), _ptr(v_out), query_dim, kv_dim, input_dim)
        return status, q, k_out, v_out

    def quantize_int8(self, x, rows, dim, group_size=0):
        groups = dim // (group_size or dim)
        codes, scales = np.zeros((rows, dim), np.int8), np.zeros((rows, groups), np.float32)
        status = self.lib.qxref_quantize_int8(_ptr(x), _ptr(codes), _ptr(scales), rows, dim, group_size)
        return status, codes, scales

    def lowbit_packed_size(self, fmt, rows, dim, group_size=0):
        wb, sc = C.c_size_t(0), C.c_size_t(0)
        status = self.lib.qxref_lowbit_packed_size(fmt, rows, dim, group_size, C.byref(wb), C.byref(sc))
        return status, wb.value, sc.value

    def lowbit_pack(self, fmt, weights, rows, dim, group_size=0):
        groups = 1 if fmt == 2 else -(-dim // group_size)
        packed = np.zeros(rows * ((dim + 1) // 2), np.uint8)
        scales = np.zeros((rows, groups), np.float32)
        status = self.lib.qxref_lowbit_pack(fmt, _ptr(weights), _ptr(packed), _ptr(scales), rows, dim,
                                            group_size)
        return status, packed, scales

    def lowbit_unpack(self, fmt, packed, scales, rows, dim, group_size=0):
        out = np.zeros((rows, dim), np.float32)
        status = self.lib.qxref_lowbit_unpack(fmt, _ptr(packed), _ptr(scales), _ptr(out), rows, dim,
                                              group_size)
        return status, out

    def lowbit_gemm(self, fmt, packed, scales, x, m, n, k, group_size=0):
        y = np.zeros((m, n), np.float32)
        status = self.lib.qxref_lowbit_gemm(fmt, _ptr(packed), _ptr(scales), _ptr(x), _ptr(y), m, n, k,
                                            group_size)
        return status, y

    def lowbit_gemm_w8a8(self, packed, scales, x, m, n, k):
        y = np.zeros((m, n), np.float32)
        status = self.lib.qxref_lowbit_gemm_w8a8(_ptr(packed), _ptr(scales), _ptr(x), _ptr(y), m, n, k)
        return status, y

    # ---- canonical prepared projections
    def quantize_canonical(self, layout, values, rows, columns, group_size=0):
        data = np.zeros(rows * columns, np.uint8)
        scales = np.zeros(rows * columns, np.float32)
        nb, ns, mode, stored = C.c_size_t(0), C.c_size_t(0), C.c_int(0), _ll(0)
        status = self.lib.qxref_quantize_canonical(
            layout, _ptr(values), rows, columns, group_size, _ptr(data), data.size, _ptr(scales),
            scales.size, C.byref(nb), C.byref(ns), C.byref(mode), C.byref(stored))
        return status, CanonicalTensor(layout, mode.value, rows, columns, stored.value,
                                       data[:nb.value].copy(), scales[:ns.value].copy())

    def canonical_validate(self, t, data_bytes=None, scale_count=None):
        return self.lib.qxref_canonical_validate(
            t.layout, t.scale_mode, t.rows, t.columns, t.group_size, _ptr(t.data),
            t.data.size if data_bytes is None else data_bytes, _ptr(t.scales),
            t.scales.size if scale_count is None else scale_count)

    def canonical_gemm(self, t, x, x_type, m, bias=None, y_type=0, activation=0,
                       x_count=None, y_count=None):
        y = np.zeros(max(m, 1) * t.rows, STORAGE_DTYPES.get(y_type, np.float32))
        status = self.lib.qxref_canonical_gemm(
            t.layout, t.scale_mode, t.rows, t.columns, t.group_size, _ptr(t.data), t.data.size,
            _ptr(t.scales), t.scales.size, _ptr(x), x_type,
            m * t.columns if x_count is None else x_count, _ptr(bias), _ptr(y), y_type,
            m * t.rows if y_count is None else y_count, m, activation)
        return status, y.reshape(max(m, 1), t.rows)

    def canonical_gemm_ex(self, t, x, x_type, m, bias=None, y_type=0, activation=0):
        y = np.zeros(max(m, 1) * t.rows, STORAGE_DTYPES.get(y_type, np.float32))
        status = self.lib.qxref_canonical_gemm_ex(
            t.layout, t.scale_mode, t.rows, t.columns, t.group_size, _ptr(t.data), t.data.size,
            _ptr(t.scales), t.scales.size, *t.extras(), _ptr(x), x_type, m * t.columns, _ptr(bias),
            _ptr(y), y_type, m * t.rows, m, activation)
        return status, y.reshape(max(m, 1), t.rows)

    def _imported(self, status, n, k, group, data, scales, zeros, meta, group_index, act_order):
        if status != 0:
            return status, None
        groups = k // group
        zc = int(meta[3])
        return status, CanonicalTensor(int(meta[0]), int(meta[1]), n, k, int(meta[2]), data[:n * k // 2],
                                       scales[:n * groups], zeros[:zc] if zc else None,
                                       group_index if meta[4] else None, act_order if meta[5] else None)

    def import_awq_u4(self, qweight, qzeros, scales, k, n, group):
        data = np.zeros(max(n * k // 2, 1), np.uint8)
        out_scales = np.zeros(max(scales.size, 1), np.float32)
        zeros = np.zeros(max(scales.size, 1), np.float32)
        meta = np.zeros(6, np.int32)
        status = self.lib.qxref_import_awq_u4(_ptr(qweight), qweight.size, _ptr(qzeros), qzeros.size,
                                              _ptr(scales), scales.size, k, n, group, _ptr(data),
                                              _ptr(out_scales), _ptr(zeros), _ptr(meta))
        return self._imported(status, n, k, group, data, out_scales, zeros, meta, None, None)

    def import_gptq_u4(self, qweight, qzeros, scales, k, n, group, symmetric=False, v2=False,
                       group_index=None, act_order=None):
        data = np.zeros(max(n * k // 2, 1), np.uint8)
        out_scales = np.zeros(max(scales.size, 1), np.float32)
        zeros = np.zeros(max(scales.size, 1), np.float32)
        meta = np.zeros(6, np.int32)
        status = self.lib.qxref_import_gptq_u4(
            _ptr(qweight), qweight.size, _ptr(qzeros), qzeros.size, _ptr(scales), scales.size,
            _ptr(group_index), 0 if group_index is None else group_index.size, _ptr(act_order),
            0 if act_order is None else act_order.size, k, n, group, int(symmetric), int(v2),
            _ptr(data), _ptr(out_scales), _ptr(zeros), _ptr(meta))
        return self._imported(status, n, k, group, data, out_scales, zeros, meta, group_index, act_order)

    def import_smoothquant(self, weights, weight_scales, activation_scales, rows, columns,
                           zero_points=None, row_sums=None):
        data = np.zeros(rows * columns, np.uint8)
        scales = np.zeros(rows, np.float32)
        sums = np.zeros(rows, np.int32)
        layout, mode, group = C.c_int(-1), C.c_int(-1), _ll(-1)
        status = self.lib.qxref_import_smoothquant(
            _ptr(weights), weights.size, _ptr(weight_scales), weight_scales.size,
            _ptr(activation_scales), activation_scales.size, _ptr(zero_points),
            0 if zero_points is None else zero_points.size, _ptr(row_sums),
            0 if row_sums is None else row_sums.size, rows, columns, _ptr(data), _ptr(scales),
            _ptr(sums), C.byref(layout), C.byref(mode), C.byref(group))
        return status, CanonicalTensor(layout.value, mode.value, rows, columns, group.value, data,
                                       scales), sums

    def set_num_threads(self, n):
        self.lib.qxref_set_num_threads(int(n))

    def num_threads(self):
        return self.lib.qxref_num_threads()

    def variants(self):
        return {
            "qgemv_q8_0": self.lib.qxref_qgemv_variant(Q8_0).decode(),
            "qgemv_q4_0": self.lib.qxref_qgemv_variant(Q4_0).decode(),
            "int8_gemm": self.lib.qxref_int8_gemm_variant().decode(),
            "qgemm_w8a32": self.lib.qxref_qgemm_w8a32_variant().decode(),
        }

    def fp16_to_fp32(self, h):
        return self.lib.qxref_fp16_to_fp32(h)

    def fp32_to_fp16(self, v):
        return self.lib.qxref_fp32_to_fp16(v)

    def float_to_bf16(self, v):
        return self.lib.qxref_float_to_bf16(v)

    def bf16_to_float(self, h):
        return self.lib.qxref_bf16_to_float(h)

    def qgemv_packed_size(self, fmt, n, k, want_size=True):
        size = C.c_size_t(0)
        status = self.lib.qxref_qgemv_packed_size(
            fmt, n, k, C.byref(size) if want_size else None)
        return status, size.value

    def pack(self, fmt, weights, n, k):
        packed = np.zeros(packed_size(fmt, n, k), np.uint8)
        status = self.lib.qxref_qgemv_pack(fmt, _ptr(weights), n, k, _ptr(packed))
        return status, packed

    def unpack(self, fmt, packed, n, k):
        out = np.zeros((n, k), np.float32)
        status = self.lib.qxref_qgemv_unpack(fmt, _ptr(packed), n, k, _ptr(out))
        return status, out

    def qgemv(self, fmt, packed, x, n, k):
        y = np.zeros(n, np.float32)
        status = self.lib.qxref_qgemv(fmt, _ptr(packed), _ptr(x), _ptr(y), n, k)
        return status, y

    def qgemm(self, fmt, packed, x, m, n, k):
        y = np.zeros((m, n), np.float32)
        status = self.lib.qxref_qgemm(fmt, _ptr(packed), _ptr(x), _ptr(y), m, n, k)
        return status, y

    def int8_gemm(self, w, x, ws, xs, m, n, k, row_sum=None, zp=None, asymmetric=False):
        y = np.zeros((m, n), np.float32)
        status = self.lib.qxref_int8_gemm(_ptr(w), _ptr(x), _ptr(ws), _ptr(xs), _ptr(row_sum),
                                          _ptr(zp), _ptr(y), m, n, k, 1 if asymmetric else 0)
        return status, y

    def qgemm_w8a8(self, w, x, ws, xs, m, n, k):
        y = np.zeros((m, n), np.float32)
        status = self.lib.qxref_qgemm_w8a8(_ptr(w), _ptr(x), _ptr(ws), _ptr(xs), _ptr(y), m, n, k)
        return status, y

    def qgemm_w8a32(self, w, ws, x, m, n, k):
        y = np.zeros((m, n), np.float32)
        status = self.lib.qxref_qgemm_w8a32(_ptr(w), _ptr(ws), _ptr(x), _ptr(y), m, n, k)
        return status, y

    def prepacked(self, fmt, packed, rows, cols, layout=0):
        handle = _vp()
        status = self.lib.qxref_packed_create(fmt, _ptr(packed), rows, cols, layout,
                                              C.byref(handle))
        return status, handle

    def prepacked_info(self, handle):
        out = (_ll * 6)()
        self.lib.qxref_packed_info(handle, out)
        keys = ["rows", "columns", "row_tile", "blocks_per_row", "block_bytes", "panel_bytes"]
        return dict(zip(keys, list(out)))

    def prepacked_panel(self, handle):
        info = self.prepacked_info(handle)
        address = self.lib.qxref_packed_panel(handle)
        return np.ctypeslib.as_array(
            C.cast(address, C.POINTER(C.c_uint8)), shape=(info["panel_bytes"],)).copy()

    def qgemm_prepacked(self, handle, x, m, n):
        y = np.zeros((m, n), np.float32)
        status = self.lib.qxref_qgemm_prepacked(handle, _ptr(x), _ptr(y), m)
        return status, y

    def prepacked_destroy(self, handle):
        self.lib.qxref_packed_destroy(handle)
