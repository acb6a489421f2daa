"""Python glue over ``libqx_b200.so`` (ctypes): the host-side mirror of the reference's
public ``quixicore_cpu::`` functions for the quantized-matmul path.

The shared library is the product; this module only marshals pointers. Functions whose
reference counterpart takes host buffers accept numpy arrays and call the host-pointer
C entry points; functions ending in ``_dev`` accept torch CUDA tensors and enqueue on
torch's current stream. Importing this module without the built library raises: there is
no Python, torch or CPU fallback for any compute entry point.

The directory name contains a hyphen, so load the package through
``__graft_entry__.load_package()`` (it registers it as ``quixicore_cpu_b200``).
"""

from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libqx_b200.so")

Q8_0, Q4_0 = 0, 1
BLOCK_BYTES = {Q8_0: 34, Q4_0: 18}
OK, INVALID_SHAPE, UNSUPPORTED_FORMAT, INVALID_ARGUMENT, OUT_OF_MEMORY, DEVICE_ERROR = range(6)
STATUS_NAMES = ["kOk", "kInvalidShape", "kUnsupportedFormat", "kInvalidArgument",
                "kOutOfMemory", "kDeviceError"]

_ll, _vp, _sz = C.c_longlong, C.c_void_p, C.c_size_t


class QxError(RuntimeError):
    def __init__(self, status, where, detail=""):
        self.status = status
        super().__init__(f"{where}: {STATUS_NAMES[status]} {detail}".strip())


class WeightsInfo(C.Structure):
    _fields_ = [("format", C.c_int), ("rows", _ll), ("columns", _ll), ("block_size", _ll),
                ("blocks_per_row", _ll), ("block_bytes", _sz), ("contract_bytes", _sz),
                ("prepared_bytes", _sz), ("memory_amplification", C.c_double),
                ("preparation_ns", C.c_uint64), ("device", C.c_int), ("has_dense_bf16", C.c_int),
                ("row_tile", _ll), ("panel_bytes", _sz)]


class PushPlan(C.Structure):
    """qx_push_plan of include/qx_b200.h."""
    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("rows_per_rank", C.c_longlong),
                ("results_local", C.c_void_p), ("inbox_local", C.c_void_p),
                ("inbox_peer", C.c_void_p * 8)]


class CanonicalTensorView(C.Structure):
    """qx_canonical_tensor of include/qx_b200.h."""
    _fields_ = [("layout", C.c_int), ("scale_mode", C.c_int), ("rows", _ll), ("columns", _ll),
                ("group_size", _ll), ("data", _vp), ("data_bytes", _sz), ("scales", _vp),
                ("scale_count", _sz), ("zero_points", _vp), ("zero_point_count", _sz),
                ("group_index", _vp), ("group_index_count", _sz), ("act_order", _vp),
                ("act_order_count", _sz)]


class AwqU4Source(C.Structure):
    """qx_awq_u4_source of include/qx_b200.h."""
    _fields_ = [("qweight", _vp), ("qweight_words", _sz), ("qzeros", _vp), ("qzero_words", _sz),
                ("scales", _vp), ("scale_count", _sz), ("input_features", _ll),
                ("output_features", _ll), ("group_size", _ll)]


class GptqU4Source(C.Structure):
    """qx_gptq_u4_source of include/qx_b200.h."""
    _fields_ = [("qweight", _vp), ("qweight_words", _sz), ("qzeros", _vp), ("qzero_words", _sz),
                ("scales", _vp), ("scale_count", _sz), ("group_index", _vp),
                ("group_index_count", _sz), ("act_order", _vp), ("act_order_count", _sz),
                ("input_features", _ll), ("output_features", _ll), ("group_size", _ll),
                ("symmetric", C.c_int), ("gptq_v2", C.c_int)]


class SmoothQuantSource(C.Structure):
    """qx_smoothquant_source of include/qx_b200.h."""
    _fields_ = [("weights", _vp), ("weight_count", _sz), ("weight_scales", _vp),
                ("weight_scale_count", _sz), ("activation_scales", _vp),
                ("activation_scale_count", _sz), ("activation_zero_points", _vp),
                ("activation_zero_point_count", _sz), ("row_sums", _vp), ("row_sum_count", _sz),
                ("rows", _ll), ("columns", _ll)]


class DeviceInfo(C.Structure):
    _fields_ = [("device", C.c_int), ("sm_major", C.c_int), ("sm_minor", C.c_int),
                ("sm_count", C.c_int), ("max_smem_per_block", C.c_int), ("l2_bytes", C.c_int),
                ("hbm_bytes", _sz), ("visible_devices", C.c_int), ("peer_access_mask", C.c_int),
                ("name", C.c_char * 64), ("nvlink_peer_mask", C.c_int), ("nvlink_peers", C.c_int),
                ("nvlink_uniform", C.c_int), ("peer_performance_rank", C.c_byte * 16)]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python quixicore-cpu_b200/build.py` "
            "(nvcc, sm_100a). There is no fallback implementation.")
    lib = C.CDLL(LIB_PATH)
    sig = {
        "qx_device_query": [C.POINTER(DeviceInfo)],
        "qx_check_device_errors": [],
        "qx_qgemv_packed_size": [C.c_int, _ll, _ll, C.POINTER(_sz)],
        "qx_qgemv_pack": [C.c_int, _vp, _ll, _ll, _vp],
        "qx_qgemv_unpack": [C.c_int, _vp, _ll, _ll, _vp],
        "qx_qgemv": [C.c_int, _vp, _vp, _vp, _ll, _ll],
        "qx_qgemm": [C.c_int, _vp, _vp, _vp, _ll, _ll, _ll],
        "qx_weights_prepare": [C.c_int, _vp, _ll, _ll, _ll, _ll, C.POINTER(_vp)],
        "qx_weights_prepare_dev": [C.c_int, _vp, _ll, _ll, _ll, _ll, _vp, C.POINTER(_vp)],
        "qx_weights_get_info": [_vp, C.POINTER(WeightsInfo)],
        "qx_workspace_create": [_sz, C.POINTER(_vp)],
        "qx_qgemm_prepacked": [_vp, _vp, _vp, _ll, _vp],
        "qx_qgemm_prepacked_dev": [_vp, _vp, _vp, _ll, _ll, _vp, _vp],
        "qx_qgemm_prepacked_bf16_dev": [_vp, _vp, _vp, _ll, _ll, _vp, _vp],
        "qx_qgemv_prepacked_noalloc_dev": [_vp, _vp, _vp, _vp],
        "qx_int8_gemm": [_vp] * 7 + [_ll, _ll, _ll, C.c_int],
        "qx_qgemm_w8a8": [_vp] * 5 + [_ll, _ll, _ll],
        "qx_qgemm_w8a8_azp": [_vp] * 7 + [_ll, _ll, _ll],
        "qx_int8_gemm_dev": [_vp] * 8 + [_ll, _ll, _ll, _ll, C.c_int, C.c_int, _vp],
        "qx_qgemm_w8a32": [_vp] * 4 + [_ll, _ll, _ll],
        "qx_qgemm_w8a32_dev": [_vp] * 4 + [_ll, _ll, _ll, _ll, C.c_int, _vp, _vp],
        "qx_qgemv_w8a8": [C.c_int, _vp, _vp, _vp, _ll, _ll],
        "qx_qgemv_w8a8_packed_size": [C.c_int, _ll, _ll, C.POINTER(_ll)],
        "qx_qgemv_w8a8_pack": [C.c_int, _vp, _ll, _ll, _vp],
        "qx_qgemv_w8a8_prepacked_dev": [_vp, _vp, _vp, _vp, _vp],
        "qx_qgemv_up_gate": [C.c_int, _vp, _vp, _vp, _vp, _vp, _ll, _ll],
        "qx_qgemv_up_gate_activation": [C.c_int, _vp, _vp, _vp, _vp, _ll, _ll, C.c_int],
        "qx_qgemv_qkv": [C.c_int] + [_vp] * 7 + [_ll, _ll, _ll],
        "qx_weights_prepare_fused": [C.c_int, C.POINTER(_vp), C.POINTER(_ll), C.c_int, _ll, C.POINTER(_vp)],
        "qx_qgemm_fused_dev": [_vp, _vp, C.POINTER(_vp), _ll, _vp, _vp],
        "qx_qgemv_up_gate_activation_dev": [_vp, _vp, _vp, _vp, C.c_int, _vp, _vp],
        "qx_lowbit_packed_size": [C.c_int, _ll, _ll, _ll, C.POINTER(_sz), C.POINTER(_sz)],
        "qx_lowbit_pack": [C.c_int, _vp, _vp, _vp, _ll, _ll, _ll],
        "qx_lowbit_unpack": [C.c_int, _vp, _vp, _vp, _ll, _ll, _ll],
        "qx_lowbit_gemm": [C.c_int, _vp, _vp, _vp, _vp, _ll, _ll, _ll, _ll],
        "qx_lowbit_gemm_dev": [C.c_int, _vp, _vp, _vp, _vp, _ll, _ll, _ll, _ll, _vp],
        "qx_lowbit_gemm_w8a8": [_vp, _vp, _vp, _vp, _ll, _ll, _ll],
        "qx_lowbit_gemm_w8a8_dev": [_vp, _vp, _vp, _vp, _vp, _ll, _ll, _ll, _vp],
        "qx_quantize_int8": [_vp, _vp, _vp, _ll, _ll, _ll],
        "qx_quantize_int8_dev": [_vp, _vp, _vp, _vp, _ll, _ll, _ll, _vp],
        "qx_canonical_prepare": [C.POINTER(CanonicalTensorView), C.POINTER(_vp)],
        "qx_qgemm_prepacked_storage": [_vp, _vp, C.c_int, _ll, _vp, C.c_int, _ll, _ll],
        "qx_qgemm_prepacked_epilogue_storage": [_vp, _vp, C.c_int, _ll, _vp, _vp, C.c_int, _ll,
                                                _ll, C.c_int],
        "qx_qgemm_prepacked_epilogue_storage_dev": [_vp, _vp, C.c_int, _vp, _vp, C.c_int, _ll,
                                                    C.c_int, _vp, _vp],
        "qx_import_smoothquant_w8a8": [C.POINTER(SmoothQuantSource),
                                       C.POINTER(CanonicalTensorView), _vp],
        "qx_import_awq_u4": [C.POINTER(AwqU4Source), C.POINTER(CanonicalTensorView), _vp, _vp, _vp],
        "qx_import_gptq_u4": [C.POINTER(GptqU4Source), C.POINTER(CanonicalTensorView), _vp, _vp, _vp],
        "qx_peer_alloc": [_sz, C.POINTER(_vp), _vp],
        "qx_peer_open": [_vp, C.POINTER(_vp)],
        "qx_peer_close": [_vp],
        "qx_peer_free": [_vp],
        "qx_qgemm_prepacked_push_dev": [_vp, _vp, _ll, C.POINTER(PushPlan), _ll, _vp, _vp],
        "qx_allgather_wait_dev": [C.POINTER(PushPlan), _ll, _ll, C.POINTER(_vp), _vp],
    }
    for name, argtypes in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = C.c_int
    for name in ("qx_last_error_string", "qx_qgemv_variant", "qx_int8_gemm_variant",
                 "qx_qgemm_w8a32_variant", "qx_qgemv_w8a8_variant", "qx_lowbit_gemm_variant",
                 "qx_lowbit_gemm_w8a8_variant", "qx_canonical_gemm_variant"):
        getattr(lib, name).restype = C.c_char_p
    lib.qx_qgemv_variant.argtypes = [C.c_int]
    lib.qx_qgemv_w8a8_variant.argtypes = [C.c_int]
    lib.qx_lowbit_gemm_variant.argtypes = [C.c_int]
    lib.qx_lowbit_w8a8_scratch_bytes.argtypes = [_ll, _ll]
    lib.qx_lowbit_w8a8_scratch_bytes.restype = _sz
    lib.qx_weights_destroy.argtypes = [_vp]
    lib.qx_weights_destroy.restype = None
    lib.qx_canonical_destroy.argtypes = [_vp]
    lib.qx_canonical_destroy.restype = None
    lib.qx_workspace_destroy.argtypes = [_vp]
    lib.qx_workspace_destroy.restype = None
    lib.qx_workspace_capacity.argtypes = [_vp]
    lib.qx_workspace_capacity.restype = _sz
    lib.qx_set_num_threads.argtypes = [C.c_int]
    lib.qx_set_num_threads.restype = None
    lib.qx_num_threads.restype = C.c_int
    lib.qx_kernel_launch_count.restype = C.c_ulonglong
    lib.qx_push_inbox_bytes.argtypes = [C.c_int, _ll, _ll]
    lib.qx_push_inbox_bytes.restype = _sz
    return lib


lib = _load()


def _np(a):
    if a is None:
        return None
    assert isinstance(a, np.ndarray) and a.flags["C_CONTIGUOUS"], "need a contiguous numpy array"
    return a.ctypes.data_as(_vp)


def _dev(t):
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous(), "need a contiguous CUDA tensor"
    return _vp(t.data_ptr())


def _stream():
    import torch
    return _vp(torch.cuda.current_stream().cuda_stream)


def last_error() -> str:
    return (lib.qx_last_error_string() or b"").decode()


def check(status: int, where: str) -> None:
    if status != OK:
        raise QxError(status, where, last_error())


def launch_count() -> int:
    return int(lib.qx_kernel_launch_count())


def device_info() -> dict:
    info = DeviceInfo()
    check(lib.qx_device_query(C.byref(info)), "qx_device_query")
    out = {name: getattr(info, name) for name, _ in DeviceInfo._fields_}
    out["name"] = info.name.decode()
    out["peer_performance_rank"] = list(info.peer_performance_rank)
    return out


# ---- reference-shaped host-pointer calls: return (status, result) like the C functions ----

def qgemv_packed_size(fmt, n, k, want_size=True):
    size = _sz(0)
    status = lib.qx_qgemv_packed_size(fmt, n, k, C.byref(size) if want_size else None)
    return status, size.value


def qgemv_pack(fmt, weights, n, k):
    packed = np.zeros(n * (k // 32) * BLOCK_BYTES[fmt], np.uint8)
    return lib.qx_qgemv_pack(fmt, _np(weights), n, k, _np(packed)), packed


def qgemv_unpack(fmt, packed, n, k):
    out = np.zeros((n, k), np.float32)
    return lib.qx_qgemv_unpack(fmt, _np(packed), n, k, _np(out)), out


def qgemv(fmt, packed, x, n, k):
    y = np.zeros(n, np.float32)
    return lib.qx_qgemv(fmt, _np(packed), _np(x), _np(y), n, k), y


def qgemm(fmt, packed, x, m, n, k):
    y = np.zeros((m, n), np.float32)
    return lib.qx_qgemm(fmt, _np(packed), _np(x), _np(y), m, n, k), y


def int8_gemm(w, x, ws, xs, m, n, k, row_sum=None, zp=None, asymmetric=False):
    y = np.zeros((m, n), np.float32)
    status = lib.qx_int8_gemm(_np(w), _np(x), _np(ws), _np(xs), _np(row_sum), _np(zp), _np(y),
                              m, n, k, 1 if asymmetric else 0)
    return status, y


def qgemm_w8a8(w, x, ws, xs, m, n, k):
    y = np.zeros((m, n), np.float32)
    return lib.qx_qgemm_w8a8(_np(w), _np(x), _np(ws), _np(xs), _np(y), m, n, k), y


def qgemm_w8a32(w, ws, x, m, n, k):
    y = np.zeros((m, n), np.float32)
    return lib.qx_qgemm_w8a32(_np(w), _np(ws), _np(x), _np(y), m, n, k), y


# ---- callers either side of the GEMV (host buffers) ----

def qgemv_w8a8(fmt, packed, x, n, k):
    y = np.zeros(n, np.float32)
    return lib.qx_qgemv_w8a8(fmt, _np(packed), _np(x), _np(y), n, k), y


def qgemv_up_gate(fmt, packed_up, packed_gate, x, n, k):
    up, gate = np.zeros(n, np.float32), np.zeros(n, np.float32)
    status = lib.qx_qgemv_up_gate(fmt, _np(packed_up), _np(packed_gate), _np(x), _np(up), _np(gate), n, k)
    return status, up, gate


def qgemv_up_gate_activation(fmt, packed_up, packed_gate, x, n, k, gelu_tanh=True):
    out = np.zeros(n, np.float32)
    status = lib.qx_qgemv_up_gate_activation(fmt, _np(packed_up), _np(packed_gate), _np(x), _np(out),
                                             n, k, 1 if gelu_tanh else 0)
    return status, out


def qgemv_qkv(fmt, wq, wk, wv, x, query_dim, kv_dim, input_dim):
    q, k_out, v_out = (np.zeros(query_dim, np.float32), np.zeros(kv_dim, np.float32),
                       np.zeros(kv_dim, np.float32))
    status = lib.qx_qgemv_qkv(fmt, _np(wq), _np(wk), _np(wv), _np(x), _np(q), _np(k_out), _np(v_out),
                              query_dim, kv_dim, input_dim)
    return status, q, k_out, v_out


LOWBIT_INT2_ROW, LOWBIT_INT3_GROUP64, LOWBIT_INT4_ROW, LOWBIT_INT4_GROUP = range(4)


def lowbit_packed_size(fmt, rows, dim, group_size=0):
    wb, sc = _sz(0), _sz(0)
    status = lib.qx_lowbit_packed_size(fmt, rows, dim, group_size, C.byref(wb), C.byref(sc))
    return status, wb.value, sc.value


def lowbit_pack(fmt, weights, rows, dim, group_size=0):
    status, wb, sc = lowbit_packed_size(fmt, rows, dim, group_size)
    packed, scales = np.zeros(max(wb, 1), np.uint8), np.zeros(max(sc, 1), np.float32)
    return lib.qx_lowbit_pack(fmt, _np(weights), _np(packed), _np(scales), rows, dim, group_size), \
        packed[:wb], scales[:sc].reshape(rows, -1) if status == OK else scales


def lowbit_unpack(fmt, packed, scales, rows, dim, group_size=0):
    out = np.zeros((rows, dim), np.float32)
    return lib.qx_lowbit_unpack(fmt, _np(packed), _np(scales), _np(out), rows, dim, group_size), out


def lowbit_gemm(fmt, packed, scales, x, m, n, k, group_size=0):
    y = np.zeros((m, n), np.float32)
    return lib.qx_lowbit_gemm(fmt, _np(packed), _np(scales), _np(x), _np(y), m, n, k, group_size), y


def lowbit_gemm_w8a8(packed, scales, x, m, n, k):
    y = np.zeros((m, n), np.float32)
    return lib.qx_lowbit_gemm_w8a8(_np(packed), _np(scales), _np(x), _np(y), m, n, k), y


def quantize_int8(x, rows, dim, group_size=0):
    groups = dim // (group_size or dim) if dim > 0 and (group_size or dim) > 0 else 1
    codes, scales = np.zeros((rows, dim), np.int8), np.zeros((rows, max(groups, 1)), np.float32)
    return lib.qx_quantize_int8(_np(x), _np(codes), _np(scales), rows, dim, group_size), codes, scales


def variants() -> dict:
    return {
        "qgemv_q8_0": lib.qx_qgemv_variant(Q8_0).decode(),
        "qgemv_q4_0": lib.qx_qgemv_variant(Q4_0).decode(),
        "int8_gemm": lib.qx_int8_gemm_variant().decode(),
        "qgemm_w8a32": lib.qx_qgemm_w8a32_variant().decode(),
    }


class PackedWeights:
    """Device-resident prepared weights (mirror of quixicore_cpu::CpuPackedWeights)."""

    def __init__(self):
        self.handle = _vp()

    def prepare(self, fmt, packed, rows, columns, row_begin=0, row_count=None) -> int:
        self.reset()
        row_count = rows if row_count is None else row_count
        if packed is not None and not isinstance(packed, np.ndarray):
            ptr = _dev(packed)
            return lib.qx_weights_prepare_dev(fmt, ptr, rows, columns, row_begin, row_count,
                                              _stream(), C.byref(self.handle))
        return lib.qx_weights_prepare(fmt, _np(packed), rows, columns, row_begin, row_count,
                                      C.byref(self.handle))

    def ready(self) -> bool:
        return bool(self.handle)

    def info(self) -> dict:
        info = WeightsInfo()
        check(lib.qx_weights_get_info(self.handle, C.byref(info)), "qx_weights_get_info")
        return {name: getattr(info, name) for name, _ in WeightsInfo._fields_}

    def reset(self) -> None:
        if self.handle:
            lib.qx_weights_destroy(self.handle)
            self.handle = _vp()

    def __del__(self):
        try:
            self.reset()
        except Exception:
            pass

    # host buffers (numpy): the reference-facing call
    def qgemm_prepacked(self, x, m, y=None):
        rows = self.info()["rows"] if self.handle else 0
        if y is None:
            y = np.zeros((m, max(rows, 1)), np.float32)
        return lib.qx_qgemm_prepacked(self.handle, _np(x), _np(y), m, None), y

    # raw host pointers (e.g. pinned torch tensors): the end-to-end timed call
    def qgemm_prepacked_ptr(self, x_ptr, y_ptr, m) -> int:
        return lib.qx_qgemm_prepacked(self.handle, _vp(x_ptr), _vp(y_ptr), m, None)

    # device tensors, torch's current stream
    def qgemm_dev(self, x, y, m, ldy=None) -> int:
        ldy = y.shape[-1] if ldy is None else ldy
        return lib.qx_qgemm_prepacked_dev(self.handle, _dev(x), _vp(y.data_ptr()), m, ldy, None,
                                          _stream())

    def prepare_fused(self, fmt, parts, rows, columns) -> int:
        """Several matrices with the same column count in one handle (numpy host bytes)."""
        self.reset()
        pointers = (_vp * len(parts))(*[p.ctypes.data for p in parts])
        counts = (_ll * len(parts))(*rows)
        self._fused_keepalive = parts
        return lib.qx_weights_prepare_fused(fmt, pointers, counts, len(parts), columns,
                                            C.byref(self.handle))

    def qgemm_fused_dev(self, x, outputs, m) -> int:
        pointers = (_vp * len(outputs))(*[o.data_ptr() for o in outputs])
        return lib.qx_qgemm_fused_dev(self.handle, _dev(x), pointers, m, None, _stream())

    def up_gate_activation_dev(self, x, out, scratch, gelu_tanh=True) -> int:
        return lib.qx_qgemv_up_gate_activation_dev(self.handle, _dev(x), _vp(out.data_ptr()),
                                                   _vp(scratch.data_ptr()), 1 if gelu_tanh else 0,
                                                   None, _stream())

    def qgemv_w8a8_dev(self, x, y) -> int:
        return lib.qx_qgemv_w8a8_prepacked_dev(self.handle, _dev(x), _vp(y.data_ptr()), None, _stream())

    def qgemv_noalloc_dev(self, x, y) -> int:
        """Decode GEMV through the entry point that never allocates device memory."""
        return lib.qx_qgemv_prepacked_noalloc_dev(self.handle, _dev(x), _vp(y.data_ptr()),
                                                  _stream())

    def qgemm_bf16_dev(self, x_bf16, y, m, ldy=None) -> int:
        ldy = y.shape[-1] if ldy is None else ldy
        return lib.qx_qgemm_prepacked_bf16_dev(self.handle, _dev(x_bf16), _vp(y.data_ptr()), m,
                                               ldy, None, _stream())


# ---- canonical prepared projections (CanonicalQuantTensor -> prepare -> typed projection) ----
INT4_SYMMETRIC, UINT4_AFFINE, INT8_SYMMETRIC = 0, 1, 2
SCALE_ROW, SCALE_CHANNEL, SCALE_GROUP = 2, 3, 4
F32, F16, BF16 = 0, 1, 2
STORAGE_DTYPES = {F32: np.float32, F16: np.uint16, BF16: np.uint16}
ACT_NONE, ACT_GELU_ERF, ACT_GELU_TANH, ACT_SILU, ACT_RELU2 = range(5)


def canonical_view(layout, scale_mode, rows, columns, group_size, data, scales,
                   data_bytes=None, scale_count=None, zeros=None, group_index=None,
                   act_order=None) -> CanonicalTensorView:
    """A qx_canonical_tensor over numpy arrays (the arrays must outlive the view)."""
    def count(a):
        return 0 if a is None else a.size
    return CanonicalTensorView(layout, scale_mode, rows, columns, group_size, _np(data),
                               count(data) if data_bytes is None else data_bytes, _np(scales),
                               count(scales) if scale_count is None else scale_count, _np(zeros),
                               count(zeros), _np(group_index), count(group_index), _np(act_order),
                               count(act_order))


class CanonicalWeights:
    """Device-resident prepared canonical tensor (CpuPackedWeights::prepare(tensor))."""

    def __init__(self):
        self.handle = _vp()
        self.rows = self.columns = 0

    def prepare(self, view: CanonicalTensorView) -> int:
        self.reset()
        status = lib.qx_canonical_prepare(C.byref(view), C.byref(self.handle))
        if status == OK:
            self.rows, self.columns = view.rows, view.columns
        return status

    def ready(self) -> bool:
        return bool(self.handle)

    def reset(self) -> None:
        if self.handle:
            lib.qx_canonical_destroy(self.handle)
        self.handle = _vp()

    def __del__(self):
        try:
            self.reset()
        except Exception:
            pass

    def qgemm_storage(self, x, x_type, m, y_type=F32, bias=None, activation=None,
                      x_count=None, y_count=None):
        """qgemm_prepacked_storage (activation None) / qgemm_prepacked_epilogue_storage."""
        y = np.zeros(max(m, 1) * max(self.rows, 1), STORAGE_DTYPES.get(y_type, np.float32))
        x_count = m * self.columns if x_count is None else x_count
        y_count = m * self.rows if y_count is None else y_count
        if activation is None and bias is None:
            status = lib.qx_qgemm_prepacked_storage(self.handle, _np(x), x_type, x_count, _np(y),
                                                    y_type, y_count, m)
        else:
            status = lib.qx_qgemm_prepacked_epilogue_storage(
                self.handle, _np(x), x_type, x_count, _np(bias), _np(y), y_type, y_count, m,
                ACT_NONE if activation is None else activation)
        return status, y.reshape(max(m, 1), max(self.rows, 1))

    def qgemm_storage_dev(self, x, x_type, y, y_type, m, bias=None, activation=ACT_NONE) -> int:
        return lib.qx_qgemm_prepacked_epilogue_storage_dev(
            self.handle, _vp(x.data_ptr()), x_type, _dev(bias), _vp(y.data_ptr()), y_type, m,
            activation, None, _stream())


def import_smoothquant_w8a8(weights, weight_scales, activation_scales, rows, columns,
                            zero_points=None, row_sums=None):
    """-> (status, qx_canonical_tensor view of the source arrays, row sums)."""
    source = SmoothQuantSource(
        _np(weights), 0 if weights is None else weights.size, _np(weight_scales),
        0 if weight_scales is None else weight_scales.size, _np(activation_scales),
        0 if activation_scales is None else activation_scales.size, _np(zero_points),
        0 if zero_points is None else zero_points.size, _np(row_sums),
        0 if row_sums is None else row_sums.size, rows, columns)
    view = CanonicalTensorView()
    sums = np.zeros(max(rows, 1), np.int32)
    status = lib.qx_import_smoothquant_w8a8(C.byref(source), C.byref(view), _np(sums))
    return status, view, sums[:max(rows, 0)]


def import_awq_u4(qweight, qzeros, scales, k, n, group):
    """-> (status, view, (data, scales, zero points) arrays the view points at)."""
    groups = max(k // group, 1) if group > 0 else 1
    data = np.zeros(max(n * k // 2, 1), np.uint8)
    out_scales = np.zeros(max(n * groups, 1), np.float32)
    zeros = np.zeros(max(n * groups, 1), np.float32)
    source = AwqU4Source(_np(qweight), 0 if qweight is None else qweight.size, _np(qzeros),
                         0 if qzeros is None else qzeros.size, _np(scales),
                         0 if scales is None else scales.size, k, n, group)
    view = CanonicalTensorView()
    status = lib.qx_import_awq_u4(C.byref(source), C.byref(view), _np(data), _np(out_scales), _np(zeros))
    return status, view, (data, out_scales, zeros)


def import_gptq_u4(qweight, qzeros, scales, k, n, group, symmetric=False, v2=False,
                   group_index=None, act_order=None):
    groups = max(k // group, 1) if group > 0 else 1
    data = np.zeros(max(n * k // 2, 1), np.uint8)
    out_scales = np.zeros(max(n * groups, 1), np.float32)
    zeros = np.zeros(max(n * groups, 1), np.float32)
    source = GptqU4Source(_np(qweight), 0 if qweight is None else qweight.size, _np(qzeros),
                          0 if qzeros is None else qzeros.size, _np(scales),
                          0 if scales is None else scales.size, _np(group_index),
                          0 if group_index is None else group_index.size, _np(act_order),
                          0 if act_order is None else act_order.size, k, n, group, int(symmetric),
                          int(v2))
    view = CanonicalTensorView()
    status = lib.qx_import_gptq_u4(C.byref(source), C.byref(view), _np(data), _np(out_scales), _np(zeros))
    return status, view, (data, out_scales, zeros)


def peer_alloc(nbytes: int):
    """(device pointer, 64-byte handle) of a zeroed buffer other processes can map."""
    ptr, handle = _vp(), C.create_string_buffer(64)
    check(lib.qx_peer_alloc(nbytes, C.byref(ptr), handle), "qx_peer_alloc")
    return ptr.value, handle.raw


def peer_open(handle: bytes) -> int:
    ptr = _vp()
    check(lib.qx_peer_open(C.create_string_buffer(handle, 64), C.byref(ptr)), "qx_peer_open")
    return ptr.value


def push_inbox_bytes(world: int, m: int, rows_per_rank: int) -> int:
    return lib.qx_push_inbox_bytes(world, m, rows_per_rank)


def qgemm_push_dev(weights: "PackedWeights", x, m: int, plan: PushPlan, step: int) -> int:
    """Sharded GEMV whose results land in every rank's buffer (fused all-gather)."""
    return lib.qx_qgemm_prepacked_push_dev(weights.handle, _dev(x), m, C.byref(plan), step, None,
                                           _stream())


def allgather_wait_dev(plan: PushPlan, m: int, step: int) -> int:
    """Enqueues the wait for step `step`; returns the device address of its results."""
    out = _vp()
    check(lib.qx_allgather_wait_dev(C.byref(plan), m, step, C.byref(out), _stream()),
          "qx_allgather_wait_dev")
    return out.value


def int8_gemm_dev(w, x, ws, xs, y, m, n, k, row_sum=None, zp=None, acc=None, ldy=None,
                  check_scales=False) -> int:
    ldy = n if ldy is None else ldy
    return lib.qx_int8_gemm_dev(_dev(w), _dev(x), _dev(ws), _dev(xs), _dev(row_sum), _dev(zp),
                                _vp(y.data_ptr()), _dev(acc), m, n, k, ldy,
                                1 if row_sum is not None else 0, 1 if check_scales else 0,
                                _stream())


def qgemm_w8a32_dev(w, ws, x, y, m, n, k, ldy=None, check_scales=False) -> int:
    ldy = n if ldy is None else ldy
    return lib.qx_qgemm_w8a32_dev(_dev(w), _dev(ws), _dev(x), _vp(y.data_ptr()), m, n, k, ldy,
                                  1 if check_scales else 0, None, _stream())
