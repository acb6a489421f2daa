// Adapter from the umbrella `quixicore::contract` KernelCall ABI to the qx_b200 entry points
// for the quantized-matmul path. The reference declares this ABI for every backend
// (include/quixicore/contract/kernel_abi.hpp:53-107: TensorView with a MemorySpace, a
// stream and a workspace) but leaves these operations unwired on the CPU backend
// (include/quixicore/cpu/contract.hpp:164-169 returns adapter_not_wired). Here they are
// wired: host tensors go to the host-pointer C entry points, device tensors to the `_dev`
// ones on `call.stream`.
//
// When the reference's own kernel_abi.hpp is on the include path it is used as is (same
// types, so a KernelCall built by a host of the reference is passed straight through);
// otherwise the declarations below restate that ABI (same namespace, names, enumerator
// order and field order).
//
// Operations and their operands (inputs / outputs in this order; shapes as in the
// reference's typed functions):
//   "qgemv"      in  W packed [n,k] bytes, x f32 [k]                     out y f32 [n]
//   "qgemm"      in  W packed [n,k] bytes, x f32 [m,k]                   out y f32 [m,n]
//   "int8_gemm"  in  W i8 [n,k], X i8 [m,k], weight_scale f32 [n], activation_scale f32 [m],
//                    (optional) weight_row_sum i32 [n], activation_zero_point i32 [m]
//                                                                         out Y f32 [m,n]
//   "qgemv_up_gate"            in up W, gate W [n,k], x f32 [k]           out up f32 [n], gate f32 [n]
//   "qgemv_up_gate_activation" in up W, gate W [n,k], x f32 [k]           out y f32 [n]
//   "qgemv_qkv"  in  Wq [q,k], Wk [kv,k], Wv [kv,k], x f32 [k]            out q [q], k [kv], v [kv]
// Attributes: "format" (i64, quixicore_cpu::QuantFormat value: 0 = q8_0, 1 = q4_0) for the
// packed operations; "gelu_tanh" (boolean, default true) for the activation; "asymmetric"
// (boolean, default: true when the two optional int8_gemm inputs are present);
// "prepared" (bytes: a qx_weights* prepared earlier) REQUIRED for packed weights in device
// memory -- the canonical bytes of such a tensor are then not read at all.
// A packed weight tensor carries its logical shape [rows, columns]; dtype `packed` or `u8`.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cstring>

#include "qx_b200.h"

#if defined(__has_include)
#if __has_include("quixicore/contract/kernel_abi.hpp")
#include "quixicore/contract/kernel_abi.hpp"
#define QX_B200_HAVE_REFERENCE_KERNEL_ABI 1
#endif
#endif

#ifndef QX_B200_HAVE_REFERENCE_KERNEL_ABI
namespace quixicore::contract {

// include/quixicore/contract/kernel_abi.hpp:10-21
enum class StatusCode : std::uint8_t {
  ok,
  invalid_argument,
  invalid_shape,
  unsupported_dtype,
  unsupported_format,
  unsupported_layout,
  insufficient_workspace,
  adapter_not_wired,
  not_implemented,
  runtime_error,
};

// :23-31
struct Status {
  StatusCode code;
  const char* operation;
  const char* detail;
  [[nodiscard]] constexpr bool is_ok() const noexcept { return code == StatusCode::ok; }
};

// :33-51
enum class DType : std::uint8_t {
  unknown, boolean, i8, u8, i16, u16, i32, u32, i64, u64, f16, bf16, f32, f64, e4m3, e5m2, packed,
};

// :53-58
enum class MemorySpace : std::uint8_t { unknown, host, device, shared };

// :60-65
enum TensorFlags : std::uint32_t {
  tensor_none = 0,
  tensor_read_only = 1U << 0,
  tensor_contiguous = 1U << 1,
  tensor_optional = 1U << 2,
};

// :67-75
struct TensorView {
  void* data;
  const std::int64_t* shape;
  const std::int64_t* strides;
  std::size_t rank;
  DType dtype;
  MemorySpace memory_space;
  std::uint32_t flags;
};

// :77-92
enum class AttributeKind : std::uint8_t { boolean, i64, f64, string, bytes };
struct Attribute {
  const char* name;
  AttributeKind kind;
  const void* data;
  std::size_t size;
  std::int64_t i64;
  double f64;
};

// :94-105
struct KernelCall {
  const TensorView* inputs;
  std::size_t input_count;
  TensorView* outputs;
  std::size_t output_count;
  const Attribute* attributes;
  std::size_t attribute_count;
  void* backend_context;
  void* stream;
  void* workspace;
  std::size_t workspace_size;
};

}  // namespace quixicore::contract
#endif  // QX_B200_HAVE_REFERENCE_KERNEL_ABI

namespace quixicore::b200::contract_api {

namespace detail {
using quixicore::contract::Attribute;
using quixicore::contract::AttributeKind;
using quixicore::contract::DType;
using quixicore::contract::KernelCall;
using quixicore::contract::MemorySpace;
using quixicore::contract::Status;
using quixicore::contract::StatusCode;
using quixicore::contract::TensorView;

inline Status make(StatusCode code, const char* operation, const char* detail) noexcept {
  return Status{code, operation, detail};
}

// quixicore_cpu::Status (qx_status) -> contract status
inline Status from_qx(qx_status status, const char* operation) noexcept {
  switch (status) {
    case QX_STATUS_OK: return make(StatusCode::ok, operation, "");
    case QX_STATUS_INVALID_SHAPE: return make(StatusCode::invalid_shape, operation, "shape rejected by the kernel entry point");
    case QX_STATUS_UNSUPPORTED_FORMAT: return make(StatusCode::unsupported_format, operation, "quantization format not served on this path");
    case QX_STATUS_INVALID_ARGUMENT: return make(StatusCode::invalid_argument, operation, "argument rejected by the kernel entry point");
    case QX_STATUS_OUT_OF_MEMORY: return make(StatusCode::insufficient_workspace, operation, "device memory exhausted");
    default: return make(StatusCode::runtime_error, operation, qx_last_error_string());
  }
}

inline const Attribute* find(const KernelCall& call, const char* name) noexcept {
  for (std::size_t i = 0; i < call.attribute_count; ++i) {
    if (call.attributes[i].name != nullptr && std::strcmp(call.attributes[i].name, name) == 0) {
      return &call.attributes[i];
    }
  }
  return nullptr;
}
inline bool boolean_attribute(const KernelCall& call, const char* name, bool fallback) noexcept {
  const Attribute* a = find(call, name);
  if (a == nullptr) return fallback;
  return a->kind == AttributeKind::boolean || a->kind == AttributeKind::i64 ? a->i64 != 0 : fallback;
}

// every tensor of the call lives in one memory space: host or device
inline bool memory_space(const KernelCall& call, MemorySpace* space) noexcept {
  MemorySpace seen = MemorySpace::unknown;
  auto merge = [&](const TensorView& t) {
    if (t.data == nullptr && (t.flags & quixicore::contract::tensor_optional) != 0) return true;
    if (t.memory_space != MemorySpace::host && t.memory_space != MemorySpace::device) return false;
    if (seen == MemorySpace::unknown) seen = t.memory_space;
    return seen == t.memory_space;
  };
  for (std::size_t i = 0; i < call.input_count; ++i) {
    if (!merge(call.inputs[i])) return false;
  }
  for (std::size_t i = 0; i < call.output_count; ++i) {
    if (!merge(call.outputs[i])) return false;
  }
  *space = seen;
  return seen != MemorySpace::unknown;
}

inline bool dense(const TensorView& t, DType dtype, std::size_t rank) noexcept {
  if (t.data == nullptr || t.shape == nullptr || t.rank != rank || t.dtype != dtype) return false;
  if (t.strides != nullptr) {  // row-major contiguous only
    std::int64_t expect = 1;
    for (std::size_t d = rank; d-- > 0;) {
      if (t.strides[d] != expect) return false;
      expect *= t.shape[d];
    }
  }
  return true;
}
inline bool packed_weights(const TensorView& t) noexcept {
  return t.shape != nullptr && t.rank == 2 && (t.dtype == DType::packed || t.dtype == DType::u8);
}
// x as a vector [k] (or [1,k]); *k receives its length
inline bool f32_vector(const TensorView& t, long long* k) noexcept {
  if (dense(t, DType::f32, 1)) { *k = t.shape[0]; return true; }
  if (dense(t, DType::f32, 2) && t.shape[0] == 1) { *k = t.shape[1]; return true; }
  return false;
}

struct Common {
  const char* op;
  MemorySpace space;
  int format;
};

inline Status common_checks(const KernelCall& call, const char* op, std::size_t inputs_min,
                            std::size_t outputs, bool needs_format, Common* out) noexcept {
  if (call.inputs == nullptr || call.outputs == nullptr || call.input_count < inputs_min ||
      call.output_count != outputs) {
    return make(StatusCode::invalid_argument, op, "wrong number of input / output tensors");
  }
  out->op = op;
  if (!memory_space(call, &out->space)) {
    return make(StatusCode::invalid_argument, op, "tensors must all be host or all be device memory");
  }
  out->format = -1;
  if (needs_format) {
    const Attribute* f = find(call, "format");
    if (f == nullptr || f->kind != AttributeKind::i64) {
      return make(StatusCode::invalid_argument, op, "attribute `format` (i64 QuantFormat value) is required");
    }
    out->format = static_cast<int>(f->i64);
  }
  return make(StatusCode::ok, op, "");
}

inline const qx_weights* prepared_handle(const KernelCall& call) noexcept {
  const Attribute* a = find(call, "prepared");
  return (a != nullptr && a->kind == AttributeKind::bytes) ? static_cast<const qx_weights*>(a->data) : nullptr;
}

// ---- qgemv / qgemm ----------------------------------------------------------------------
inline Status qgemm_like(const KernelCall& call, const char* op, bool vector) noexcept {
  Common c{};
  const Status pre = common_checks(call, op, 2, 1, true, &c);
  if (!pre.is_ok()) return pre;
  const TensorView& w = call.inputs[0];
  const TensorView& x = call.inputs[1];
  const TensorView& y = call.outputs[0];
  if (!packed_weights(w)) return make(StatusCode::unsupported_dtype, op, "weights: rank-2 packed bytes expected");
  const long long n = w.shape[0], k = w.shape[1];
  long long m = 1, xk = 0;
  if (vector) {
    if (!f32_vector(x, &xk)) return make(StatusCode::unsupported_dtype, op, "x: f32 [k] expected");
    long long yn = 0;
    if (!f32_vector(y, &yn) || yn != n) return make(StatusCode::invalid_shape, op, "y: f32 [n] expected");
  } else {
    if (!dense(x, DType::f32, 2)) return make(StatusCode::unsupported_dtype, op, "x: f32 [m,k] expected");
    m = x.shape[0];
    xk = x.shape[1];
    if (!dense(y, DType::f32, 2) || y.shape[0] != m || y.shape[1] != n) {
      return make(StatusCode::invalid_shape, op, "y: f32 [m,n] expected");
    }
  }
  if (xk != k) return make(StatusCode::invalid_shape, op, "x and the weights disagree on k");
  if (c.space == MemorySpace::host) {
    return from_qx(qx_qgemm(c.format, w.data, static_cast<const float*>(x.data), static_cast<float*>(y.data),
                            m, n, k), op);
  }
  const qx_weights* handle = prepared_handle(call);
  if (handle == nullptr) {
    return make(StatusCode::invalid_argument, op,
                "device tensors need the attribute `prepared` (a qx_weights handle)");
  }
  qx_weights_info info{};
  if (qx_weights_get_info(handle, &info) != QX_STATUS_OK || info.rows != n || info.columns != k ||
      info.format != c.format) {
    return make(StatusCode::invalid_shape, op, "prepared handle does not match the weight tensor");
  }
  return from_qx(qx_qgemm_prepacked_dev(handle, static_cast<const float*>(x.data), static_cast<float*>(y.data),
                                        m, n, nullptr, call.stream), op);
}

// ---- int8_gemm --------------------------------------------------------------------------
inline Status int8_gemm(const KernelCall& call) noexcept {
  const char* op = "int8_gemm";
  Common c{};
  const Status pre = common_checks(call, op, 4, 1, false, &c);
  if (!pre.is_ok()) return pre;
  const TensorView& w = call.inputs[0];
  const TensorView& x = call.inputs[1];
  if (!dense(w, DType::i8, 2) || !dense(x, DType::i8, 2)) {
    return make(StatusCode::unsupported_dtype, op, "W [n,k] and X [m,k] must be i8");
  }
  const long long n = w.shape[0], k = w.shape[1], m = x.shape[0];
  if (x.shape[1] != k) return make(StatusCode::invalid_shape, op, "W and X disagree on k");
  const TensorView& ws = call.inputs[2];
  const TensorView& as = call.inputs[3];
  if (!dense(ws, DType::f32, 1) || ws.shape[0] != n || !dense(as, DType::f32, 1) || as.shape[0] != m) {
    return make(StatusCode::invalid_shape, op, "scales: f32 [n] and f32 [m] expected");
  }
  const void* row_sum = nullptr;
  const void* zero_point = nullptr;
  if (call.input_count >= 6 && call.inputs[4].data != nullptr && call.inputs[5].data != nullptr) {
    if (!dense(call.inputs[4], DType::i32, 1) || call.inputs[4].shape[0] != n ||
        !dense(call.inputs[5], DType::i32, 1) || call.inputs[5].shape[0] != m) {
      return make(StatusCode::invalid_shape, op, "row sums i32 [n] and zero points i32 [m] expected");
    }
    row_sum = call.inputs[4].data;
    zero_point = call.inputs[5].data;
  }
  const bool asymmetric = boolean_attribute(call, "asymmetric", row_sum != nullptr);
  if (asymmetric && row_sum == nullptr) {
    return make(StatusCode::invalid_argument, op, "asymmetric needs the row sums and zero points");
  }
  const TensorView& y = call.outputs[0];
  if (!dense(y, DType::f32, 2) || y.shape[0] != m || y.shape[1] != n) {
    return make(StatusCode::invalid_shape, op, "Y: f32 [m,n] expected");
  }
  if (c.space == MemorySpace::host) {
    return from_qx(qx_int8_gemm(static_cast<const int8_t*>(w.data), static_cast<const int8_t*>(x.data),
                                static_cast<const float*>(ws.data), static_cast<const float*>(as.data),
                                static_cast<const int32_t*>(row_sum), static_cast<const int*>(zero_point),
                                static_cast<float*>(y.data), m, n, k, asymmetric ? 1 : 0), op);
  }
  return from_qx(qx_int8_gemm_dev(static_cast<const int8_t*>(w.data), static_cast<const int8_t*>(x.data),
                                  static_cast<const float*>(ws.data), static_cast<const float*>(as.data),
                                  static_cast<const int32_t*>(row_sum), static_cast<const int*>(zero_point),
                                  static_cast<float*>(y.data), nullptr, m, n, k, n, asymmetric ? 1 : 0, 0,
                                  call.stream), op);
}

// ---- fused decode projections (host tensors) ---------------------------------------------
inline Status fused(const KernelCall& call, const char* op, int matrices, int outputs) noexcept {
  Common c{};
  const Status pre = common_checks(call, op, static_cast<std::size_t>(matrices) + 1,
                                   static_cast<std::size_t>(outputs), true, &c);
  if (!pre.is_ok()) return pre;
  if (c.space != MemorySpace::host) {
    return make(StatusCode::unsupported_layout, op,
                "device tensors: prepare a fused handle (qx_weights_prepare_fused) and call qx_qgemm_fused_dev");
  }
  for (int i = 0; i < matrices; ++i) {
    if (!packed_weights(call.inputs[i])) return make(StatusCode::unsupported_dtype, op, "weights: rank-2 packed bytes expected");
  }
  long long k = 0;
  if (!f32_vector(call.inputs[matrices], &k)) return make(StatusCode::unsupported_dtype, op, "x: f32 [k] expected");
  for (int i = 0; i < matrices; ++i) {
    if (call.inputs[i].shape[1] != k) return make(StatusCode::invalid_shape, op, "x and the weights disagree on k");
  }
  const float* x = static_cast<const float*>(call.inputs[matrices].data);
  auto out_vector = [&](std::size_t index, long long rows, float** ptr) {
    long long len = 0;
    if (!f32_vector(call.outputs[index], &len) || len != rows) return false;
    *ptr = static_cast<float*>(call.outputs[index].data);
    return true;
  };
  const long long n = call.inputs[0].shape[0];
  if (matrices == 2) {
    if (call.inputs[1].shape[0] != n) return make(StatusCode::invalid_shape, op, "up and gate disagree on n");
    float* a = nullptr;
    float* b = nullptr;
    if (!out_vector(0, n, &a) || (outputs == 2 && !out_vector(1, n, &b))) {
      return make(StatusCode::invalid_shape, op, "outputs: f32 [n] expected");
    }
    if (outputs == 2) {
      return from_qx(qx_qgemv_up_gate(c.format, call.inputs[0].data, call.inputs[1].data, x, a, b, n, k), op);
    }
    return from_qx(qx_qgemv_up_gate_activation(c.format, call.inputs[0].data, call.inputs[1].data, x, a, n, k,
                                               boolean_attribute(call, "gelu_tanh", true) ? 1 : 0), op);
  }
  const long long kv = call.inputs[1].shape[0];
  if (call.inputs[2].shape[0] != kv) return make(StatusCode::invalid_shape, op, "k and v projections disagree on rows");
  float* q = nullptr;
  float* ko = nullptr;
  float* vo = nullptr;
  if (!out_vector(0, n, &q) || !out_vector(1, kv, &ko) || !out_vector(2, kv, &vo)) {
    return make(StatusCode::invalid_shape, op, "outputs: f32 [q], [kv], [kv] expected");
  }
  return from_qx(qx_qgemv_qkv(c.format, call.inputs[0].data, call.inputs[1].data, call.inputs[2].data, x, q, ko,
                              vo, n, kv, k), op);
}

}  // namespace detail

// The operations of the quantized-matmul path by their contract names
// (include/quixicore/contract/operations.hpp:132, 215-222); anything else is reported as
// adapter_not_wired, like the reference's own dispatch.
[[nodiscard]] inline quixicore::contract::Status dispatch(
    const char* operation, const quixicore::contract::KernelCall& call) noexcept {
  using namespace detail;
  if (operation == nullptr) return make(StatusCode::invalid_argument, "unknown_operation", "null operation name");
  if (std::strcmp(operation, "qgemv") == 0) return qgemm_like(call, "qgemv", true);
  if (std::strcmp(operation, "qgemm") == 0) return qgemm_like(call, "qgemm", false);
  if (std::strcmp(operation, "int8_gemm") == 0) return int8_gemm(call);
  if (std::strcmp(operation, "qgemv_up_gate") == 0) return fused(call, "qgemv_up_gate", 2, 2);
  if (std::strcmp(operation, "qgemv_up_gate_activation") == 0) return fused(call, "qgemv_up_gate_activation", 2, 1);
  if (std::strcmp(operation, "qgemv_qkv") == 0) return fused(call, "qgemv_qkv", 3, 3);
  return make(StatusCode::adapter_not_wired, operation,
              "not part of the quantized-matmul path served by this library");
}

#ifdef QX_B200_HAVE_REFERENCE_KERNEL_ABI
}  // namespace quixicore::b200::contract_api
#include "quixicore/contract/operations.hpp"
namespace quixicore::b200::contract_api {
// Same, keyed by the reference's generated OperationId.
[[nodiscard]] inline quixicore::contract::Status dispatch(
    quixicore::contract::OperationId operation, const quixicore::contract::KernelCall& call) noexcept {
  const auto name = quixicore::contract::operation_name(operation);
  char buffer[64] = {0};
  if (name.empty() || name.size() >= sizeof buffer) return dispatch(static_cast<const char*>(nullptr), call);
  std::memcpy(buffer, name.data(), name.size());
  return dispatch(buffer, call);
}
#endif

}  // namespace quixicore::b200::contract_api
