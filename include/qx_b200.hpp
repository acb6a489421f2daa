// C++ face of the qx_b200 C ABI with the names and calling conventions of the reference's
// public API for this path (namespace quixicore_cpu): a translation unit written against
//   include/quixicore_cpu/status.h, qgemv.h, qgemm.h, packed_weights.h, threading.h
// of the reference compiles against this header instead and links libqx_b200.so.
// Header-only; every function forwards to the C entry point named in its comment.
// Differences from the reference, all additive: Status::kDeviceError (a CUDA failure or no
// sm_100 device; last_error() has the text), and only QuantFormat::kQ8_0 / kQ4_0 are served
// (every other format reports kUnsupportedFormat).
#pragma once

#include <cstddef>
#include <cstdint>
#include <utility>

#include "qx_b200.h"

namespace quixicore_cpu {

// include/quixicore_cpu/status.h:5-11 (values identical) + one additive value
enum class Status : int {
  kOk = 0,
  kInvalidShape = 1,
  kUnsupportedFormat = 2,
  kInvalidArgument = 3,
  kOutOfMemory = 4,
  kDeviceError = 5,
};

// include/quixicore_cpu/qgemv.h:10-51: numeric values are part of the contract; the two
// formats of this path
enum class QuantFormat : int {
  kQ8_0 = 0,
  kQ4_0 = 1,
};

inline Status to_status(qx_status s) { return static_cast<Status>(static_cast<int>(s)); }
inline const char* last_error() { return qx_last_error_string(); }

// include/quixicore_cpu/qgemv.h:68-71 -> qx_qgemv_packed_size
inline Status qgemv_packed_size(QuantFormat format, long long n, long long k, std::size_t* size) {
  return to_status(qx_qgemv_packed_size(static_cast<int>(format), n, k, size));
}
// src/dispatch/qgemv.cpp:210-300 -> qx_qgemv_pack / qx_qgemv_unpack
inline Status qgemv_pack(QuantFormat format, const float* weights, long long n, long long k,
                         void* packed) {
  return to_status(qx_qgemv_pack(static_cast<int>(format), weights, n, k, packed));
}
inline Status qgemv_unpack(QuantFormat format, const void* packed, long long n, long long k,
                           float* weights) {
  return to_status(qx_qgemv_unpack(static_cast<int>(format), packed, n, k, weights));
}
// include/quixicore_cpu/qgemv.h:108-109 -> qx_qgemv
inline Status qgemv(QuantFormat format, const void* packed, const float* x, float* y, long long n,
                    long long k) {
  return to_status(qx_qgemv(static_cast<int>(format), packed, x, y, n, k));
}
// include/quixicore_cpu/qgemm.h:19-20 -> qx_qgemm
inline Status qgemm(QuantFormat format, const void* packed_weights, const float* x, float* y,
                    long long m, long long n, long long k) {
  return to_status(qx_qgemm(static_cast<int>(format), packed_weights, x, y, m, n, k));
}
inline const char* qgemv_variant(QuantFormat format) {
  return qx_qgemv_variant(static_cast<int>(format));
}

// include/quixicore_cpu/packed_weights.h:14-20, same enumerators and values. The argument
// selects a CPU row tile in the reference; the device panel has one layout (tiles of 128
// rows), so every value is accepted and info().layout reports kAuto.
enum class CpuPanelLayout {
  kAuto,
  kPortableRows1,
  kNeonRows4,
  kAvx2Rows8,
  kAvx512Rows16,
};

// include/quixicore_cpu/packed_weights.h:36-67: the fields that have a meaning for q8_0 /
// q4_0 weights on the device, under the reference's names.
struct CpuPackedWeightsInfo {
  QuantFormat format = QuantFormat::kQ8_0;
  CpuPanelLayout layout = CpuPanelLayout::kAuto;
  long long rows = 0;
  long long columns = 0;
  long long row_tile = 0;      // 128 on the device
  long long block_size = 0;
  long long blocks_per_row = 0;
  std::size_t block_bytes = 0;
  std::size_t contract_bytes = 0;
  std::size_t panel_bytes = 0;
  std::size_t prepared_bytes = 0;
  double memory_amplification = 0.0;
  std::uint64_t preparation_ns = 0;
};

using Workspace = qx_workspace;  // opaque; nullptr = the library's own

// include/quixicore_cpu/packed_weights.h:72-97 (move-only owner of prepared weights) ->
// qx_weights_prepare / qx_weights_get_info / qx_weights_destroy. The handle owns a device
// copy; the caller may free the canonical bytes after prepare().
class CpuPackedWeights {
 public:
  CpuPackedWeights() = default;
  CpuPackedWeights(const CpuPackedWeights&) = delete;
  CpuPackedWeights& operator=(const CpuPackedWeights&) = delete;
  CpuPackedWeights(CpuPackedWeights&& other) noexcept : handle_(std::exchange(other.handle_, nullptr)) {}
  CpuPackedWeights& operator=(CpuPackedWeights&& other) noexcept {
    if (this != &other) {
      reset();
      handle_ = std::exchange(other.handle_, nullptr);
    }
    return *this;
  }
  ~CpuPackedWeights() { reset(); }

  Status prepare(QuantFormat format, const void* packed, long long rows, long long columns,
                 CpuPanelLayout /*layout*/ = CpuPanelLayout::kAuto) {
    return prepare_rows(format, packed, rows, columns, 0, rows);
  }
  // additive: keep only rows [row_begin, row_begin + row_count) on this GPU (row sharding)
  Status prepare_rows(QuantFormat format, const void* packed, long long rows, long long columns,
                      long long row_begin, long long row_count) {
    qx_weights* fresh = nullptr;
    const Status status = to_status(qx_weights_prepare(static_cast<int>(format), packed, rows, columns,
                                                       row_begin, row_count, &fresh));
    if (status == Status::kOk) {  // like the reference: a failed prepare leaves *this untouched
      reset();
      handle_ = fresh;
    }
    return status;
  }
  bool ready() const noexcept { return handle_ != nullptr; }
  void reset() noexcept {
    qx_weights_destroy(handle_);
    handle_ = nullptr;
  }
  CpuPackedWeightsInfo info() const {
    CpuPackedWeightsInfo out;
    qx_weights_info raw{};
    if (handle_ != nullptr && qx_weights_get_info(handle_, &raw) == QX_STATUS_OK) {
      out.format = static_cast<QuantFormat>(raw.format);
      out.rows = raw.rows;
      out.columns = raw.columns;
      out.block_size = raw.block_size;
      out.blocks_per_row = raw.blocks_per_row;
      out.block_bytes = raw.block_bytes;
      out.contract_bytes = raw.contract_bytes;
      out.prepared_bytes = raw.prepared_bytes;
      out.memory_amplification = raw.memory_amplification;
      out.preparation_ns = raw.preparation_ns;
      out.row_tile = raw.row_tile;
      out.panel_bytes = raw.panel_bytes;
    }
    return out;
  }
  // packed_weights.h:89-90. The canonical bytes are not kept once the device panel is built
  // (the caller still owns its copy), so contract_data() is null; panel_data() is the
  // DEVICE address of the panel.
  const void* contract_data() const noexcept { return nullptr; }
  const void* panel_data() const noexcept { return qx_weights_panel_dev(handle_); }
  const qx_weights* handle() const noexcept { return handle_; }

 private:
  qx_weights* handle_ = nullptr;
};

// include/quixicore_cpu/qgemm.h:26-27 -> qx_qgemm_prepacked
inline Status qgemm_prepacked(const CpuPackedWeights& weights, const float* x, float* y, long long m,
                              Workspace* workspace = nullptr) {
  return to_status(qx_qgemm_prepacked(weights.handle(), x, y, m, workspace));
}

// include/quixicore_cpu/qgemm.h:235-257 -> qx_int8_gemm / qx_qgemm_w8a8[_azp] / qx_qgemm_w8a32
inline Status int8_gemm(const std::int8_t* weights, const std::int8_t* x, const float* weight_scale,
                        const float* activation_scale, const std::int32_t* weight_row_sum,
                        const int* activation_zero_point, float* y, long long m, long long n,
                        long long k, bool asymmetric = false) {
  return to_status(qx_int8_gemm(weights, x, weight_scale, activation_scale, weight_row_sum,
                                activation_zero_point, y, m, n, k, asymmetric ? 1 : 0));
}
inline Status qgemm_w8a8(const std::int8_t* weights, const std::int8_t* x, const float* weight_scale,
                         const float* activation_scale, float* y, long long m, long long n,
                         long long k) {
  return to_status(qx_qgemm_w8a8(weights, x, weight_scale, activation_scale, y, m, n, k));
}
inline Status qgemm_w8a8_azp(const std::int8_t* weights, const std::int8_t* x, const float* weight_scale,
                             const float* activation_scale, const std::int32_t* weight_row_sum,
                             const int* activation_zero_point, float* y, long long m, long long n,
                             long long k) {
  return to_status(qx_qgemm_w8a8_azp(weights, x, weight_scale, activation_scale, weight_row_sum,
                                     activation_zero_point, y, m, n, k));
}
inline Status qgemm_w8a32(const std::int8_t* weights, const float* weight_scale, const float* x,
                          float* y, long long m, long long n, long long k) {
  return to_status(qx_qgemm_w8a32(weights, weight_scale, x, y, m, n, k));
}
inline const char* int8_gemm_variant() { return qx_int8_gemm_variant(); }
inline const char* qgemm_w8a32_variant() { return qx_qgemm_w8a32_variant(); }

// include/quixicore_cpu/qgemv_w8a8.h:17-29 -> qx_qgemv_w8a8*
inline Status qgemv_w8a8(QuantFormat format, const void* packed_weights, const float* x, float* y,
                         long long n, long long k) {
  return to_status(qx_qgemv_w8a8(static_cast<int>(format), packed_weights, x, y, n, k));
}
inline Status qgemv_w8a8_packed_size(QuantFormat format, long long n, long long k, long long* bytes) {
  return to_status(qx_qgemv_w8a8_packed_size(static_cast<int>(format), n, k, bytes));
}
inline Status qgemv_w8a8_pack(QuantFormat format, const float* weights, long long n, long long k,
                              void* packed) {
  return to_status(qx_qgemv_w8a8_pack(static_cast<int>(format), weights, n, k, packed));
}
inline const char* qgemv_w8a8_variant(QuantFormat format) {
  return qx_qgemv_w8a8_variant(static_cast<int>(format));
}

// include/quixicore_cpu/qgemv.h:143-154 -> qx_qgemv_up_gate[_activation] / qx_qgemv_qkv
inline Status qgemv_up_gate(QuantFormat format, const void* packed_up, const void* packed_gate,
                            const float* x, float* up, float* gate, long long n, long long k) {
  return to_status(qx_qgemv_up_gate(static_cast<int>(format), packed_up, packed_gate, x, up, gate, n, k));
}
inline Status qgemv_up_gate_activation(QuantFormat format, const void* packed_up,
                                       const void* packed_gate, const float* x, float* out,
                                       long long n, long long k, bool gelu_tanh = true) {
  return to_status(qx_qgemv_up_gate_activation(static_cast<int>(format), packed_up, packed_gate, x, out,
                                               n, k, gelu_tanh ? 1 : 0));
}
inline Status qgemv_qkv(QuantFormat format, const void* packed_q, const void* packed_k,
                        const void* packed_v, const float* x, float* q, float* k_out, float* v_out,
                        long long query_dim, long long kv_dim, long long input_dim) {
  return to_status(qx_qgemv_qkv(static_cast<int>(format), packed_q, packed_k, packed_v, x, q, k_out,
                                v_out, query_dim, kv_dim, input_dim));
}

// include/quixicore_cpu/lowbit.h:15-47 (values identical) -> qx_lowbit_*
enum class LowBitFormat {
  kInt2Row,
  kInt3Group64,
  kInt4Row,
  kInt4Group,
};
inline Status lowbit_packed_size(LowBitFormat format, long long rows, long long dim,
                                 long long group_size, std::size_t* weight_bytes,
                                 std::size_t* scale_count) {
  return to_status(qx_lowbit_packed_size(static_cast<int>(format), rows, dim, group_size, weight_bytes,
                                         scale_count));
}
inline Status lowbit_pack(LowBitFormat format, const float* weights, std::uint8_t* packed,
                          float* scales, long long rows, long long dim, long long group_size = 0) {
  return to_status(qx_lowbit_pack(static_cast<int>(format), weights, packed, scales, rows, dim, group_size));
}
inline Status lowbit_unpack(LowBitFormat format, const std::uint8_t* packed, const float* scales,
                            float* weights, long long rows, long long dim, long long group_size = 0) {
  return to_status(qx_lowbit_unpack(static_cast<int>(format), packed, scales, weights, rows, dim, group_size));
}
inline Status lowbit_gemm(LowBitFormat format, const std::uint8_t* packed_weights,
                          const float* weight_scales, const float* x, float* y, long long m,
                          long long n, long long k, long long group_size = 0) {
  return to_status(qx_lowbit_gemm(static_cast<int>(format), packed_weights, weight_scales, x, y, m, n, k,
                                  group_size));
}
inline Status lowbit_gemm_w8a8(const std::uint8_t* packed_weights, const float* weight_scales,
                               const float* x, float* y, long long m, long long n, long long k) {
  return to_status(qx_lowbit_gemm_w8a8(packed_weights, weight_scales, x, y, m, n, k));
}
inline const char* lowbit_gemm_w8a8_variant() { return qx_lowbit_gemm_w8a8_variant(); }
inline const char* lowbit_gemm_variant(LowBitFormat format) {
  return qx_lowbit_gemm_variant(static_cast<int>(format));
}
// include/quixicore_cpu/quantization.h:42-43 -> qx_quantize_int8
inline Status quantize_int8(const float* x, std::int8_t* codes, float* scales, long long rows,
                            long long dim, long long group_size) {
  return to_status(qx_quantize_int8(x, codes, scales, rows, dim, group_size));
}

// include/quixicore_cpu/threading.h: kept for source compatibility (the GPU path has no
// thread pool; the value is stored and returned)
// ---- canonical prepared projections ---------------------------------------------------
// include/quixicore_cpu/quant_contract.h:12-38, float_storage.h:18-30, ops.h:56 (values equal)
enum class CanonicalQuantLayout : int { kInt4Symmetric = 0, kUInt4Affine = 1, kInt8Symmetric = 2 };
enum class QuantScaleMode : int { kNone = 0, kTensor = 1, kRow = 2, kChannel = 3, kGroup = 4 };
enum class FloatStorageType : int { kF32 = 0, kF16 = 1, kBF16 = 2 };
enum class LinearActivation : int { kNone = 0, kGeluErf = 1, kGeluTanh = 2, kSilu = 3, kRelu2 = 4 };
struct FloatStorageInput {
  const void* data = nullptr;
  FloatStorageType type = FloatStorageType::kF32;
  long long count = 0;
};
struct FloatStorageOutput {
  void* data = nullptr;
  FloatStorageType type = FloatStorageType::kF32;
  long long count = 0;
};
// The fields of quixicore_cpu::CanonicalQuantTensor (include/quixicore_cpu/quant_import.h:24-36)
// this path reads, as a view over the caller's arrays.
struct CanonicalQuantTensorView {
  CanonicalQuantLayout layout = CanonicalQuantLayout::kInt8Symmetric;
  QuantScaleMode scale_mode = QuantScaleMode::kRow;
  long long logical_rows = 0, logical_columns = 0, group_size = 0;
  const std::uint8_t* data = nullptr;
  std::size_t data_bytes = 0;
  const float* scales = nullptr;
  std::size_t scale_count = 0;
  const float* zero_points = nullptr;   // kUInt4Affine
  std::size_t zero_point_count = 0;
  const int* group_index = nullptr;     // GPTQ: packed column -> scale group
  std::size_t group_index_count = 0;
  const int* act_order = nullptr;       // GPTQ: packed column -> activation column
  std::size_t act_order_count = 0;
};
inline qx_canonical_tensor to_c(const CanonicalQuantTensorView& t) {
  return qx_canonical_tensor{static_cast<int>(t.layout), static_cast<int>(t.scale_mode), t.logical_rows,
                             t.logical_columns, t.group_size, t.data, t.data_bytes, t.scales,
                             t.scale_count, t.zero_points, t.zero_point_count, t.group_index,
                             t.group_index_count, t.act_order, t.act_order_count};
}
inline CanonicalQuantTensorView from_c(const qx_canonical_tensor& v) {
  CanonicalQuantTensorView t;
  t.layout = static_cast<CanonicalQuantLayout>(v.layout);
  t.scale_mode = static_cast<QuantScaleMode>(v.scale_mode);
  t.logical_rows = v.rows;
  t.logical_columns = v.columns;
  t.group_size = v.group_size;
  t.data = v.data;
  t.data_bytes = v.data_bytes;
  t.scales = v.scales;
  t.scale_count = v.scale_count;
  t.zero_points = v.zero_points;
  t.zero_point_count = v.zero_point_count;
  t.group_index = v.group_index;
  t.group_index_count = v.group_index_count;
  t.act_order = v.act_order;
  t.act_order_count = v.act_order_count;
  return t;
}
// CpuPackedWeights::prepare(const CanonicalQuantTensor&) (packed_weights.h) -> qx_canonical_prepare
class CanonicalPackedWeights {
 public:
  CanonicalPackedWeights() = default;
  CanonicalPackedWeights(const CanonicalPackedWeights&) = delete;
  CanonicalPackedWeights& operator=(const CanonicalPackedWeights&) = delete;
  ~CanonicalPackedWeights() { reset(); }
  Status prepare(const CanonicalQuantTensorView& t) {
    const qx_canonical_tensor view = to_c(t);
    qx_canonical_weights* fresh = nullptr;
    const Status status = to_status(qx_canonical_prepare(&view, &fresh));
    if (status == Status::kOk) {
      reset();
      handle_ = fresh;
    }
    return status;
  }
  bool ready() const noexcept { return handle_ != nullptr; }
  void reset() noexcept {
    qx_canonical_destroy(handle_);
    handle_ = nullptr;
  }
  const qx_canonical_weights* handle() const noexcept { return handle_; }

 private:
  qx_canonical_weights* handle_ = nullptr;
};
// include/quixicore_cpu/qgemm.h:32-42
inline Status qgemm_prepacked_epilogue_storage(const CanonicalPackedWeights& weights, FloatStorageInput x,
                                               const float* bias, FloatStorageOutput y, long long m,
                                               LinearActivation activation, Workspace* = nullptr) {
  return to_status(qx_qgemm_prepacked_epilogue_storage(weights.handle(), x.data, static_cast<int>(x.type),
                                                       x.count, bias, y.data, static_cast<int>(y.type),
                                                       y.count, m, static_cast<int>(activation)));
}
inline Status qgemm_prepacked_storage(const CanonicalPackedWeights& weights, FloatStorageInput x,
                                      FloatStorageOutput y, long long m, Workspace* = nullptr) {
  return to_status(qx_qgemm_prepacked_storage(weights.handle(), x.data, static_cast<int>(x.type), x.count,
                                              y.data, static_cast<int>(y.type), y.count, m));
}
// include/quixicore_cpu/quant_import.h:117-133: the view aliases the source's arrays; the row
// sums of the codes are written to row_sums[rows]
using SmoothQuantW8A8Source = qx_smoothquant_source;
inline Status import_smoothquant_w8a8(const SmoothQuantW8A8Source& source, CanonicalQuantTensorView* tensor,
                                      std::int32_t* row_sums) {
  if (tensor == nullptr) return Status::kInvalidArgument;
  qx_canonical_tensor view{};
  const Status status = to_status(qx_import_smoothquant_w8a8(&source, &view, row_sums));
  if (status == Status::kOk) *tensor = from_c(view);
  return status;
}
// include/quixicore_cpu/quant_import.h:56-92: the caller provides the arrays the view points at
// (data N*K/2 bytes, scales and zero points N*K/group floats)
using AwqU4Source = qx_awq_u4_source;
using GptqU4Source = qx_gptq_u4_source;
inline Status import_awq_u4(const AwqU4Source& source, CanonicalQuantTensorView* tensor, std::uint8_t* data,
                            float* scales, float* zero_points) {
  if (tensor == nullptr) return Status::kInvalidArgument;
  qx_canonical_tensor view{};
  const Status status = to_status(qx_import_awq_u4(&source, &view, data, scales, zero_points));
  if (status == Status::kOk) *tensor = from_c(view);
  return status;
}
inline Status import_gptq_u4(const GptqU4Source& source, CanonicalQuantTensorView* tensor, std::uint8_t* data,
                             float* scales, float* zero_points) {
  if (tensor == nullptr) return Status::kInvalidArgument;
  qx_canonical_tensor view{};
  const Status status = to_status(qx_import_gptq_u4(&source, &view, data, scales, zero_points));
  if (status == Status::kOk) *tensor = from_c(view);
  return status;
}

inline void set_num_threads(int n) { qx_set_num_threads(n); }
inline int num_threads() { return qx_num_threads(); }

}  // namespace quixicore_cpu
