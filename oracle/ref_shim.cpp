// TEST INFRASTRUCTURE ONLY: a C-ABI wrapper around the unmodified QuixiCore-CPU
// reference library, so Python tests and the CPU-baseline leg of the bench can
// call the reference's own public dispatch entry points. Nothing on the
// product path links or loads this file. It contains no reference code: it only
// forwards to the public functions declared in the reference's headers
// (include/quixicore_cpu/qgemv.h, qgemm.h, packed_weights.h, threading.h).

#include <cstddef>
#include <cstdint>
#include <new>

#include "kernels/common/fp16.h"
#include "quixicore_cpu/float_storage.h"
#include "quixicore_cpu/packed_weights.h"
#include "quixicore_cpu/qgemm.h"
#include "quixicore_cpu/qgemv.h"
#include "quixicore_cpu/threading.h"

namespace qc = quixicore_cpu;

extern "C" {

int qxref_qgemv_packed_size(int format, long long n, long long k,
                            size_t* size) {
  return static_cast<int>(
      qc::qgemv_packed_size(static_cast<qc::QuantFormat>(format), n, k, size));
}

int qxref_qgemv_pack(int format, const float* weights, long long n,
                     long long k, void* packed) {
  return static_cast<int>(qc::qgemv_pack(static_cast<qc::QuantFormat>(format),
                                         weights, n, k, packed));
}

int qxref_qgemv_unpack(int format, const void* packed, long long n,
                       long long k, float* weights) {
  return static_cast<int>(qc::qgemv_unpack(
      static_cast<qc::QuantFormat>(format), packed, n, k, weights));
}

int qxref_qgemv(int format, const void* packed, const float* x, float* y,
                long long n, long long k) {
  return static_cast<int>(
      qc::qgemv(static_cast<qc::QuantFormat>(format), packed, x, y, n, k));
}

int qxref_qgemm(int format, const void* packed, const float* x, float* y,
                long long m, long long n, long long k) {
  return static_cast<int>(
      qc::qgemm(static_cast<qc::QuantFormat>(format), packed, x, y, m, n, k));
}

int qxref_int8_gemm(const int8_t* weights, const int8_t* x,
                    const float* weight_scale, const float* activation_scale,
                    const int32_t* weight_row_sum,
                    const int* activation_zero_point, float* y, long long m,
                    long long n, long long k, int asymmetric) {
  return static_cast<int>(qc::int8_gemm(weights, x, weight_scale,
                                        activation_scale, weight_row_sum,
                                        activation_zero_point, y, m, n, k,
                                        asymmetric != 0));
}

int qxref_qgemm_w8a8(const int8_t* weights, const int8_t* x,
                     const float* weight_scale, const float* activation_scale,
                     float* y, long long m, long long n, long long k) {
  return static_cast<int>(
      qc::qgemm_w8a8(weights, x, weight_scale, activation_scale, y, m, n, k));
}

int qxref_qgemm_w8a32(const int8_t* weights, const float* weight_scale,
                      const float* x, float* y, long long m, long long n,
                      long long k) {
  return static_cast<int>(
      qc::qgemm_w8a32(weights, weight_scale, x, y, m, n, k));
}

// Prepared-weights handle (quixicore_cpu::CpuPackedWeights).
int qxref_packed_create(int format, const void* contract_packed,
                        long long rows, long long columns, int layout,
                        void** handle) {
  auto* weights = new (std::nothrow) qc::CpuPackedWeights();
  if (weights == nullptr) return static_cast<int>(qc::Status::kOutOfMemory);
  const qc::Status status =
      weights->prepare(static_cast<qc::QuantFormat>(format), contract_packed,
                       rows, columns, static_cast<qc::CpuPanelLayout>(layout));
  if (status != qc::Status::kOk) {
    delete weights;
    *handle = nullptr;
    return static_cast<int>(status);
  }
  *handle = weights;
  return 0;
}

void qxref_packed_destroy(void* handle) {
  delete static_cast<qc::CpuPackedWeights*>(handle);
}

// out[0..5] = rows, columns, row_tile, blocks_per_row, block_bytes, panel_bytes
void qxref_packed_info(const void* handle, long long* out) {
  const qc::CpuPackedWeightsInfo info =
      static_cast<const qc::CpuPackedWeights*>(handle)->info();
  out[0] = info.rows;
  out[1] = info.columns;
  out[2] = info.row_tile;
  out[3] = info.blocks_per_row;
  out[4] = static_cast<long long>(info.block_bytes);
  out[5] = static_cast<long long>(info.panel_bytes);
}

const void* qxref_packed_panel(const void* handle) {
  return static_cast<const qc::CpuPackedWeights*>(handle)->panel_data();
}

int qxref_qgemm_prepacked(const void* handle, const float* x, float* y,
                          long long m) {
  return static_cast<int>(qc::qgemm_prepacked(
      *static_cast<const qc::CpuPackedWeights*>(handle), x, y, m, nullptr));
}

void qxref_set_num_threads(int n) { qc::set_num_threads(n); }
int qxref_num_threads() { return qc::num_threads(); }

const char* qxref_qgemv_variant(int format) {
  return qc::qgemv_variant(static_cast<qc::QuantFormat>(format));
}
const char* qxref_int8_gemm_variant() { return qc::int8_gemm_variant(); }
const char* qxref_qgemm_w8a32_variant() { return qc::qgemm_w8a32_variant(); }

uint16_t qxref_fp32_to_fp16(float value) { return qc::fp32_to_fp16(value); }
float qxref_fp16_to_fp32(uint16_t bits) { return qc::fp16_to_fp32(bits); }
uint16_t qxref_float_to_bf16(float value) { return qc::float_to_bf16(value); }
float qxref_bf16_to_float(uint16_t bits) { return qc::bf16_to_float(bits); }

}  // extern "C"

// ---- the callers either side of the GEMV: activation-quantising GEMV, fused decode
// projections, compact int4 rows, int8 activation quantiser -----------------------------
#include "quixicore_cpu/lowbit.h"
#include "quixicore_cpu/qgemv_w8a8.h"
#include "quixicore_cpu/quantization.h"

extern "C" {

int qxref_qgemv_w8a8(int format, const void* packed, const float* x, float* y,
                     long long n, long long k) {
  return static_cast<int>(qc::qgemv_w8a8(static_cast<qc::QuantFormat>(format),
                                         packed, x, y, n, k));
}
const char* qxref_qgemv_w8a8_variant(int format) {
  return qc::qgemv_w8a8_variant(static_cast<qc::QuantFormat>(format));
}
int qxref_qgemv_up_gate(int format, const void* up_w, const void* gate_w,
                        const float* x, float* up, float* gate, long long n,
                        long long k) {
  return static_cast<int>(qc::qgemv_up_gate(static_cast<qc::QuantFormat>(format),
                                            up_w, gate_w, x, up, gate, n, k));
}
int qxref_qgemv_up_gate_activation(int format, const void* up_w,
                                   const void* gate_w, const float* x,
                                   float* out, long long n, long long k,
                                   int gelu_tanh) {
  return static_cast<int>(qc::qgemv_up_gate_activation(
      static_cast<qc::QuantFormat>(format), up_w, gate_w, x, out, n, k,
      gelu_tanh != 0));
}
int qxref_qgemv_qkv(int format, const void* wq, const void* wk, const void* wv,
                    const float* x, float* q, float* k_out, float* v_out,
                    long long query_dim, long long kv_dim, long long input_dim) {
  return static_cast<int>(qc::qgemv_qkv(static_cast<qc::QuantFormat>(format), wq,
                                        wk, wv, x, q, k_out, v_out, query_dim,
                                        kv_dim, input_dim));
}
int qxref_quantize_int8(const float* x, int8_t* codes, float* scales,
                        long long rows, long long dim, long long group_size) {
  return static_cast<int>(
      qc::quantize_int8(x, codes, scales, rows, dim, group_size));
}
int qxref_lowbit_packed_size(int format, long long rows, long long dim,
                             long long group_size, size_t* weight_bytes,
                             size_t* scale_count) {
  return static_cast<int>(qc::lowbit_packed_size(
      static_cast<qc::LowBitFormat>(format), rows, dim, group_size,
      weight_bytes, scale_count));
}
int qxref_lowbit_pack(int format, const float* weights, uint8_t* packed,
                      float* scales, long long rows, long long dim,
                      long long group_size) {
  return static_cast<int>(qc::lowbit_pack(static_cast<qc::LowBitFormat>(format),
                                          weights, packed, scales, rows, dim,
                                          group_size));
}
int qxref_lowbit_unpack(int format, const uint8_t* packed, const float* scales,
                        float* weights, long long rows, long long dim,
                        long long group_size) {
  return static_cast<int>(qc::lowbit_unpack(
      static_cast<qc::LowBitFormat>(format), packed, scales, weights, rows, dim,
      group_size));
}
int qxref_lowbit_gemm(int format, const uint8_t* packed, const float* scales,
                      const float* x, float* y, long long m, long long n,
                      long long k, long long group_size) {
  return static_cast<int>(qc::lowbit_gemm(static_cast<qc::LowBitFormat>(format),
                                          packed, scales, x, y, m, n, k,
                                          group_size));
}
int qxref_lowbit_gemm_w8a8(const uint8_t* packed, const float* scales,
                           const float* x, float* y, long long m, long long n,
                           long long k) {
  return static_cast<int>(qc::lowbit_gemm_w8a8(packed, scales, x, y, m, n, k));
}
const char* qxref_lowbit_gemm_w8a8_variant() {
  return qc::lowbit_gemm_w8a8_variant();
}
const char* qxref_lowbit_gemm_variant(int format) {
  return qc::lowbit_gemm_variant(static_cast<qc::LowBitFormat>(format));
}

}  // extern "C"

// ---- canonical prepared projections: CanonicalQuantTensor -> CpuPackedWeights::prepare ->
// qgemm_prepacked_epilogue_storage, the canonical quantiser and the SmoothQuant importer ---
#include <algorithm>
#include <vector>

#include "quixicore_cpu/ops.h"
#include "quixicore_cpu/quant_import.h"

extern "C" {

// quantize_canonical for a layout with f32 scales (int8 / int4 symmetric): writes the
// canonical bytes, the scale table and the metadata the projection needs.
int qxref_quantize_canonical(int layout, const float* values, long long rows,
                             long long columns, long long group_size,
                             uint8_t* data, size_t data_capacity, float* scales,
                             size_t scale_capacity, size_t* data_bytes,
                             size_t* scale_count, int* scale_mode,
                             long long* stored_group_size) {
  qc::CanonicalQuantTensor tensor;
  const qc::Status status = qc::quantize_canonical(
      {values, qc::FloatStorageType::kF32, rows * columns}, rows, columns,
      static_cast<qc::CanonicalQuantLayout>(layout), group_size, &tensor);
  if (status != qc::Status::kOk) return static_cast<int>(status);
  if (tensor.data.size() > data_capacity || tensor.scales.size() > scale_capacity) {
    return static_cast<int>(qc::Status::kInvalidShape);
  }
  std::copy(tensor.data.begin(), tensor.data.end(), data);
  std::copy(tensor.scales.begin(), tensor.scales.end(), scales);
  *data_bytes = tensor.data.size();
  *scale_count = tensor.scales.size();
  *scale_mode = static_cast<int>(tensor.metadata.scale_mode);
  *stored_group_size = tensor.metadata.group_size;
  return 0;
}

static qc::Status make_tensor(int layout, int scale_mode, long long rows,
                              long long columns, long long group_size,
                              const uint8_t* data, size_t data_bytes,
                              const float* scales, size_t scale_count,
                              qc::CanonicalQuantTensor* tensor) {
  tensor->metadata.layout = static_cast<qc::CanonicalQuantLayout>(layout);
  tensor->metadata.logical_rows = rows;
  tensor->metadata.logical_columns = columns;
  tensor->metadata.group_size = group_size;
  tensor->metadata.scale_mode = static_cast<qc::QuantScaleMode>(scale_mode);
  tensor->metadata.scale_encoding = qc::QuantScaleEncoding::kFP32;
  tensor->metadata.scale_count = scale_count;
  tensor->data.assign(data, data + data_bytes);
  tensor->scales.assign(scales, scales + scale_count);
  return qc::validate_canonical_quant_tensor(*tensor);
}

// validate_canonical_quant_tensor on a tensor assembled from plain arrays
int qxref_canonical_validate(int layout, int scale_mode, long long rows,
                             long long columns, long long group_size,
                             const uint8_t* data, size_t data_bytes,
                             const float* scales, size_t scale_count) {
  qc::CanonicalQuantTensor tensor;
  return static_cast<int>(make_tensor(layout, scale_mode, rows, columns, group_size,
                                      data, data_bytes, scales, scale_count, &tensor));
}

// CpuPackedWeights::prepare(tensor) + qgemm_prepacked_epilogue_storage
int qxref_canonical_gemm(int layout, int scale_mode, long long rows,
                         long long columns, long long group_size,
                         const uint8_t* data, size_t data_bytes,
                         const float* scales, size_t scale_count, const void* x,
                         int x_type, long long x_count, const float* bias, void* y,
                         int y_type, long long y_count, long long m,
                         int activation) {
  qc::CanonicalQuantTensor tensor;
  qc::Status status = make_tensor(layout, scale_mode, rows, columns, group_size, data,
                                  data_bytes, scales, scale_count, &tensor);
  if (status != qc::Status::kOk) return static_cast<int>(status);
  qc::CpuPackedWeights prepared;
  status = prepared.prepare(tensor);
  if (status != qc::Status::kOk) return static_cast<int>(status);
  return static_cast<int>(qc::qgemm_prepacked_epilogue_storage(
      prepared, {x, static_cast<qc::FloatStorageType>(x_type), x_count}, bias,
      {y, static_cast<qc::FloatStorageType>(y_type), y_count}, m,
      static_cast<qc::LinearActivation>(activation)));
}

// import_smoothquant_w8a8: returns the tensor's fields through plain arrays
int qxref_import_smoothquant(const int8_t* weights, size_t weight_count,
                             const float* weight_scales, size_t weight_scale_count,
                             const float* activation_scales,
                             size_t activation_scale_count,
                             const int* activation_zero_points,
                             size_t activation_zero_point_count,
                             const int32_t* row_sums, size_t row_sum_count,
                             long long rows, long long columns, uint8_t* data_out,
                             float* scales_out, int32_t* row_sums_out, int* layout,
                             int* scale_mode, long long* group_size) {
  qc::SmoothQuantW8A8Source source;
  source.weights = weights;
  source.weight_count = weight_count;
  source.weight_scales = weight_scales;
  source.weight_scale_count = weight_scale_count;
  source.activation_scales = activation_scales;
  source.activation_scale_count = activation_scale_count;
  source.activation_zero_points = activation_zero_points;
  source.activation_zero_point_count = activation_zero_point_count;
  source.row_sums = row_sums;
  source.row_sum_count = row_sum_count;
  source.rows = rows;
  source.columns = columns;
  qc::CanonicalQuantTensor tensor;
  const qc::Status status = qc::import_smoothquant_w8a8(source, &tensor);
  if (status != qc::Status::kOk) return static_cast<int>(status);
  std::copy(tensor.data.begin(), tensor.data.end(), data_out);
  std::copy(tensor.scales.begin(), tensor.scales.end(), scales_out);
  std::copy(tensor.row_sums.begin(), tensor.row_sums.end(), row_sums_out);
  *layout = static_cast<int>(tensor.metadata.layout);
  *scale_mode = static_cast<int>(tensor.metadata.scale_mode);
  *group_size = tensor.metadata.group_size;
  return 0;
}


// tensors with zero points and the GPTQ column maps
static qc::Status make_tensor_ex(int layout, int scale_mode, long long rows, long long columns,
                                 long long group_size, const uint8_t* data, size_t data_bytes,
                                 const float* scales, size_t scale_count, const float* zeros,
                                 size_t zero_count, const int* group_index, size_t group_index_count,
                                 const int* act_order, size_t act_order_count,
                                 qc::CanonicalQuantTensor* tensor) {
  tensor->metadata.layout = static_cast<qc::CanonicalQuantLayout>(layout);
  tensor->metadata.logical_rows = rows;
  tensor->metadata.logical_columns = columns;
  tensor->metadata.group_size = group_size;
  tensor->metadata.scale_mode = static_cast<qc::QuantScaleMode>(scale_mode);
  tensor->metadata.scale_encoding = qc::QuantScaleEncoding::kFP32;
  tensor->metadata.scale_count = scale_count;
  tensor->metadata.zero_point_mode =
      zero_count != 0 ? qc::QuantZeroPointMode::kFractional : qc::QuantZeroPointMode::kNone;
  tensor->metadata.zero_point_count = zero_count;
  tensor->metadata.group_index_count = group_index_count;
  tensor->metadata.act_order_count = act_order_count;
  tensor->data.assign(data, data + data_bytes);
  tensor->scales.assign(scales, scales + scale_count);
  if (zero_count != 0) tensor->zero_points.assign(zeros, zeros + zero_count);
  if (group_index_count != 0) tensor->group_index.assign(group_index, group_index + group_index_count);
  if (act_order_count != 0) tensor->act_order.assign(act_order, act_order + act_order_count);
  return qc::validate_canonical_quant_tensor(*tensor);
}

int qxref_canonical_gemm_ex(int layout, int scale_mode, long long rows, long long columns,
                            long long group_size, const uint8_t* data, size_t data_bytes,
                            const float* scales, size_t scale_count, const float* zeros,
                            size_t zero_count, const int* group_index, size_t group_index_count,
                            const int* act_order, size_t act_order_count, const void* x,
                            int x_type, long long x_count, const float* bias, void* y,
                            int y_type, long long y_count, long long m, int activation) {
  qc::CanonicalQuantTensor tensor;
  qc::Status status = make_tensor_ex(layout, scale_mode, rows, columns, group_size, data, data_bytes,
                                     scales, scale_count, zeros, zero_count, group_index,
                                     group_index_count, act_order, act_order_count, &tensor);
  if (status != qc::Status::kOk) return static_cast<int>(status);
  qc::CpuPackedWeights prepared;
  status = prepared.prepare(tensor);
  if (status != qc::Status::kOk) return static_cast<int>(status);
  return static_cast<int>(qc::qgemm_prepacked_epilogue_storage(
      prepared, {x, static_cast<qc::FloatStorageType>(x_type), x_count}, bias,
      {y, static_cast<qc::FloatStorageType>(y_type), y_count}, m,
      static_cast<qc::LinearActivation>(activation)));
}

static int export_tensor(const qc::CanonicalQuantTensor& tensor, uint8_t* data_out, float* scales_out,
                         float* zeros_out, int* meta) {
  std::copy(tensor.data.begin(), tensor.data.end(), data_out);
  std::copy(tensor.scales.begin(), tensor.scales.end(), scales_out);
  std::copy(tensor.zero_points.begin(), tensor.zero_points.end(), zeros_out);
  meta[0] = static_cast<int>(tensor.metadata.layout);
  meta[1] = static_cast<int>(tensor.metadata.scale_mode);
  meta[2] = static_cast<int>(tensor.metadata.group_size);
  meta[3] = static_cast<int>(tensor.zero_points.size());
  meta[4] = static_cast<int>(tensor.group_index.size());
  meta[5] = static_cast<int>(tensor.act_order.size());
  return 0;
}

int qxref_import_awq_u4(const uint32_t* qweight, size_t qweight_words, const uint32_t* qzeros,
                        size_t qzero_words, const float* scales, size_t scale_count,
                        long long input_features, long long output_features, long long group_size,
                        uint8_t* data_out, float* scales_out, float* zeros_out, int* meta) {
  qc::AwqU4Source source;
  source.qweight = qweight;
  source.qweight_words = qweight_words;
  source.qzeros = qzeros;
  source.qzero_words = qzero_words;
  source.scales = scales;
  source.scale_count = scale_count;
  source.input_features = input_features;
  source.output_features = output_features;
  source.group_size = group_size;
  qc::CanonicalQuantTensor tensor;
  const qc::Status status = qc::import_awq_u4(source, &tensor);
  if (status != qc::Status::kOk) return static_cast<int>(status);
  return export_tensor(tensor, data_out, scales_out, zeros_out, meta);
}

int qxref_import_gptq_u4(const uint32_t* qweight, size_t qweight_words, const uint32_t* qzeros,
                         size_t qzero_words, const float* scales, size_t scale_count,
                         const int* group_index, size_t group_index_count, const int* act_order,
                         size_t act_order_count, long long input_features,
                         long long output_features, long long group_size, int symmetric,
                         int gptq_v2, uint8_t* data_out, float* scales_out, float* zeros_out,
                         int* meta) {
  qc::GptqU4Source source;
  source.qweight = qweight;
  source.qweight_words = qweight_words;
  source.qzeros = qzeros;
  source.qzero_words = qzero_words;
  source.scales = scales;
  source.scale_count = scale_count;
  source.group_index = group_index;
  source.group_index_count = group_index_count;
  source.act_order = act_order;
  source.act_order_count = act_order_count;
  source.input_features = input_features;
  source.output_features = output_features;
  source.group_size = group_size;
  source.symmetric = symmetric != 0;
  source.gptq_v2 = gptq_v2 != 0;
  qc::CanonicalQuantTensor tensor;
  const qc::Status status = qc::import_gptq_u4(source, &tensor);
  if (status != qc::Status::kOk) return static_cast<int>(status);
  return export_tensor(tensor, data_out, scales_out, zeros_out, meta);
}

}  // extern "C"
