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
