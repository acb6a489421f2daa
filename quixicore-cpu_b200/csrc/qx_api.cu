// extern "C" entry points. Validation order and status values follow the reference's
// dispatch layer (file:line given at each function); the host-pointer forms then stage
// the operands through device memory on the library's own stream and wait for the
// result, the `_dev` forms only enqueue.

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <limits>

#include "qx_gemv_tc.cuh"
#include "qx_int8_gemm.cuh"
#include "qx_weights.cuh"

namespace qx {
qx_status launch_pack(int format, const float* w_dev, long long total_blocks, void* packed_dev,
                      int* bad_dev, cudaStream_t stream);
qx_status launch_unpack(int format, const void* packed_dev, long long total_blocks, float* w_dev,
                        cudaStream_t stream);
qx_status launch_gate_activation(const float* up, const float* gate, float* out, long long n,
                                 bool gelu_tanh, cudaStream_t stream);
qx_status launch_q4_gemm_bf16(const qx_weights* w, const uint16_t* x_bf16_dev, float* y_dev,
                              long long m, long long ldy, qx_workspace* ws, cudaStream_t stream);

namespace {

// Carves 256-byte aligned pieces out of the context's staging buffer.
struct Staging {
  DeviceContext* ctx;
  size_t offset = 0;
  size_t sizes[8];
  int count = 0;
  size_t add(size_t bytes) {
    sizes[count++] = bytes;
    const size_t at = offset;
    offset += align_up(bytes == 0 ? 1 : bytes, 256);
    return at;
  }
  uint8_t* at(size_t off) const { return static_cast<uint8_t*>(ctx->staging) + off; }
};

qx_status h2d(void* dst, const void* src, size_t bytes, cudaStream_t s) {
  QX_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, s));
  return QX_STATUS_OK;
}
// Small inputs in pinned (device-addressable) host memory are fetched by a kernel instead of
// the copy engine: the kernel lets the compute kernel queued behind it start at once
// (programmatic dependent launch), so that one's weight prefetch runs while the activations
// cross PCIe; a copy-engine transfer in front of a kernel is a full dependency.
__global__ void __launch_bounds__(256) stage_in_kernel(const uint4* __restrict__ src,
                                                       uint4* __restrict__ dst, size_t n16) {
  asm volatile("griddepcontrol.launch_dependents;");
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n16) dst[i] = src[i];
}
qx_status stage_in(void* dst, const void* src, size_t bytes, cudaStream_t s) {
  constexpr size_t kLimit = 256 * 1024;
  if (bytes > 0 && bytes <= kLimit && bytes % 16 == 0 &&
      reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0) {
    cudaPointerAttributes attributes{};
    if (cudaPointerGetAttributes(&attributes, src) == cudaSuccess &&
        attributes.type == cudaMemoryTypeHost && attributes.devicePointer != nullptr) {
      const size_t n16 = bytes / 16;
      stage_in_kernel<<<static_cast<unsigned>((n16 + 255) / 256), 256, 0, s>>>(
          static_cast<const uint4*>(attributes.devicePointer), static_cast<uint4*>(dst), n16);
      count_launch();
      QX_CUDA_TRY(cudaGetLastError());
      return QX_STATUS_OK;
    }
    (void)cudaGetLastError();  // unregistered host memory is not an error here
  }
  return h2d(dst, src, bytes, s);
}
qx_status d2h(void* dst, const void* src, size_t bytes, cudaStream_t s) {
  QX_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, s));
  return QX_STATUS_OK;
}

qx_status take_device_error(DeviceContext* ctx);

// Waits for the stream and reports a kernel whose bounded wait gave up (it leaves its role
// code in the context's error word, host memory the kernels can address).
qx_status sync_and_check(DeviceContext* ctx, cudaStream_t s) {
  // Decode-sized calls finish within tens of microseconds: poll for a short while before
  // falling back to the blocking wait (whose wake-up alone costs about that much).
  const auto poll_until = std::chrono::steady_clock::now() + std::chrono::microseconds(150);
  cudaError_t state = cudaStreamQuery(s);
  while (state == cudaErrorNotReady && std::chrono::steady_clock::now() < poll_until) {
    state = cudaStreamQuery(s);
  }
  if (state == cudaErrorNotReady) {
    (void)cudaGetLastError();
    state = cudaStreamSynchronize(s);
  }
  if (state != cudaSuccess) {
    set_last_error("waiting for the stream", state);
    return QX_STATUS_DEVICE_ERROR;
  }
  return take_device_error(ctx);
}

// Reads and clears the error word of `ctx`; an aborted kernel may leave arrival counters
// behind, so the default workspace's counter area is cleared with it.
qx_status take_device_error(DeviceContext* ctx) {
  const int code = *static_cast<volatile int*>(ctx->error_host);
  if (code == 0) return QX_STATUS_OK;
  *static_cast<volatile int*>(ctx->error_host) = 0;
  if (ctx->workspace.base != nullptr) {
    (void)cudaMemset(ctx->workspace.base, 0, kWorkspaceCounterBytes);
  }
  char text[96];
  std::snprintf(text, sizeof text,
                "a kernel gave up a bounded wait (pipeline stalled, role code %d)", code);
  set_last_error_text(text);
  return QX_STATUS_DEVICE_ERROR;
}

bool all_finite_host(const float* v, long long count) {
  for (long long i = 0; i < count; ++i) {
    if (!std::isfinite(v[i])) return false;
  }
  return true;
}

}  // namespace
}  // namespace qx

using namespace qx;

extern "C" {

// src/dispatch/qgemv.cpp:198-208
qx_status qx_qgemv_packed_size(int format, long long n, long long k, size_t* size) {
  QX_TRY(validate_nk(format, n, k));
  if (size == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  return packed_bytes(format, n, k, size);
}

// src/dispatch/qgemv.cpp:215-275 (q8_0 / q4_0 branch)
qx_status qx_qgemv_pack(int format, const float* weights, long long n, long long k,
                        void* packed) {
  QX_TRY(validate_nk(format, n, k));
  size_t bytes = 0;
  if (packed_bytes(format, n, k, &bytes) != QX_STATUS_OK) return QX_STATUS_INVALID_SHAPE;
  if (weights == nullptr || packed == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  std::lock_guard<std::mutex> lock(ctx->mutex);
  Staging st{ctx};
  const size_t w_bytes = static_cast<size_t>(n) * k * sizeof(float);
  const size_t off_w = st.add(w_bytes), off_p = st.add(bytes);
  QX_TRY(ctx->ensure_staging(st.offset));
  QX_CUDA_TRY(cudaMemsetAsync(ctx->flag, 0, 4, ctx->stream));
  QX_TRY(h2d(st.at(off_w), weights, w_bytes, ctx->stream));
  QX_TRY(launch_pack(format, reinterpret_cast<const float*>(st.at(off_w)), n * (k / kBlockK),
                     st.at(off_p), ctx->flag, ctx->stream));
  int bad = 0;
  QX_TRY(d2h(&bad, ctx->flag, 4, ctx->stream));
  QX_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  if (bad != 0) return QX_STATUS_INVALID_ARGUMENT;  // non-finite weight, nothing written
  QX_CUDA_TRY(cudaMemcpy(packed, st.at(off_p), bytes, cudaMemcpyDeviceToHost));
  return QX_STATUS_OK;
}

// src/dispatch/qgemv.cpp:277-300
qx_status qx_qgemv_unpack(int format, const void* packed, long long n, long long k,
                          float* weights) {
  QX_TRY(validate_nk(format, n, k));
  size_t bytes = 0;
  if (packed_bytes(format, n, k, &bytes) != QX_STATUS_OK) return QX_STATUS_INVALID_SHAPE;
  if (packed == nullptr || weights == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  std::lock_guard<std::mutex> lock(ctx->mutex);
  Staging st{ctx};
  const size_t w_bytes = static_cast<size_t>(n) * k * sizeof(float);
  const size_t off_p = st.add(bytes), off_w = st.add(w_bytes);
  QX_TRY(ctx->ensure_staging(st.offset));
  QX_TRY(h2d(st.at(off_p), packed, bytes, ctx->stream));
  QX_TRY(launch_unpack(format, st.at(off_p), n * (k / kBlockK),
                       reinterpret_cast<float*>(st.at(off_w)), ctx->stream));
  QX_TRY(d2h(weights, st.at(off_w), w_bytes, ctx->stream));
  QX_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  return QX_STATUS_OK;
}

// kernels/quantization/qgemm_ref.cpp:141-164: shape -> null -> packed-size status.
qx_status qx_qgemm(int format, const void* packed_weights, const float* x, float* y,
                   long long m, long long n, long long k) {
  if (!valid_product2(m, k) || !valid_product2(m, n)) return QX_STATUS_INVALID_SHAPE;
  if (packed_weights == nullptr || x == nullptr || y == nullptr) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  size_t bytes = 0;
  QX_TRY(qx_qgemv_packed_size(format, n, k, &bytes));
  qx_weights* w = nullptr;
  QX_TRY(qx_weights_prepare(format, packed_weights, n, k, 0, n, &w));
  const qx_status status = qx_qgemm_prepacked(w, x, y, m, nullptr);
  qx_weights_destroy(w);
  return status;
}

// src/dispatch/qgemv.cpp:337-365: format/shape -> size -> null pointers.
qx_status qx_qgemv(int format, const void* packed, const float* x, float* y, long long n,
                   long long k) {
  QX_TRY(validate_nk(format, n, k));
  size_t bytes = 0;
  if (packed_bytes(format, n, k, &bytes) != QX_STATUS_OK) return QX_STATUS_INVALID_SHAPE;
  if (packed == nullptr || x == nullptr || y == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  return qx_qgemm(format, packed, x, y, 1, n, k);
}

qx_status qx_check_device_errors(void) {
  int device = -1;
  QX_CUDA_TRY(cudaGetDevice(&device));
  DeviceContext* ctx = existing_context(device);
  return ctx == nullptr ? QX_STATUS_OK : take_device_error(ctx);
}

// ---- qgemv_w8a8: block-quantised int8 activations (include/quixicore_cpu/qgemv_w8a8.h) ----

// src/dispatch/qgemv_w8a8.cpp:109-125
qx_status qx_qgemv_w8a8_packed_size(int format, long long n, long long k, long long* bytes) {
  size_t packed = 0;
  QX_TRY(qx_qgemv_packed_size(format, n, k, &packed));
  if (bytes == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  if (packed > static_cast<size_t>(std::numeric_limits<long long>::max())) return QX_STATUS_INVALID_SHAPE;
  *bytes = static_cast<long long>(packed);
  return QX_STATUS_OK;
}

// src/dispatch/qgemv_w8a8.cpp:127-130
qx_status qx_qgemv_w8a8_pack(int format, const float* weights, long long n, long long k,
                             void* packed) {
  return qx_qgemv_pack(format, weights, n, k, packed);
}

const char* qx_qgemv_w8a8_variant(int format) {
  if (format == QX_FORMAT_Q8_0 || format == QX_FORMAT_Q4_0) return "sm100a_tcgen05_i8_blocks";
  return "unsupported";
}

qx_status qx_qgemv_w8a8_prepacked_dev(const qx_weights* weights, const float* x_dev, float* y_dev,
                                      qx_workspace* workspace, void* stream) {
  if (weights == nullptr || x_dev == nullptr || y_dev == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  if (weights->segments != 1) return QX_STATUS_INVALID_ARGUMENT;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  GemvOptions options;
  options.int8_activations = true;
  return launch_qgemm_f32(weights, x_dev, y_dev, 1, weights->rows,
                          workspace != nullptr ? workspace : &ctx->workspace,
                          static_cast<cudaStream_t>(stream), nullptr, &options);
}

// src/dispatch/qgemv_w8a8.cpp:131-153: format/shape -> null pointers -> finite activations
qx_status qx_qgemv_w8a8(int format, const void* packed_weights, const float* x, float* y,
                        long long n, long long k) {
  QX_TRY(validate_nk(format, n, k));
  size_t bytes = 0;
  QX_TRY(packed_bytes(format, n, k, &bytes));
  if (packed_weights == nullptr || x == nullptr || y == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  if (!all_finite_host(x, k)) return QX_STATUS_INVALID_ARGUMENT;
  qx_weights* w = nullptr;
  QX_TRY(qx_weights_prepare(format, packed_weights, n, k, 0, n, &w));
  DeviceContext* ctx = nullptr;
  qx_status status = current_context(&ctx);
  if (status == QX_STATUS_OK) {
    std::lock_guard<std::mutex> lock(ctx->mutex);
    Staging st{ctx};
    const size_t off_x = st.add(k * sizeof(float)), off_y = st.add(n * sizeof(float));
    status = ctx->ensure_staging(st.offset);
    if (status == QX_STATUS_OK) status = h2d(st.at(off_x), x, k * sizeof(float), ctx->stream);
    if (status == QX_STATUS_OK) {
      status = qx_qgemv_w8a8_prepacked_dev(w, reinterpret_cast<const float*>(st.at(off_x)),
                                           reinterpret_cast<float*>(st.at(off_y)), nullptr, ctx->stream);
    }
    if (status == QX_STATUS_OK) status = d2h(y, st.at(off_y), n * sizeof(float), ctx->stream);
    if (status == QX_STATUS_OK) status = sync_and_check(ctx, ctx->stream);
  }
  qx_weights_destroy(w);
  return status;
}

// ---- fused decode projections (include/quixicore_cpu/qgemv.h:143-154) ----------------------

qx_status qx_qgemm_fused_dev(const qx_weights* weights, const float* x_dev, float* const* y_dev,
                             long long m, qx_workspace* workspace, void* stream) {
  if (weights == nullptr || x_dev == nullptr || y_dev == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  if (m <= 0 || m > kGemvMaxBatch) return QX_STATUS_INVALID_SHAPE;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  GemvOptions options;
  for (int s = 0; s < weights->segments; ++s) {
    if (y_dev[s] == nullptr) return QX_STATUS_INVALID_ARGUMENT;
    options.segment_y[s] = y_dev[s];
  }
  return launch_qgemm_f32(weights, x_dev, y_dev[0], m, weights->seg_rows[0],
                          workspace != nullptr ? workspace : &ctx->workspace,
                          static_cast<cudaStream_t>(stream), nullptr, &options);
}

qx_status qx_qgemv_up_gate_activation_dev(const qx_weights* up_gate, const float* x_dev,
                                          float* out_dev, float* scratch_dev, int gelu_tanh,
                                          qx_workspace* workspace, void* stream) {
  if (up_gate == nullptr || x_dev == nullptr || out_dev == nullptr || scratch_dev == nullptr) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  if (up_gate->segments != 2 || up_gate->seg_rows[0] != up_gate->seg_rows[1]) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  const long long n = up_gate->seg_rows[0];
  float* outputs[2] = {scratch_dev, scratch_dev + n};
  QX_TRY(qx_qgemm_fused_dev(up_gate, x_dev, outputs, 1, workspace, stream));
  return launch_gate_activation(outputs[0], outputs[1], out_dev, n, gelu_tanh != 0,
                                static_cast<cudaStream_t>(stream));
}

namespace {
// Shared host-pointer driver of the fused entry points: one fused handle from the parts,
// x in, one GEMV launch, (optional activation), the outputs back.
qx_status fused_host(int format, const void* const* parts, const long long* rows, int count,
                     long long k, const float* x, float* const* outputs, float* activation_out,
                     bool gelu_tanh) {
  qx_weights* w = nullptr;
  QX_TRY(qx_weights_prepare_fused(format, parts, rows, count, k, &w));
  DeviceContext* ctx = nullptr;
  qx_status status = current_context(&ctx);
  if (status == QX_STATUS_OK) {
    std::lock_guard<std::mutex> lock(ctx->mutex);
    Staging st{ctx};
    const size_t off_x = st.add(k * sizeof(float));
    size_t off_y[qx_weights::kMaxSegments] = {};
    for (int s = 0; s < count; ++s) off_y[s] = st.add(rows[s] * sizeof(float));
    const size_t off_out = st.add(rows[0] * sizeof(float));
    status = ctx->ensure_staging(st.offset);
    if (status == QX_STATUS_OK) status = h2d(st.at(off_x), x, k * sizeof(float), ctx->stream);
    float* y_dev[qx_weights::kMaxSegments] = {};
    for (int s = 0; s < count; ++s) y_dev[s] = reinterpret_cast<float*>(st.at(off_y[s]));
    if (status == QX_STATUS_OK) {
      status = qx_qgemm_fused_dev(w, reinterpret_cast<const float*>(st.at(off_x)), y_dev, 1, nullptr,
                                  ctx->stream);
    }
    if (status == QX_STATUS_OK && activation_out != nullptr) {
      status = launch_gate_activation(y_dev[0], y_dev[1], reinterpret_cast<float*>(st.at(off_out)),
                                      rows[0], gelu_tanh, ctx->stream);
      if (status == QX_STATUS_OK) {
        status = d2h(activation_out, st.at(off_out), rows[0] * sizeof(float), ctx->stream);
      }
    } else if (status == QX_STATUS_OK) {
      for (int s = 0; s < count && status == QX_STATUS_OK; ++s) {
        status = d2h(outputs[s], y_dev[s], rows[s] * sizeof(float), ctx->stream);
      }
    }
    if (status == QX_STATUS_OK) status = sync_and_check(ctx, ctx->stream);
  }
  qx_weights_destroy(w);
  return status;
}

// kernels/quantization/qgemv_fused_ref.cpp:170-182, 206-209: a format this path does not
// serve is kUnsupportedFormat, a shape that does not fit the format kInvalidShape
qx_status fused_layout_status(int format, long long n, long long k) {
  size_t block_bytes = 0;
  if (!format_info(format, &block_bytes)) return QX_STATUS_UNSUPPORTED_FORMAT;
  size_t bytes = 0;
  if (validate_nk(format, n, k) != QX_STATUS_OK || packed_bytes(format, n, k, &bytes) != QX_STATUS_OK) {
    return QX_STATUS_INVALID_SHAPE;
  }
  return QX_STATUS_OK;
}
}  // namespace

// kernels/quantization/qgemv_fused_ref.cpp:195-237
qx_status qx_qgemv_up_gate(int format, const void* packed_up, const void* packed_gate,
                           const float* x, float* up, float* gate, long long n, long long k) {
  if (!valid_product2(n, k)) return QX_STATUS_INVALID_SHAPE;
  if (packed_up == nullptr || packed_gate == nullptr || x == nullptr || up == nullptr ||
      gate == nullptr) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  QX_TRY(fused_layout_status(format, n, k));
  const void* parts[2] = {packed_up, packed_gate};
  const long long rows[2] = {n, n};
  float* outputs[2] = {up, gate};
  return fused_host(format, parts, rows, 2, k, x, outputs, nullptr, false);
}

// kernels/quantization/qgemv_fused_ref.cpp:239-286
qx_status qx_qgemv_up_gate_activation(int format, const void* packed_up, const void* packed_gate,
                                      const float* x, float* out, long long n, long long k,
                                      int gelu_tanh) {
  if (!valid_product2(n, k)) return QX_STATUS_INVALID_SHAPE;
  if (packed_up == nullptr || packed_gate == nullptr || x == nullptr || out == nullptr) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  QX_TRY(fused_layout_status(format, n, k));
  const void* parts[2] = {packed_up, packed_gate};
  const long long rows[2] = {n, n};
  float* outputs[2] = {nullptr, nullptr};
  return fused_host(format, parts, rows, 2, k, x, outputs, out, gelu_tanh != 0);
}

// kernels/quantization/qgemv_fused_ref.cpp:288-340
qx_status qx_qgemv_qkv(int format, const void* packed_q, const void* packed_k, const void* packed_v,
                       const float* x, float* q, float* k_out, float* v_out, long long query_dim,
                       long long kv_dim, long long input_dim) {
  if (!valid_product3(query_dim, kv_dim, input_dim)) return QX_STATUS_INVALID_SHAPE;
  if (kv_dim > (std::numeric_limits<long long>::max() - query_dim) / 2) return QX_STATUS_INVALID_SHAPE;
  if (packed_q == nullptr || packed_k == nullptr || packed_v == nullptr || x == nullptr ||
      q == nullptr || k_out == nullptr || v_out == nullptr) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  QX_TRY(fused_layout_status(format, query_dim, input_dim));
  if (fused_layout_status(format, kv_dim, input_dim) != QX_STATUS_OK) return QX_STATUS_INVALID_SHAPE;
  const void* parts[3] = {packed_q, packed_k, packed_v};
  const long long rows[3] = {query_dim, kv_dim, kv_dim};
  float* outputs[3] = {q, k_out, v_out};
  return fused_host(format, parts, rows, 3, input_dim, x, outputs, nullptr, false);
}

const char* qx_qgemv_variant(int format) {
  if (format == QX_FORMAT_Q8_0 || format == QX_FORMAT_Q4_0) return gemv_variant_name();
  return "unsupported";
}

// kernels/quantization/qgemm_panel.cpp:214-233
qx_status qx_qgemm_prepacked(const qx_weights* weights, const float* x, float* y, long long m,
                             qx_workspace* workspace) {
  if (weights == nullptr) return QX_STATUS_INVALID_ARGUMENT;  // !weights.ready()
  if (!valid_product3(m, weights->rows, weights->columns)) return QX_STATUS_INVALID_SHAPE;
  if (x == nullptr || y == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  std::lock_guard<std::mutex> lock(ctx->mutex);
  Staging st{ctx};
  const size_t x_bytes = static_cast<size_t>(m) * weights->columns * sizeof(float);
  const size_t y_bytes = static_cast<size_t>(m) * weights->rows * sizeof(float);
  const size_t off_x = st.add(x_bytes), off_y = st.add(y_bytes);
  QX_TRY(ctx->ensure_staging(st.offset));
  QX_TRY(stage_in(st.at(off_x), x, x_bytes, ctx->stream));
  // Results go straight to the caller's buffer when the GPU can address it (pinned or
  // registered host memory): the kernel's row finishers write it over PCIe and the copy
  // back is saved. Pageable memory takes the staged copy.
  float* y_target = reinterpret_cast<float*>(st.at(off_y));
  bool direct = false;
  cudaPointerAttributes attributes{};
  if (cudaPointerGetAttributes(&attributes, y) == cudaSuccess &&
      attributes.type == cudaMemoryTypeHost && attributes.devicePointer != nullptr) {
    y_target = static_cast<float*>(attributes.devicePointer);
    direct = true;
  } else {
    (void)cudaGetLastError();  // unregistered host memory is not an error here
  }
  QX_TRY(launch_qgemm_f32(weights, reinterpret_cast<const float*>(st.at(off_x)), y_target, m,
                          weights->rows, workspace != nullptr ? workspace : &ctx->workspace,
                          ctx->stream));
  if (!direct) QX_TRY(d2h(y, st.at(off_y), y_bytes, ctx->stream));
  return sync_and_check(ctx, ctx->stream);
}

qx_status qx_qgemm_prepacked_dev(const qx_weights* weights, const float* x_dev, float* y_dev,
                                 long long m, long long ldy, qx_workspace* workspace,
                                 void* stream) {
  if (weights == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  if (!valid_product3(m, weights->rows, weights->columns) || ldy < weights->rows) {
    return QX_STATUS_INVALID_SHAPE;
  }
  if (x_dev == nullptr || y_dev == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  return launch_qgemm_f32(weights, x_dev, y_dev, m, ldy,
                          workspace != nullptr ? workspace : &ctx->workspace,
                          static_cast<cudaStream_t>(stream));
}

qx_status qx_qgemm_prepacked_bf16_dev(const qx_weights* weights, const uint16_t* x_bf16_dev,
                                      float* y_dev, long long m, long long ldy,
                                      qx_workspace* workspace, void* stream) {
  if (weights == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  if (!valid_product3(m, weights->rows, weights->columns) || ldy < weights->rows) {
    return QX_STATUS_INVALID_SHAPE;
  }
  if (x_bf16_dev == nullptr || y_dev == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  return launch_q4_gemm_bf16(weights, x_bf16_dev, y_dev, m, ldy,
                             workspace != nullptr ? workspace : &ctx->workspace,
                             static_cast<cudaStream_t>(stream));
}

// src/dispatch/int8_gemm.cpp:67-94: shape -> null -> finite scales.
qx_status qx_int8_gemm(const int8_t* weights, const int8_t* x, const float* weight_scale,
                       const float* activation_scale, const int32_t* weight_row_sum,
                       const int* activation_zero_point, float* y, long long m, long long n,
                       long long k, int asymmetric) {
  if (!valid_product3(m, n, k)) return QX_STATUS_INVALID_SHAPE;
  if (weights == nullptr || x == nullptr || weight_scale == nullptr ||
      activation_scale == nullptr || y == nullptr ||
      (asymmetric && (weight_row_sum == nullptr || activation_zero_point == nullptr))) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  if (!all_finite_host(weight_scale, n) || !all_finite_host(activation_scale, m)) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  std::lock_guard<std::mutex> lock(ctx->mutex);
  Staging st{ctx};
  const size_t w_bytes = static_cast<size_t>(n) * k, x_bytes = static_cast<size_t>(m) * k;
  const size_t y_bytes = static_cast<size_t>(m) * n * sizeof(float);
  const size_t off_w = st.add(w_bytes), off_x = st.add(x_bytes), off_ws = st.add(n * 4),
               off_as = st.add(m * 4), off_rs = st.add(n * 4), off_zp = st.add(m * 4),
               off_y = st.add(y_bytes);
  QX_TRY(ctx->ensure_staging(st.offset));
  cudaStream_t s = ctx->stream;
  QX_TRY(h2d(st.at(off_w), weights, w_bytes, s));
  QX_TRY(h2d(st.at(off_x), x, x_bytes, s));
  QX_TRY(h2d(st.at(off_ws), weight_scale, n * 4, s));
  QX_TRY(h2d(st.at(off_as), activation_scale, m * 4, s));
  if (asymmetric) {
    QX_TRY(h2d(st.at(off_rs), weight_row_sum, n * 4, s));
    QX_TRY(h2d(st.at(off_zp), activation_zero_point, m * 4, s));
  }
  Int8GemmArgs a{};
  a.w = reinterpret_cast<const int8_t*>(st.at(off_w));
  a.x = reinterpret_cast<const int8_t*>(st.at(off_x));
  a.ws = reinterpret_cast<const float*>(st.at(off_ws));
  a.as = reinterpret_cast<const float*>(st.at(off_as));
  a.row_sum = asymmetric ? reinterpret_cast<const int32_t*>(st.at(off_rs)) : nullptr;
  a.zp = asymmetric ? reinterpret_cast<const int*>(st.at(off_zp)) : nullptr;
  a.y = reinterpret_cast<float*>(st.at(off_y));
  a.acc = nullptr;
  a.m = m;
  a.n = n;
  a.k = k;
  a.ldy = n;
  a.asymmetric = asymmetric != 0;
  QX_TRY(launch_int8_gemm(a, s));
  QX_TRY(d2h(y, st.at(off_y), y_bytes, s));
  return sync_and_check(ctx, s);
}

// kernels/quantization/qgemm_extended_ref.cpp:142-147
qx_status qx_qgemm_w8a8(const int8_t* weights, const int8_t* x, const float* weight_scale,
                        const float* activation_scale, float* y, long long m, long long n,
                        long long k) {
  return qx_int8_gemm(weights, x, weight_scale, activation_scale, nullptr, nullptr, y, m, n, k, 0);
}

// kernels/quantization/qgemm_extended_ref.cpp:149-156
qx_status qx_qgemm_w8a8_azp(const int8_t* weights, const int8_t* x, const float* weight_scale,
                            const float* activation_scale, const int32_t* weight_row_sum,
                            const int* activation_zero_point, float* y, long long m,
                            long long n, long long k) {
  return qx_int8_gemm(weights, x, weight_scale, activation_scale, weight_row_sum,
                      activation_zero_point, y, m, n, k, 1);
}

const char* qx_int8_gemm_variant(void) { return int8_gemm_variant_name(); }

qx_status qx_int8_gemm_dev(const int8_t* weights_dev, const int8_t* x_dev,
                           const float* weight_scale_dev, const float* activation_scale_dev,
                           const int32_t* weight_row_sum_dev, const int* activation_zero_point_dev,
                           float* y_dev, int32_t* acc_i32_dev, long long m, long long n,
                           long long k, long long ldy, int asymmetric, int check_scales,
                           void* stream) {
  if (!valid_product3(m, n, k) || ldy < n) return QX_STATUS_INVALID_SHAPE;
  if (weights_dev == nullptr || x_dev == nullptr || weight_scale_dev == nullptr ||
      activation_scale_dev == nullptr || y_dev == nullptr ||
      (asymmetric && (weight_row_sum_dev == nullptr || activation_zero_point_dev == nullptr))) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (check_scales) {
    QX_CUDA_TRY(cudaMemsetAsync(ctx->flag, 0, 4, s));
    QX_TRY(launch_check_finite(weight_scale_dev, n, ctx->flag, s));
    QX_TRY(launch_check_finite(activation_scale_dev, m, ctx->flag, s));
    int bad = 0;
    QX_CUDA_TRY(cudaMemcpyAsync(&bad, ctx->flag, 4, cudaMemcpyDeviceToHost, s));
    QX_CUDA_TRY(cudaStreamSynchronize(s));
    if (bad != 0) return QX_STATUS_INVALID_ARGUMENT;
  }
  Int8GemmArgs a{weights_dev, x_dev, weight_scale_dev, activation_scale_dev, weight_row_sum_dev,
                 activation_zero_point_dev, y_dev, acc_i32_dev, m, n, k, ldy, asymmetric != 0};
  return launch_int8_gemm(a, s);
}

// src/dispatch/w8a32_gemm.cpp:61-73
qx_status qx_qgemm_w8a32(const int8_t* weights, const float* weight_scale, const float* x,
                         float* y, long long m, long long n, long long k) {
  if (!valid_product3(m, n, k)) return QX_STATUS_INVALID_SHAPE;
  if (weights == nullptr || weight_scale == nullptr || x == nullptr || y == nullptr) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  if (!all_finite_host(weight_scale, n)) return QX_STATUS_INVALID_ARGUMENT;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  std::lock_guard<std::mutex> lock(ctx->mutex);
  Staging st{ctx};
  const size_t w_bytes = static_cast<size_t>(n) * k;
  const size_t x_bytes = static_cast<size_t>(m) * k * sizeof(float);
  const size_t y_bytes = static_cast<size_t>(m) * n * sizeof(float);
  const size_t off_w = st.add(w_bytes), off_ws = st.add(n * 4), off_x = st.add(x_bytes),
               off_y = st.add(y_bytes);
  QX_TRY(ctx->ensure_staging(st.offset));
  cudaStream_t s = ctx->stream;
  QX_TRY(h2d(st.at(off_w), weights, w_bytes, s));
  QX_TRY(h2d(st.at(off_ws), weight_scale, n * 4, s));
  QX_TRY(h2d(st.at(off_x), x, x_bytes, s));
  QX_TRY(launch_w8a32(reinterpret_cast<const int8_t*>(st.at(off_w)),
                      reinterpret_cast<const float*>(st.at(off_ws)),
                      reinterpret_cast<const float*>(st.at(off_x)),
                      reinterpret_cast<float*>(st.at(off_y)), m, n, k, n, &ctx->workspace, s));
  QX_TRY(d2h(y, st.at(off_y), y_bytes, s));
  return sync_and_check(ctx, s);
}

const char* qx_qgemm_w8a32_variant(void) { return "sm100a_stream_fma+tcgen05_digit_planes"; }

qx_status qx_qgemm_w8a32_dev(const int8_t* weights_dev, const float* weight_scale_dev,
                             const float* x_dev, float* y_dev, long long m, long long n,
                             long long k, long long ldy, int check_scales,
                             qx_workspace* workspace, void* stream) {
  if (!valid_product3(m, n, k) || ldy < n) return QX_STATUS_INVALID_SHAPE;
  if (weights_dev == nullptr || weight_scale_dev == nullptr || x_dev == nullptr ||
      y_dev == nullptr) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (check_scales) {
    QX_CUDA_TRY(cudaMemsetAsync(ctx->flag, 0, 4, s));
    QX_TRY(launch_check_finite(weight_scale_dev, n, ctx->flag, s));
    int bad = 0;
    QX_CUDA_TRY(cudaMemcpyAsync(&bad, ctx->flag, 4, cudaMemcpyDeviceToHost, s));
    QX_CUDA_TRY(cudaStreamSynchronize(s));
    if (bad != 0) return QX_STATUS_INVALID_ARGUMENT;
  }
  return launch_w8a32(weights_dev, weight_scale_dev, x_dev, y_dev, m, n, k, ldy,
                      workspace != nullptr ? workspace : &ctx->workspace, s);
}

}  // extern "C"
