// Prefill GEMM over prepared q4_0 / q8_0 weights with bf16 activations:
// Y[m, rows] = bf16_to_f32(X)[m, k] . dequant(W)^T. Counterpart of qgemm_prepacked for
// m >= 64 (kernels/quantization/qgemm_panel.cpp:242-287) with the bf16 -> f32 input
// conversion of float_storage (kernels/utils/float_storage_ref.cpp:195-200).

#include "qx_gemv.cuh"
#include "qx_gemv_tc.cuh"
#include "qx_weights.cuh"

namespace qx {
namespace {

__global__ void __launch_bounds__(256) bf16_to_f32_kernel(const uint16_t* __restrict__ in,
                                                          float* __restrict__ out,
                                                          long long count) {
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < count; i += gridDim.x * 256LL) {
    out[i] = __uint_as_float(static_cast<uint32_t>(in[i]) << 16);
  }
}

}  // namespace

qx_status launch_q4_gemm_bf16(const qx_weights* w, const uint16_t* x_bf16_dev, float* y_dev,
                              long long m, long long ldy, qx_workspace* ws, cudaStream_t stream) {
  // Exact path: widen the activations to f32 (bf16 -> f32 is exact) and reuse the f32
  // batched kernel; its scratch sits at the start of the workspace and the widened copy
  // behind it.
  const long long count = m * w->columns;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  GemvScratch scratch;
  QX_TRY(gemv_scratch_layout(w, static_cast<int>(m < kGemvMaxBatch ? m : kGemvMaxBatch),
                             ctx->prop.multiProcessorCount, &scratch));
  const size_t table_bytes = align_up(scratch.total_bytes, 256);
  QX_TRY(ws->reserve(table_bytes + static_cast<size_t>(count) * sizeof(float)));
  float* x_f32 = reinterpret_cast<float*>(static_cast<uint8_t*>(ws->base) + table_bytes);
  const unsigned grid = static_cast<unsigned>(min((count + 255) / 256, 4096LL));
  bf16_to_f32_kernel<<<grid, 256, 0, stream>>>(x_bf16_dev, x_f32, count);
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  return launch_qgemm_f32(w, x_f32, y_dev, m, ldy, ws, stream);
}

}  // namespace qx
