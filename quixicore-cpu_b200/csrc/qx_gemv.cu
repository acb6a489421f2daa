// Decode GEMV / small-batch qgemm over prepared q8_0 and q4_0 weights: activation digit
// quantizer, the CUDA-core (dp4a) kernel and the dispatch between it and the
// tensor-core kernel of qx_gemv_tc.cu.
//
// Replaces q8_0_gemv_ref / q4_0_gemv_ref / q4_rows of the reference
// (kernels/quantization/qgemv_ref.cpp:62-92, qgemv_w8a8_ref.cpp:95-118,
// qgemv_gguf_avx2.cpp:295-318) and the per-row loop of qgemm
// (kernels/quantization/qgemm_ref.cpp:156-162).

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "qx_gemv.cuh"
#include "qx_gemv_tc.cuh"
#include "qx_weights.cuh"

namespace qx {
namespace {

// Balanced base-256 digit `d` (0..3) of t: t = sum_d 256^d * digit_d, digits 0..2 in
// [-128, 127].
__device__ __forceinline__ int balanced_digit(int t, int d) {
  int p = ((t + 128) & 255) - 128;
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    if (i < d) {
      t = (t - p) >> 8;
      p = i == 2 ? t : ((t + 128) & 255) - 128;
    }
  }
  return p;
}

// Envelope of one 32-element block: *scale_up = 2^(22-e), *scale = 2^(e-22) with 2^e
// above the largest magnitude; NaN scale (and *finite false) for a non-finite element.
__device__ __forceinline__ void block_envelope(const float (&v)[32], float* scale_up, float* scale,
                                               bool* finite) {
  // max of |bits|: orders finite < inf < NaN, so non-finite inputs are detected
  uint32_t amax_bits = 0;
#pragma unroll
  for (int i = 0; i < 32; ++i) amax_bits = max(amax_bits, __float_as_uint(v[i]) & 0x7FFFFFFFu);
  const uint32_t eb_raw = amax_bits >> 23;
  *finite = eb_raw != 255u;
  const uint32_t eb = max(eb_raw, 30u);                  // envelope 2^(eb-126) > amax
  *scale_up = __uint_as_float((275u - eb) << 23);        // 2^(22 - e)
  *scale = *finite ? __uint_as_float((eb - 21u) << 23)   // 2^(e - 22)
                   : __uint_as_float(0x7FC00000u);       // NaN/inf in -> NaN out
}

// One block of activations (16-byte loads when the row allows them).
__device__ __forceinline__ void load_block(const float* src, int x_vector, float (&v)[32]) {
  if (x_vector != 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 f = __ldg(reinterpret_cast<const float4*>(src) + i);
      v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __ldg(src + i);
  }
}

// ------------------------------------------------------------------------------------
// Activation digits: x[m][k] f32 -> one image per K-slab (layout: qx_gemv.cuh). The first
// `chunk_threads` threads write one 16-byte chunk of a digit row each (zeros outside the
// block class of the row, for padded rows and for the K padding); the remaining threads
// write one XConst each.
// ------------------------------------------------------------------------------------
template <int FMT>
__global__ void __launch_bounds__(256) quantize_x_kernel(const float* __restrict__ x,
                                                         uint8_t* __restrict__ ximg, int m, int mp,
                                                         int k, int nb, int x_vector,
                                                         long long chunk_threads,
                                                         long long total_threads) {
  // let the GEMV kernel behind this one start its set-up and weight pipeline right away
  asm volatile("griddepcontrol.launch_dependents;");
  // This kernel is launched programmatically, so it may start while the kernel in front of
  // it still runs. That kernel may be the producer of x (the previous layer's GEMV, the
  // wait kernel of a sharded step) and may still read the images (the previous GEMV):
  // nothing is read or written before it has finished.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const long long t = blockIdx.x * 256LL + threadIdx.x;
  if (t >= total_threads) return;
  const int ncols = digit_columns(FMT, mp);
  const int group = group_blocks(FMT, mp);
  const size_t image_bytes = ximage_bytes(FMT, mp);
  float v[32];
  if (t < chunk_threads) {
    const int c16 = static_cast<int>(t & 15);
    const int n = static_cast<int>((t >> 4) % ncols);
    const long long slab = (t >> 4) / ncols;
    const int which = c16 >> 3, cc = c16 & 7;
    const int j = FMT == QX_FORMAT_Q8_0 ? 4 * which + (cc >> 1) : cc;
    const int half = cc & 1;
    const int klass = n / (4 * mp), row = (n >> 2) % mp, d = n & 3;
    const long long b = slab * kSlabBlocks + j;
    const bool digit_used = FMT == QX_FORMAT_Q8_0 ? d < 3 : true;
    const bool active = (j % group) == klass && row < m && b < nb && digit_used;
    uint4 out = make_uint4(0u, 0u, 0u, 0u);
    if (active) {
      load_block(x + static_cast<long long>(row) * k + b * 32, x_vector, v);
      float scale_up, scale;
      bool finite;
      block_envelope(v, &scale_up, &scale, &finite);
      uint32_t word[4] = {0u, 0u, 0u, 0u};
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        int value = 0;
        if (finite) {
          if (FMT == QX_FORMAT_Q8_0) {
            value = __float2int_rn((half != 0 ? v[16 + i] : v[i]) * scale_up);  // |t| <= 2^22
          } else {
            const int lo = __float2int_rn(v[i] * scale_up);
            value = which == 0 ? 16 * lo : __float2int_rn(v[16 + i] * scale_up) - 16 * lo;
          }
        }
        word[i >> 2] |= static_cast<uint32_t>(balanced_digit(value, d) & 255) << (8 * (i & 3));
      }
      out = make_uint4(word[0], word[1], word[2], word[3]);
    }
    *reinterpret_cast<uint4*>(ximg + slab * image_bytes + ximage_chunk_offset(ncols, which, n, cc)) =
        out;
  } else {
    const long long u = t - chunk_threads;
    const int row = static_cast<int>(u % mp);
    const int j = static_cast<int>((u / mp) % kSlabBlocks);
    const long long slab = u / (static_cast<long long>(mp) * kSlabBlocks);
    const long long b = slab * kSlabBlocks + j;
    XConst c;
    c.scale = 0.0f;
    c.k_lo = c.k_hi = c.pad = 0;
    if (row < m && b < nb) {
      load_block(x + static_cast<long long>(row) * k + b * 32, x_vector, v);
      float scale_up;
      bool finite;
      block_envelope(v, &scale_up, &c.scale, &finite);
      if (FMT == QX_FORMAT_Q4_0 && finite) {
        int sum = 0;  // |sum| <= 32 * 2^22
#pragma unroll
        for (int i = 0; i < 32; ++i) sum += __float2int_rn(v[i] * scale_up);
        q4_offset_constants(sum, &c.k_lo, &c.k_hi);
      }
      if (FMT == QX_FORMAT_Q4_0) c.scale *= 0.0625f;  // the digit sums carry a factor 16
    }
    *reinterpret_cast<XConst*>(ximg + slab * image_bytes + ximage_const_offset(ncols, mp, j, row)) = c;
  }
}

__device__ __forceinline__ float warp_tree_sum(float v) {
#pragma unroll
  for (int h = 16; h >= 1; h >>= 1) v += __shfl_xor_sync(0xffffffffu, v, h);
  return v;
}

// ------------------------------------------------------------------------------------
// CUDA-core kernel: one warp per (weight row, activation row); lanes stride over blocks.
// Same digit arithmetic as the tensor-core kernel, block by block with dp4a. Reduction:
// per group of 32 consecutive blocks a fixed xor-butterfly (16, 8, 4, 2, 1), groups added
// in ascending order, so the result does not depend on the launch shape.
// ------------------------------------------------------------------------------------
template <int FMT>
__global__ void __launch_bounds__(256) gemv_dp4a_kernel(
    const uint8_t* __restrict__ panel, const uint8_t* __restrict__ ximg, int mp,
    float* __restrict__ y, long long n, int nb, long long slabs, long long ldy) {
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * 8LL + (threadIdx.x >> 5);
  if (row >= n) return;
  const int m = blockIdx.y;
  const int ncols = digit_columns(FMT, mp);
  const long long tile = row / kTileRows;
  const int r = static_cast<int>(row % kTileRows);
  float acc = 0.0f;
  for (int base = 0; base < nb; base += 32) {
    const int b = base + lane;
    float v = 0.0f;
    if (b < nb) {
      const int j = b % kSlabBlocks;
      const uint8_t* span = panel + (tile * slabs + b / kSlabBlocks) * slab_span_bytes(FMT);
      const uint8_t* image = ximg + static_cast<long long>(b / kSlabBlocks) * ximage_bytes(FMT, mp);
      const XConst c = *reinterpret_cast<const XConst*>(image + ximage_const_offset(ncols, mp, j, m));
      int s[4] = {0, 0, 0, 0};
      if (FMT == QX_FORMAT_Q8_0) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const uint4 w = __ldg(reinterpret_cast<const uint4*>(span + panel_code_offset_q8(r, j, half)));
#pragma unroll
          for (int d = 0; d < 3; ++d) {
            const uint4 g = __ldg(reinterpret_cast<const uint4*>(
                image + ximage_chunk_offset(ncols, j >> 2, digit_row(FMT, mp, j, m, d),
                                            2 * (j & 3) + half)));
            s[d] = dp4a_ss(w.x, g.x, s[d]);
            s[d] = dp4a_ss(w.y, g.y, s[d]);
            s[d] = dp4a_ss(w.z, g.z, s[d]);
            s[d] = dp4a_ss(w.w, g.w, s[d]);
          }
        }
      } else {
        // raw bytes against the digits of 16*t_i, masked bytes against the digits of z_i
        const uint4 w = __ldg(reinterpret_cast<const uint4*>(span + panel_code_offset_q4(r, j)));
        const uint4 h = make_uint4(w.x & 0xF0F0F0F0u, w.y & 0xF0F0F0F0u, w.z & 0xF0F0F0F0u,
                                   w.w & 0xF0F0F0F0u);
#pragma unroll
        for (int d = 0; d < 4; ++d) {
          const int nrow = digit_row(FMT, mp, j, m, d);
          const uint4 g = __ldg(reinterpret_cast<const uint4*>(image + ximage_chunk_offset(ncols, 0, nrow, j)));
          s[d] = dp4a_us(w.x, g.x, s[d]);
          s[d] = dp4a_us(w.y, g.y, s[d]);
          s[d] = dp4a_us(w.z, g.z, s[d]);
          s[d] = dp4a_us(w.w, g.w, s[d]);
          const uint4 z = __ldg(reinterpret_cast<const uint4*>(image + ximage_chunk_offset(ncols, 1, nrow, j)));
          s[d] = dp4a_us(h.x, z.x, s[d]);
          s[d] = dp4a_us(h.y, z.y, s[d]);
          s[d] = dp4a_us(h.z, z.z, s[d]);
          s[d] = dp4a_us(h.w, z.w, s[d]);
        }
      }
      const float d = half_bits_to_float(
          *reinterpret_cast<const unsigned short*>(span + panel_scale_offset(FMT, r, j)));
      const float sum = FMT == QX_FORMAT_Q8_0 ? block_sum(s[0], s[1], s[2])
                                              : block_sum(s[0], s[1], s[2], s[3], c.k_lo, c.k_hi);
      v = __fmul_rn(sum, __fmul_rn(d, c.scale));
    }
    acc += warp_tree_sum(v);
  }
  if (lane == 0) y[m * ldy + row] = acc;
}

// out[i] = activate(gate[i]) * up[i], the formulas of
// kernels/quantization/qgemv_fused_ref.cpp:184-192 (tanh-GELU or SiLU) in f32.
__global__ void __launch_bounds__(256) gate_activation_kernel(const float* __restrict__ up,
                                                              const float* __restrict__ gate,
                                                              float* __restrict__ out, long long n,
                                                              int gelu_tanh) {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");  // up / gate come from the GEMV in front
  const long long i = blockIdx.x * 256LL + threadIdx.x;
  if (i >= n) return;
  const float g = gate[i];
  float a;
  if (gelu_tanh != 0) {
    const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    a = 0.5f * g * (1.0f + tanhf(inner));
  } else {
    a = g / (1.0f + expf(-g));
  }
  out[i] = a * up[i];
}

bool force_dp4a() {
  static const bool forced = []() {
    const char* v = std::getenv("QX_B200_GEMV_VARIANT");
    return v != nullptr && std::strcmp(v, "dp4a") == 0;
  }();
  return forced;
}

// Enqueues the quantizer for `m` activation rows (x_dev [m][columns]) into `ximg`.
// `programmatic`: launched so that it may start before the kernel ahead of it in the stream
// has finished (it waits for that kernel itself before it writes).
qx_status launch_quantizer(const qx_weights* w, const float* x_dev, uint8_t* ximg, int m,
                           bool programmatic, cudaStream_t stream) {
  const int mp = padded_batch(m);
  const long long chunk_threads =
      static_cast<long long>(w->slabs) * digit_columns(w->format, mp) * 16;
  const long long total_threads = chunk_threads + static_cast<long long>(w->slabs) * kSlabBlocks * mp;
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(static_cast<unsigned>((total_threads + 255) / 256));
  config.blockDim = dim3(256);
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = programmatic ? 1 : 0;
  const int k = static_cast<int>(w->columns), nb = static_cast<int>(w->blocks_per_row);
  const int x_vector = reinterpret_cast<uintptr_t>(x_dev) % 16 == 0 ? 1 : 0;
  if (w->format == QX_FORMAT_Q8_0) {
    QX_CUDA_TRY(cudaLaunchKernelEx(&config, quantize_x_kernel<QX_FORMAT_Q8_0>, x_dev, ximg, m, mp, k,
                                   nb, x_vector, chunk_threads, total_threads));
  } else {
    QX_CUDA_TRY(cudaLaunchKernelEx(&config, quantize_x_kernel<QX_FORMAT_Q4_0>, x_dev, ximg, m, mp, k,
                                   nb, x_vector, chunk_threads, total_threads));
  }
  count_launch();
  return QX_STATUS_OK;
}

}  // namespace

qx_status launch_gate_activation(const float* up, const float* gate, float* out, long long n,
                                 bool gelu_tanh, cudaStream_t stream) {
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(static_cast<unsigned>((n + 255) / 256));
  config.blockDim = dim3(256);
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  QX_CUDA_TRY(cudaLaunchKernelEx(&config, gate_activation_kernel, up, gate, out, n, gelu_tanh ? 1 : 0));
  count_launch();
  return QX_STATUS_OK;
}

// digits: activations as base-256 digits, exact int8 sums; tcgen05: the persistent tensor-core
// kernel; mma: the streaming single-row kernel with warp-level MMAs (small matrices)
const char* gemv_variant_name() {
  if (force_dp4a()) return "sm100a_dp4a";
  return gemv_decode_enabled() ? "sm100a_digits_tcgen05+mma" : "sm100a_digits_tcgen05";
}

// Workspace layout of one GEMV call: [row counters | activation slab images | per-unit
// partial sums]; sizes depend only on (m, k, rows).
qx_status launch_qgemm_f32(const qx_weights* w, const float* x_dev, float* y_dev,
                           long long m, long long ldy, qx_workspace* ws,
                           cudaStream_t stream, const GemvPush* push, const GemvOptions* options) {
  if ((w->segments > 1 || (options != nullptr && options->int8_activations)) &&
      (force_dp4a() || m > kGemvMaxBatch)) {
    set_last_error_text("qgemm: fused handles and int8 activations take at most 32 activation rows "
                        "(tensor-core kernel)");
    return QX_STATUS_INVALID_SHAPE;
  }
  if (push != nullptr && (m > kGemvMaxBatch || force_dp4a())) {
    set_last_error_text("qgemm: pushing launches take at most 32 activation rows (tensor-core kernel)");
    return QX_STATUS_INVALID_SHAPE;
  }
  if (w->columns > (1LL << 24) || w->rows > (1LL << 31) - 256) {
    set_last_error_text("qgemm: shape beyond the GEMV kernels' 32-bit tile indices");
    return QX_STATUS_INVALID_SHAPE;
  }
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  for (long long m0 = 0; m0 < m; m0 += kGemvMaxBatch) {
    const int mc = static_cast<int>(m - m0 < kGemvMaxBatch ? m - m0 : kGemvMaxBatch);
    GemvScratch scratch;
    QX_TRY(gemv_scratch_layout(w, mc, ctx->prop.multiProcessorCount, &scratch));
    QX_TRY(ws->reserve(scratch.total_bytes));
    uint8_t* base = static_cast<uint8_t*>(ws->base);
    uint8_t* ximg = base + scratch.ximg_offset;
    const float* x = x_dev + m0 * w->columns;
    if (force_dp4a() || !gemv_tc_quantizes_in_kernel(mc)) {
      QX_TRY(launch_quantizer(w, x, ximg, mc, true, stream));
    }
    float* y = y_dev + m0 * ldy;
    if (!force_dp4a()) {
      QX_TRY(launch_gemv_tc(w, x, ximg, y, mc, ldy, base, scratch, stream, push, options));
    } else {
      const dim3 grid(static_cast<unsigned>((w->rows + 7) / 8), static_cast<unsigned>(mc));
      const int mp = padded_batch(mc), nb = static_cast<int>(w->blocks_per_row);
      if (w->format == QX_FORMAT_Q8_0) {
        gemv_dp4a_kernel<QX_FORMAT_Q8_0><<<grid, 256, 0, stream>>>(w->panel, ximg, mp, y, w->rows, nb,
                                                                   w->slabs, ldy);
      } else {
        gemv_dp4a_kernel<QX_FORMAT_Q4_0><<<grid, 256, 0, stream>>>(w->panel, ximg, mp, y, w->rows, nb,
                                                                   w->slabs, ldy);
      }
      count_launch();
    }
    QX_CUDA_TRY(cudaGetLastError());
  }
  return QX_STATUS_OK;
}

}  // namespace qx

// ------------------------------------------------------------------------------------
// Decode GEMV for callers that must not allocate device memory.
//
// Some hosts of this library run the decode step where cudaMalloc is off limits: inside a
// serving loop whose memory is handed out once at start-up by the application's own pool,
// inside a process whose GPU allocations are metered or capped by an external broker, or
// in a latency-critical thread where the implicit device synchronisation of cudaMalloc /
// cudaFree is not acceptable. The regular entry points grow a workspace on demand and so
// may allocate; this one never does. Its scratch memory (activation slab images, per-unit
// partial sums and per-row counters) lives in the array below,
// which every GPU that loads the library holds from module load until the process exits.
// ------------------------------------------------------------------------------------
namespace qx {
namespace {

constexpr size_t kNoAllocScratchBytes = 6u << 20;  // 6 MiB per GPU
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

struct NoAllocDevice {
  uint8_t* scratch = nullptr;  // device address of g_noalloc_scratch on this GPU
  int sm_count = 0;
  bool ready = false;
};
NoAllocDevice g_noalloc_devices[64];
std::mutex g_noalloc_mutex;

// Once per device, with that device current: resolve the array's device address. The name
// g_noalloc_scratch is only a host-side handle in host code; kernels need this address.
qx_status noalloc_device(NoAllocDevice** out) {
  int device = -1;
  QX_CUDA_TRY(cudaGetDevice(&device));
  if (device < 0 || device >= 64) {
    set_last_error_text("device ordinal out of range");
    return QX_STATUS_DEVICE_ERROR;
  }
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  NoAllocDevice& entry = g_noalloc_devices[device];
  if (!entry.ready) {
    int major = 0, sms = 0;
    QX_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
    QX_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    if (major != 10) {
      set_last_error_text("device is not compute capability 10.x (B200); kernels are sm_100a only");
      return QX_STATUS_DEVICE_ERROR;
    }
    void* address = nullptr;
    QX_CUDA_TRY(cudaGetSymbolAddress(&address, g_noalloc_scratch));
    entry.scratch = static_cast<uint8_t*>(address);
    entry.sm_count = sms;
    entry.ready = true;
  }
  *out = &entry;
  return QX_STATUS_OK;
}

}  // namespace
}  // namespace qx

extern "C" qx_status qx_qgemv_prepacked_noalloc_dev(const qx_weights* weights, const float* x_dev,
                                                     float* y_dev, void* stream) {
  using namespace qx;
  if (weights == nullptr || x_dev == nullptr || y_dev == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  NoAllocDevice* dev = nullptr;
  QX_TRY(noalloc_device(&dev));
  int device = -1;
  QX_CUDA_TRY(cudaGetDevice(&device));
  if (weights->device != device) {
    set_last_error_text("qgemv (no-alloc): the weights were prepared on another device");
    return QX_STATUS_INVALID_ARGUMENT;
  }
  if (weights->columns > (1LL << 24)) return QX_STATUS_INVALID_SHAPE;
  GemvScratch scratch;
  QX_TRY(gemv_scratch_layout(weights, 1, dev->sm_count, &scratch));
  if (align_up(scratch.total_bytes, 256) > kNoAllocScratchBytes) {
    set_last_error_text(
        "qgemv (no-alloc): this weight matrix needs more scratch than the 6 MiB static array "
        "(limit is about rows * min(16, columns/256) * 4 B <= 5 MiB; use qx_qgemm_prepacked_dev)");
    return QX_STATUS_INVALID_SHAPE;
  }
  // A bounded wait that gives up inside the kernel reports through the same word as every
  // other entry point: the device's context was created when the weights were prepared, so
  // looking it up allocates nothing. qx_check_device_errors() or the next host-pointer call
  // on this device returns QX_STATUS_DEVICE_ERROR with the role code.
  DeviceContext* ctx = existing_context(device);
  if (ctx == nullptr) {
    set_last_error_text("qgemv (no-alloc): no context on this device (prepare the weights here first)");
    return QX_STATUS_DEVICE_ERROR;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* base = dev->scratch;
  // The array keeps whatever the previous call left. The kernel expects the row counters it
  // uses to be zero; everything else is fully rewritten before it is read.
  QX_CUDA_TRY(cudaMemsetAsync(base, 0, static_cast<size_t>(weights->tiles) * kTileRows * sizeof(int), s));

  uint8_t* ximg = base + scratch.ximg_offset;
  return launch_gemv_tc_at(weights, x_dev, ximg, y_dev, 1, weights->rows, base, scratch,
                           ctx->error_dev, s);
}
