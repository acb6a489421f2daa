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

// ------------------------------------------------------------------------------------
// activation digits: x[m][k] f32 -> one image per K-slab (see ximage_bytes): digit rows
// (row 4*m+d = digit d of activation row m, d < 3; row 4*m+3, unused rows and the K padding
// are written as zeros) followed by the per-block constants.
// One group of 8 threads per (virtual row, block); virtual rows beyond m only zero-fill.
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) quantize_x_kernel(const float* __restrict__ x,
                                                         uint8_t* __restrict__ ximg, int m, int k,
                                                         int nb, int nbpad, int ncols,
                                                         long long total_groups) {
  // let the GEMV kernel behind this one start its set-up and weight pipeline right away
  asm volatile("griddepcontrol.launch_dependents;");
  const long long group = blockIdx.x * 32LL + (threadIdx.x >> 3);
  const int q = threadIdx.x & 7;
  const bool in_range = group < total_groups;
  const int vm = in_range ? static_cast<int>(group / nbpad) : 0;
  const int b = in_range ? static_cast<int>(group % nbpad) : 0;
  const bool real = in_range && vm < m && b < nb;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (real) {
    const float* src = x + static_cast<long long>(vm) * k + b * 32 + q * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = src[i];
  }
  // max of |bits|: orders finite < inf < NaN, so non-finite inputs are detected
  uint32_t amax_bits = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) amax_bits = max(amax_bits, __float_as_uint(v[i]) & 0x7FFFFFFFu);
#pragma unroll
  for (int s = 1; s < 8; s <<= 1) amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, s));
  const uint32_t eb_raw = amax_bits >> 23;
  const bool finite = eb_raw != 255u;
  const uint32_t eb = max(eb_raw, 30u);                       // envelope 2^(eb-126) > amax
  const float scale_up = __uint_as_float((275u - eb) << 23);  // 2^(22 - e)
  float scale = __uint_as_float((eb - 21u) << 23);            // 2^(e - 22)
  if (!finite) scale = __uint_as_float(0x7FC00000u);          // NaN/inf in -> NaN out
  uint32_t word[3] = {0, 0, 0};
  int psum[3] = {0, 0, 0};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = finite ? __float2int_rn(v[i] * scale_up) : 0;  // |t| <= 2^22
    const int p0 = ((t + 128) & 255) - 128;
    const int t1 = (t - p0) >> 8;
    const int p1 = ((t1 + 128) & 255) - 128;
    const int p2 = (t1 - p1) >> 8;
    word[0] |= static_cast<uint32_t>(p0 & 255) << (8 * i);
    word[1] |= static_cast<uint32_t>(p1 & 255) << (8 * i);
    word[2] |= static_cast<uint32_t>(p2 & 255) << (8 * i);
    psum[0] += p0;
    psum[1] += p1;
    psum[2] += p2;
  }
#pragma unroll
  for (int d = 0; d < 3; ++d) {
#pragma unroll
    for (int s = 1; s < 8; s <<= 1) psum[d] += __shfl_xor_sync(0xffffffffu, psum[d], s);
  }
  if (!in_range) return;
  // The images may still be read by the GEMV launched before this kernel (both are
  // launched programmatically, so this kernel can start early): wait for it to finish.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  uint8_t* image = ximg + static_cast<long long>(b / kSlabBlocks) * ximage_bytes(ncols);
  const int j = b % kSlabBlocks;
#pragma unroll
  for (int d = 0; d < kDigitStride; ++d) {
    const int col = vm * kDigitStride + d;
    if (col < ncols) {
      *reinterpret_cast<uint32_t*>(image + ximage_digit_offset(col, j, q)) =
          (real && d < 3) ? word[d < 3 ? d : 0] : 0u;
    }
  }
  if (q == 0 && vm < m) {
    XConst c;
    c.scale = real ? scale : 0.0f;
    c.k01 = real ? 8 * (256 * psum[1] + psum[0]) : 0;
    c.p2x8 = real ? 8 * psum[2] : 0;
    c.pad = 0;
    reinterpret_cast<XConst*>(image + ncols * 128)[vm * kSlabBlocks + j] = c;
  }
}

__device__ __forceinline__ float warp_tree_sum(float v) {
#pragma unroll
  for (int h = 16; h >= 1; h >>= 1) v += __shfl_xor_sync(0xffffffffu, v, h);
  return v;
}

// ------------------------------------------------------------------------------------
// CUDA-core kernel: one warp per (weight row, activation row); lanes stride over blocks.
// Reduction: per group of 32 consecutive blocks a fixed xor-butterfly (16, 8, 4, 2, 1),
// groups added in ascending order, so the result does not depend on the launch shape.
// ------------------------------------------------------------------------------------
template <int FMT>
__global__ void __launch_bounds__(256) gemv_dp4a_kernel(
    const uint8_t* __restrict__ panel, const uint8_t* __restrict__ ximg, int ncols,
    float* __restrict__ y, long long n, int nb, long long slabs, long long ldy) {
  constexpr int kVec = FMT == QX_FORMAT_Q8_0 ? 2 : 1;  // 16-byte vectors of codes per block
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * 8LL + (threadIdx.x >> 5);
  if (row >= n) return;
  const int m = blockIdx.y;
  constexpr size_t kCodeBytes = FMT == QX_FORMAT_Q8_0 ? 32 : 16;
  constexpr size_t kSlabCodes = kTileRows * kSlabBlocks * kCodeBytes;
  const long long tile = row / kTileRows;
  const int r = static_cast<int>(row % kTileRows);
  float acc = 0.0f;
  for (int base = 0; base < nb; base += 32) {
    const int b = base + lane;
    float v = 0.0f;
    if (b < nb) {
      const long long ts = tile * slabs + b / kSlabBlocks;
      const int j = b % kSlabBlocks;
      const uint8_t* span = panel + ts * (kSlabCodes + kTileRows * kSlabBlocks * 2);
      const uint4* codes = reinterpret_cast<const uint4*>(span + (r * kSlabBlocks + j) * kCodeBytes);
      const uint8_t* image = ximg + static_cast<long long>(b / kSlabBlocks) * ximage_bytes(ncols);
      uint32_t w[8];
#pragma unroll
      for (int i = 0; i < kVec; ++i) {
        const uint4 c = __ldg(codes + i);
        w[4 * i] = c.x; w[4 * i + 1] = c.y; w[4 * i + 2] = c.z; w[4 * i + 3] = c.w;
      }
      uint32_t dig[3][8];
#pragma unroll
      for (int d = 0; d < 3; ++d) {
        const int col = m * kDigitStride + d;
        const uint4 lo = __ldg(reinterpret_cast<const uint4*>(image + ximage_digit_offset(col, j, 0)));
        const uint4 hi = __ldg(reinterpret_cast<const uint4*>(image + ximage_digit_offset(col, j, 4)));
        dig[d][0] = lo.x; dig[d][1] = lo.y; dig[d][2] = lo.z; dig[d][3] = lo.w;
        dig[d][4] = hi.x; dig[d][5] = hi.y; dig[d][6] = hi.z; dig[d][7] = hi.w;
      }
      const XConst c = reinterpret_cast<const XConst*>(image + ncols * 128)[m * kSlabBlocks + j];
      int s[3];
      if (FMT == QX_FORMAT_Q8_0) {
#pragma unroll
        for (int d = 0; d < 3; ++d) {
          int t = 0;
#pragma unroll
          for (int i = 0; i < 8; ++i) t = dp4a_ss(w[i], dig[d][i], t);
          s[d] = t;
        }
      } else {
        // byte i of the block: low nibble = element i, high nibble = element i + 16; the
        // high nibbles are used in place (16 * nibble), so their sums are multiples of 16
#pragma unroll
        for (int d = 0; d < 3; ++d) {
          int lo = 0, hi = 0;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            lo = dp4a_us(w[i] & 0x0F0F0F0Fu, dig[d][i], lo);
            hi = dp4a_us(w[i] & 0xF0F0F0F0u, dig[d][4 + i], hi);
          }
          s[d] = lo + (hi >> 4);
        }
        s[0] -= c.k01;  // together with s[1]*256 below: -8 * sum_j (256*p1 + p0)
        s[2] -= c.p2x8;
      }
      const float d = half_bits_to_float(
          reinterpret_cast<const unsigned short*>(span + kSlabCodes)[j * kTileRows + r]);
      v = __fmul_rn(combine_digits(s[1] * 256 + s[0], s[2]), __fmul_rn(d, c.scale));
    }
    acc += warp_tree_sum(v);
  }
  if (lane == 0) y[m * ldy + row] = acc;
}

bool force_dp4a() {
  static const bool forced = []() {
    const char* v = std::getenv("QX_B200_GEMV_VARIANT");
    return v != nullptr && std::strcmp(v, "dp4a") == 0;
  }();
  return forced;
}

}  // namespace

const char* gemv_variant_name() { return force_dp4a() ? "sm100a_dp4a" : "sm100a_tcgen05_digits"; }

// Workspace layout of one GEMV call: [row counters | activation slab images | per-unit
// partial sums]; sizes depend only on (m, k, rows).
qx_status launch_qgemm_f32(const qx_weights* w, const float* x_dev, float* y_dev,
                           long long m, long long ldy, qx_workspace* ws,
                           cudaStream_t stream) {
  const int nb = static_cast<int>(w->blocks_per_row);
  const int nbpad = static_cast<int>(w->slabs) * kSlabBlocks;
  const long long kpad = static_cast<long long>(nbpad) * 32;
  if (w->columns > (1LL << 24) || w->rows > (1LL << 31) - 256) {
    set_last_error_text("qgemm: shape beyond the GEMV kernels' 32-bit tile indices");
    return QX_STATUS_INVALID_SHAPE;
  }
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  for (long long m0 = 0; m0 < m; m0 += kGemvMaxBatch) {
    const int mc = static_cast<int>(m - m0 < kGemvMaxBatch ? m - m0 : kGemvMaxBatch);
    const int ncols = digit_columns(mc);
    GemvScratch scratch;
    QX_TRY(gemv_scratch_layout(w, mc, ctx->prop.multiProcessorCount, &scratch));
    QX_TRY(ws->reserve(scratch.total_bytes));
    uint8_t* base = static_cast<uint8_t*>(ws->base);
    uint8_t* ximg = base + scratch.ximg_offset;

    const int vrows = ncols / kDigitStride;
    const long long groups = static_cast<long long>(vrows) * nbpad;
    {
      cudaLaunchConfig_t config{};
      config.gridDim = dim3(static_cast<unsigned>((groups + 31) / 32));
      config.blockDim = dim3(256);
      config.stream = stream;
      cudaLaunchAttribute attribute{};
      attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attribute.val.programmaticStreamSerializationAllowed = 1;
      config.attrs = &attribute;
      config.numAttrs = 1;
      QX_CUDA_TRY(cudaLaunchKernelEx(&config, quantize_x_kernel, x_dev + m0 * w->columns, ximg, mc,
                                     static_cast<int>(w->columns), nb, nbpad, ncols, groups));
    }
    count_launch();
    float* y = y_dev + m0 * ldy;
    if (!force_dp4a()) {
      QX_TRY(launch_gemv_tc(w, ximg, y, mc, ldy, base, scratch, stream));
    } else {
      const dim3 grid(static_cast<unsigned>((w->rows + 7) / 8), static_cast<unsigned>(mc));
      if (w->format == QX_FORMAT_Q8_0) {
        gemv_dp4a_kernel<QX_FORMAT_Q8_0><<<grid, 256, 0, stream>>>(w->panel, ximg, ncols, y, w->rows,
                                                                   nb, w->slabs, ldy);
      } else {
        gemv_dp4a_kernel<QX_FORMAT_Q4_0><<<grid, 256, 0, stream>>>(w->panel, ximg, ncols, y, w->rows,
                                                                   nb, w->slabs, ldy);
      }
      count_launch();
    }
    QX_CUDA_TRY(cudaGetLastError());
    (void)kpad;
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
// partial sums, per-row counters and the pipeline error word) lives in the array below,
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
  const size_t error_offset = align_up(scratch.total_bytes, 256);
  if (error_offset + 256 > kNoAllocScratchBytes) {
    set_last_error_text(
        "qgemv (no-alloc): this weight matrix needs more scratch than the 6 MiB static array "
        "(limit is about rows * ceil(columns/128 units) * 4 B <= 5 MiB; use qx_qgemm_prepacked_dev)");
    return QX_STATUS_INVALID_SHAPE;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* base = dev->scratch;
  // The array keeps whatever the previous call left. The kernel expects the row counters it
  // uses and the error word to be zero; everything else is fully rewritten before it is read.
  QX_CUDA_TRY(cudaMemsetAsync(base, 0, static_cast<size_t>(weights->tiles) * kTileRows * sizeof(int), s));
  QX_CUDA_TRY(cudaMemsetAsync(base + error_offset, 0, 256, s));

  uint8_t* ximg = base + scratch.ximg_offset;
  const int nb = static_cast<int>(weights->blocks_per_row);
  const int nbpad = static_cast<int>(weights->slabs) * kSlabBlocks;
  const int ncols = digit_columns(1);
  const long long groups = static_cast<long long>(ncols / kDigitStride) * nbpad;
  quantize_x_kernel<<<static_cast<unsigned>((groups + 31) / 32), 256, 0, s>>>(
      x_dev, ximg, 1, static_cast<int>(weights->columns), nb, nbpad, ncols, groups);
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  return launch_gemv_tc_at(weights, ximg, y_dev, 1, weights->rows, base, scratch,
                           reinterpret_cast<int*>(base + error_offset), s);
}
