// The reference's compact 4-bit row formats and the int8 activation quantiser:
//   quantize_int8        kernels/quantization/quantization_ref.cpp:143-168
//   lowbit_gemm_w8a8     src/dispatch/lowbit_w8a8.cpp:68-101,
//                        kernels/quantization/lowbit_w8a8_ref.cpp:7-32   (W4A8, exact integer)
//   lowbit_gemm          kernels/quantization/lowbit_ref.cpp:229-256     (int4 x f32)
//   lowbit_pack / unpack kernels/quantization/lowbit_ref.cpp:277-352     (authoring)
// for LowBitFormat::kInt4Row and kInt4Group (include/quixicore_cpu/lowbit.h:15-47). Unlike
// the GGUF q4_0 blocks these rows hold ADJACENT elements per byte (element 2i in the low
// nibble, 2i + 1 in the high one, value = nibble - 8) and keep their f32 scales in a
// separate array (one per row, or one per group of `group_size` inputs).
//
// Both matmuls are weight-streaming kernels for decode-sized batches: a warp owns an output
// channel, lanes read 16 bytes (32 weights) at a time, the weights are read ONCE for up to
// MT activation rows. W4A8 multiplies with dp4a (the nibbles of a word as two unsigned
// operands against the even / odd activation codes, the -8 folded into 8 * sum(codes) per
// row) and reproduces the reference bit for bit: exact int32 dot, then
// float(dot) * weight_scale * activation_scale as two rounded multiplies.

#include <cmath>
#include <limits>

#include "qx_common.cuh"
#include "qx_int8_gemm.cuh"

namespace qx {
namespace {

constexpr int kInt2Row = 0, kInt3Group64 = 1, kInt4Row = 2, kInt4Group = 3;

// Launch with programmatic dependent launch allowed: the kernel may start while the kernel
// in front of it on the stream still runs and waits for it itself (griddepcontrol.wait).
template <class... Params, class... Args>
cudaError_t launch_dependent(void (*kernel)(Params...), unsigned grid, unsigned block,
                             cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(block);
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// ---- quantize_int8 ---------------------------------------------------------------------
// One warp per (row, group). max() is exact in any order; the divisions are IEEE like the
// reference's; nearbyint = round half to even.
__global__ void __launch_bounds__(256) quantize_int8_kernel(const float* __restrict__ x,
                                                            int8_t* __restrict__ codes,
                                                            float* __restrict__ scales,
                                                            int* __restrict__ code_sums,
                                                            long long groups_total,
                                                            long long group_size) {
  const int lane = threadIdx.x & 31;
  const long long g = blockIdx.x * 8LL + (threadIdx.x >> 5);
  if (g >= groups_total) return;
  const float* in = x + g * group_size;
  float maximum = 0.0f;
  for (long long i = lane; i < group_size; i += 32) maximum = fmaxf(maximum, fabsf(in[i]));
#pragma unroll
  for (int h = 16; h >= 1; h >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, h));
  const float scale = __fdiv_rn(maximum, 127.0f);
  const float inverse = scale > 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
  int sum = 0;
  for (long long i = lane; i < group_size; i += 32) {
    int q = __float2int_rn(__fmul_rn(in[i], inverse));
    q = max(-127, min(127, q));
    codes[g * group_size + i] = static_cast<int8_t>(q);
    sum += q;
  }
#pragma unroll
  for (int h = 16; h >= 1; h >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, h);
  if (lane == 0) {
    scales[g] = scale;
    if (code_sums != nullptr) code_sums[g] = sum;
  }
}

// Long groups (a whole activation row of a few thousand elements): one block per group, so
// the row is read with 256 lanes instead of 32. Same values: max and the integer sum do not
// depend on the order. It lets the kernel behind it (the W4A8 GEMM, which first fetches
// weights) start at once and waits for the kernel in front itself.
__global__ void __launch_bounds__(256) quantize_int8_block_kernel(const float* __restrict__ x,
                                                                  int8_t* __restrict__ codes,
                                                                  float* __restrict__ scales,
                                                                  int* __restrict__ code_sums,
                                                                  long long group_size) {
  asm volatile("griddepcontrol.launch_dependents;");
  // x may be the output of the kernel in front, and the codes are read by the GEMM in front
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __shared__ float warp_max[8];
  __shared__ int warp_sum[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long g = blockIdx.x;
  const float* in = x + g * group_size;
  float maximum = 0.0f;
  for (long long i = threadIdx.x; i < group_size; i += 256) maximum = fmaxf(maximum, fabsf(in[i]));
#pragma unroll
  for (int h = 16; h >= 1; h >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, h));
  if (lane == 0) warp_max[warp] = maximum;
  __syncthreads();
#pragma unroll
  for (int w = 0; w < 8; ++w) maximum = fmaxf(maximum, warp_max[w]);
  const float scale = __fdiv_rn(maximum, 127.0f);
  const float inverse = scale > 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
  int sum = 0;
  for (long long i = threadIdx.x; i < group_size; i += 256) {
    int q = __float2int_rn(__fmul_rn(in[i], inverse));
    q = max(-127, min(127, q));
    codes[g * group_size + i] = static_cast<int8_t>(q);
    sum += q;
  }
#pragma unroll
  for (int h = 16; h >= 1; h >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, h);
  if (lane == 0) warp_sum[warp] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    int total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += warp_sum[w];
    scales[g] = scale;
    if (code_sums != nullptr) code_sums[g] = total;
  }
}

// ---- W4A8 ------------------------------------------------------------------------------
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// One warp per output channel, MT activation rows per pass. x codes [m][k] int8, code_sums
// [m] (sum of a row's codes: sum (nib - 8) q = sum nib q - 8 sum q).
template <int MT>
__global__ void __launch_bounds__(256) lowbit_w8a8_kernel(
    const uint8_t* __restrict__ packed, const float* __restrict__ weight_scales,
    const int8_t* __restrict__ x, const float* __restrict__ activation_scales,
    const int* __restrict__ code_sums, float* __restrict__ y, int m, long long n, long long k,
    int vector_ok) {
  asm volatile("griddepcontrol.launch_dependents;");
  const int lane = threadIdx.x & 31;
  const long long o = blockIdx.x * 8LL + (threadIdx.x >> 5);
  if (o >= n) return;
  const long long row_bytes = (k + 1) / 2;
  const uint8_t* wr = packed + o * row_bytes;
  int acc[MT];
#pragma unroll
  for (int r = 0; r < MT; ++r) acc[r] = 0;
  // 32 weights of this lane (four words) against the activation codes k0 .. k0 + 31 of every row
  auto consume = [&](const uint32_t (&w)[4], long long k0, bool whole) {
#pragma unroll
    for (int r = 0; r < MT; ++r) {
      if (r < m) {
        const int8_t* xr = x + static_cast<long long>(r) * k + k0;
        uint32_t xw[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
        if (whole) {
          const uint4 a = __ldg(reinterpret_cast<const uint4*>(xr));
          const uint4 b = __ldg(reinterpret_cast<const uint4*>(xr) + 1);
          xw[0] = a.x; xw[1] = a.y; xw[2] = a.z; xw[3] = a.w;
          xw[4] = b.x; xw[5] = b.y; xw[6] = b.z; xw[7] = b.w;
        } else {
          for (int i = 0; i < 32 && k0 + i < k; ++i) {
            xw[i >> 2] |= static_cast<uint32_t>(static_cast<uint8_t>(xr[i])) << (8 * (i & 3));
          }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          // word q of the weights = elements 8q .. 8q+7: low nibbles are the even ones
          const uint32_t lo = w[q] & 0x0F0F0F0Fu, hi = (w[q] >> 4) & 0x0F0F0F0Fu;
          const uint32_t even = __byte_perm(xw[2 * q], xw[2 * q + 1], 0x6420);
          const uint32_t odd = __byte_perm(xw[2 * q], xw[2 * q + 1], 0x7531);
          acc[r] = dp4a_us(lo, even, acc[r]);
          acc[r] = dp4a_us(hi, odd, acc[r]);
        }
      }
    }
  };
  if (vector_ok != 0 && (k & 1023) == 0) {
    // whole strides of the warp: the weight loads of four strides leave before they are used,
    // the first four before this kernel waits for the activation codes of the kernel in front
    bool waited = false;
    for (long long kb = lane * 32LL; kb < k; kb += 4 * 1024) {
      uint4 v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (kb + i * 1024 < k) v[i] = __ldg(reinterpret_cast<const uint4*>(wr + ((kb + i * 1024) >> 1)));
      }
      if (!waited) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        waited = true;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (kb + i * 1024 < k) {
          const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
          consume(w, kb + i * 1024, true);
        }
      }
    }
  } else {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (long long k0 = lane * 32LL; k0 < k; k0 += 32 * 32) {
      uint32_t w[4] = {0u, 0u, 0u, 0u};
      const bool whole = vector_ok != 0 && k0 + 32 <= k;
      if (whole) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(wr + (k0 >> 1)));
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
      } else {
        for (int i = 0; i < 16 && (k0 >> 1) + i < row_bytes; ++i) {
          w[i >> 2] |= static_cast<uint32_t>(wr[(k0 >> 1) + i]) << (8 * (i & 3));
        }
      }
      consume(w, k0, whole);
    }
  }
  // an odd k leaves the high nibble of the last byte unused: its activation code is zero
  // padding above, so it contributed nothing
  const float ws = weight_scales[o];
#pragma unroll
  for (int r = 0; r < MT; ++r) {
    int dot = acc[r];
#pragma unroll
    for (int h = 16; h >= 1; h >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, h);
    if (lane == 0 && r < m) {
      dot -= 8 * code_sums[r];
      y[static_cast<long long>(r) * n + o] =
          __fmul_rn(__fmul_rn(static_cast<float>(dot), ws), activation_scales[r]);
    }
  }
}

// ---- int4 x f32 ------------------------------------------------------------------------
// Same structure with f32 FMAs: lane = 32 consecutive inputs per step (they lie in one
// group when group_size % 32 == 0, the fast path), nibble -> f32 through the mantissa of
// 2^23; each 32-input partial is scaled by its group's scale before it is accumulated.
template <int MT>
__global__ void __launch_bounds__(256) lowbit_f32_kernel(
    const uint8_t* __restrict__ packed, const float* __restrict__ scales,
    const float* __restrict__ x, float* __restrict__ y, int m, long long n, long long k,
    long long groups, long long group_size, int vector_ok) {
  const int lane = threadIdx.x & 31;
  const long long o = blockIdx.x * 8LL + (threadIdx.x >> 5);
  if (o >= n) return;
  const long long row_bytes = (k + 1) / 2;
  const uint8_t* wr = packed + o * row_bytes;
  const float* row_scales = scales + o * groups;
  float acc[MT];
#pragma unroll
  for (int r = 0; r < MT; ++r) acc[r] = 0.0f;
  for (long long k0 = lane * 32LL; k0 < k; k0 += 32 * 32) {
    uint32_t w[4] = {0u, 0u, 0u, 0u};
    const bool whole = vector_ok != 0 && k0 + 32 <= k;
    if (whole) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(wr + (k0 >> 1)));
      w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    } else {
      for (int i = 0; i < 16 && (k0 >> 1) + i < row_bytes; ++i) {
        w[i >> 2] |= static_cast<uint32_t>(wr[(k0 >> 1) + i]) << (8 * (i & 3));
      }
    }
    float wf[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const uint32_t nib = (w[i >> 3] >> (4 * (i & 7))) & 15u;
      wf[i] = __uint_as_float(0x4B000000u | nib) - 8388616.0f;  // nib - 8
    }
    const bool one_group = whole && (k0 / group_size == (k0 + 31) / group_size);
#pragma unroll
    for (int r = 0; r < MT; ++r) {
      if (r < m) {
        const float* xr = x + static_cast<long long>(r) * k + k0;
        if (one_group) {
          float partial = 0.0f;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 xv = __ldg(reinterpret_cast<const float4*>(xr) + q);
            partial = fmaf(xv.x, wf[4 * q], partial);
            partial = fmaf(xv.y, wf[4 * q + 1], partial);
            partial = fmaf(xv.z, wf[4 * q + 2], partial);
            partial = fmaf(xv.w, wf[4 * q + 3], partial);
          }
          acc[r] = fmaf(partial, row_scales[k0 / group_size], acc[r]);
        } else {
          for (int i = 0; i < 32 && k0 + i < k; ++i) {
            acc[r] = fmaf(xr[i] * wf[i], row_scales[(k0 + i) / group_size], acc[r]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < MT; ++r) {
    float sum = acc[r];
#pragma unroll
    for (int h = 16; h >= 1; h >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, h);
    if (lane == 0 && r < m) y[static_cast<long long>(r) * n + o] = sum;
  }
}

// ---- authoring -------------------------------------------------------------------------
// One warp per (row, group): scale = max(amax / 7, 1e-8), code = clamp(nearbyint(w / scale),
// -8, 7) + 8 (kernels/quantization/lowbit_ref.cpp:302-343). Bytes are written whole by the
// lane that owns both of their nibbles (groups of odd size share a byte: handled by the
// caller choosing the byte-wise path).
__global__ void __launch_bounds__(256) int4_pack_kernel(const float* __restrict__ weights,
                                                        uint8_t* __restrict__ packed,
                                                        float* __restrict__ scales,
                                                        long long rows, long long dim,
                                                        long long groups, long long group_size,
                                                        int* __restrict__ bad) {
  const int lane = threadIdx.x & 31;
  const long long item = blockIdx.x * 8LL + (threadIdx.x >> 5);
  if (item >= rows * groups) return;
  const long long row = item / groups, group = item % groups;
  const long long first = group * group_size;
  const long long last = first + group_size < dim ? first + group_size : dim;
  const float* src = weights + row * dim;
  float maximum = 0.0f;
  bool finite = true;
  for (long long i = first + lane; i < last; i += 32) {
    const float v = src[i];
    finite = finite && (__float_as_uint(v) & 0x7F800000u) != 0x7F800000u;
    maximum = fmaxf(maximum, fabsf(v));
  }
#pragma unroll
  for (int h = 16; h >= 1; h >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, h));
  if (!__all_sync(0xffffffffu, finite)) {
    if (lane == 0) atomicOr(bad, 1);
    return;
  }
  const float scale = fmaxf(__fdiv_rn(maximum, 7.0f), 1e-8f);
  if (lane == 0) scales[row * groups + group] = scale;
  uint8_t* dst = packed + row * ((dim + 1) / 2);
  // whole bytes inside the group; a byte shared with a neighbouring group (odd boundaries)
  // is assembled with atomics on the containing word
  for (long long i = first + lane; i < last; i += 32) {
    int code = __float2int_rn(__fdiv_rn(src[i], scale));
    code = max(-8, min(7, code)) + 8;
    const long long byte = i >> 1;
    const uint32_t shifted = static_cast<uint32_t>(code) << (4 * (i & 1));
    uint32_t* word = reinterpret_cast<uint32_t*>(reinterpret_cast<uintptr_t>(dst + byte) & ~uintptr_t(3));
    const int byte_in_word = static_cast<int>(reinterpret_cast<uintptr_t>(dst + byte) & 3);
    atomicOr(word, shifted << (8 * byte_in_word));
  }
}

__global__ void __launch_bounds__(256) int4_unpack_kernel(const uint8_t* __restrict__ packed,
                                                          const float* __restrict__ scales,
                                                          float* __restrict__ weights,
                                                          long long rows, long long dim,
                                                          long long groups, long long group_size) {
  const long long i = blockIdx.x * 256LL + threadIdx.x;
  if (i >= rows * dim) return;
  const long long row = i / dim, input = i % dim;
  const int code = static_cast<int>((packed[row * ((dim + 1) / 2) + (input >> 1)] >> (4 * (input & 1))) & 15) - 8;
  weights[i] = __fmul_rn(static_cast<float>(code), scales[row * groups + input / group_size]);
}

// include/quixicore_cpu/lowbit.h + kernels/quantization/lowbit_ref.cpp:41-68
struct Layout {
  long long row_bytes = 0, groups = 0, group_size = 0;
};
bool layout_for(int format, long long dim, long long group_size, Layout* layout) {
  if (dim <= 0) return false;
  switch (format) {
    case kInt2Row:
      *layout = {(dim + 3) / 4, 1, dim};
      return true;
    case kInt3Group64: {
      const long long groups = (dim + 63) / 64;
      if (groups > std::numeric_limits<long long>::max() / 24) return false;
      *layout = {groups * 24, groups, 64};
      return true;
    }
    case kInt4Row:
      *layout = {(dim + 1) / 2, 1, dim};
      return true;
    case kInt4Group:
      if (group_size <= 0) return false;
      *layout = {(dim + 1) / 2, (dim + group_size - 1) / group_size, group_size};
      return true;
    default:
      return false;
  }
}
bool checked_size(long long a, long long b, size_t* out) {
  if (a < 0 || b < 0) return false;
  const size_t ua = static_cast<size_t>(a), ub = static_cast<size_t>(b);
  if (ua != 0 && ub > std::numeric_limits<size_t>::max() / ua) return false;
  *out = ua * ub;
  return true;
}
bool finite_host(const float* v, long long count) {
  for (long long i = 0; i < count; ++i) {
    if (!std::isfinite(v[i])) return false;
  }
  return true;
}
// kernels/quantization/lowbit_ref.cpp:203-222 (the scale check is the caller's: it needs
// the scales on the host)
qx_status validate_lowbit(int format, const void* packed, const void* scales, long long rows,
                          long long dim, long long group_size, Layout* layout) {
  const bool layout_ok = layout_for(format, dim, group_size, layout);
  if (!valid_product2(rows, dim) || packed == nullptr || scales == nullptr || !layout_ok) {
    return rows <= 0 || dim <= 0 || !layout_ok ? QX_STATUS_INVALID_SHAPE : QX_STATUS_INVALID_ARGUMENT;
  }
  size_t ignored = 0;
  if (!checked_size(rows, layout->row_bytes, &ignored) || !checked_size(rows, layout->groups, &ignored)) {
    return QX_STATUS_INVALID_SHAPE;
  }
  return QX_STATUS_OK;
}
bool int4_format(int format) { return format == kInt4Row || format == kInt4Group; }

qx_status launch_quantize_int8(const float* x, int8_t* codes, float* scales, int* code_sums,
                               long long rows, long long dim, long long group_size,
                               cudaStream_t stream) {
  const long long groups_total = rows * (dim / group_size);
  if (group_size >= 1024 && groups_total <= 65535) {
    QX_CUDA_TRY(launch_dependent(quantize_int8_block_kernel, static_cast<unsigned>(groups_total), 256,
                                 stream, x, codes, scales, code_sums, group_size));
  } else {
    quantize_int8_kernel<<<static_cast<unsigned>((groups_total + 7) / 8), 256, 0, stream>>>(
        x, codes, scales, code_sums, groups_total, group_size);
  }
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  return QX_STATUS_OK;
}

template <class Launch>
qx_status for_row_chunks(long long m, Launch&& launch) {
  for (long long r0 = 0; r0 < m; r0 += 8) {
    const int mc = static_cast<int>(m - r0 < 8 ? m - r0 : 8);
    launch(r0, mc);
    count_launch();
    QX_CUDA_TRY(cudaGetLastError());
  }
  return QX_STATUS_OK;
}

}  // namespace

// y[m][n] from W4A8 operands already on the device (codes, scales, code sums of x).
qx_status launch_lowbit_w8a8(const uint8_t* packed, const float* weight_scales, const int8_t* codes,
                             const float* activation_scales, const int* code_sums, float* y,
                             long long m, long long n, long long k, cudaStream_t stream) {
  const int vector_ok = (reinterpret_cast<uintptr_t>(packed) % 16 == 0 && k % 32 == 0 &&
                         reinterpret_cast<uintptr_t>(codes) % 16 == 0)
                            ? 1
                            : 0;
  const unsigned grid = static_cast<unsigned>((n + 7) / 8);
  return for_row_chunks(m, [&](long long r0, int mc) {
    if (mc <= 2) {
      (void)launch_dependent(lowbit_w8a8_kernel<2>, grid, 256, stream, packed, weight_scales,
                             codes + r0 * k, activation_scales + r0, code_sums + r0, y + r0 * n, mc,
                             n, k, vector_ok);
    } else {
      (void)launch_dependent(lowbit_w8a8_kernel<8>, grid, 256, stream, packed, weight_scales,
                             codes + r0 * k, activation_scales + r0, code_sums + r0, y + r0 * n, mc,
                             n, k, vector_ok);
    }
  });
}

qx_status launch_lowbit_f32(const uint8_t* packed, const float* scales, const float* x, float* y,
                            long long m, long long n, long long k, long long groups,
                            long long group_size, cudaStream_t stream) {
  // rows of an even number of columns with scale groups of a multiple of 16 columns: the digit
  // kernels (exact 8-bit activation digits, dp4a); everything else: the float kernel below
  if (int4_offset8_digits_serves(m, k, groups, group_size)) {
    return launch_int4_offset8_digits(packed, scales, x, y, m, n, k, groups, group_size, stream);
  }
  const int vector_ok = (reinterpret_cast<uintptr_t>(packed) % 16 == 0 && k % 32 == 0 &&
                         reinterpret_cast<uintptr_t>(x) % 16 == 0)
                            ? 1
                            : 0;
  const unsigned grid = static_cast<unsigned>((n + 7) / 8);
  return for_row_chunks(m, [&](long long r0, int mc) {
    if (mc <= 2) {
      lowbit_f32_kernel<2><<<grid, 256, 0, stream>>>(packed, scales, x + r0 * k, y + r0 * n, mc, n, k,
                                                     groups, group_size, vector_ok);
    } else {
      lowbit_f32_kernel<8><<<grid, 256, 0, stream>>>(packed, scales, x + r0 * k, y + r0 * n, mc, n, k,
                                                     groups, group_size, vector_ok);
    }
  });
}

}  // namespace qx

using namespace qx;

extern "C" {

// lowbit_packed_size, kernels/quantization/lowbit_ref.cpp:258-272
qx_status qx_lowbit_packed_size(int format, long long rows, long long dim, long long group_size,
                                size_t* weight_bytes, size_t* scale_count) {
  if (rows <= 0 || dim <= 0) return QX_STATUS_INVALID_SHAPE;
  if (weight_bytes == nullptr || scale_count == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  Layout layout;
  if (!layout_for(format, dim, group_size, &layout) || !checked_size(rows, layout.row_bytes, weight_bytes) ||
      !checked_size(rows, layout.groups, scale_count)) {
    return QX_STATUS_INVALID_SHAPE;
  }
  return QX_STATUS_OK;
}

// quantize_int8, kernels/quantization/quantization_ref.cpp:143-168 (DEVICE pointers).
// code_sums_dev (optional) receives the sum of every group's codes.
qx_status qx_quantize_int8_dev(const float* x_dev, int8_t* codes_dev, float* scales_dev,
                               int* code_sums_dev, long long rows, long long dim,
                               long long group_size, void* stream) {
  if (!valid_product2(rows, dim)) return QX_STATUS_INVALID_SHAPE;
  if (group_size == 0) group_size = dim;
  if (group_size <= 0 || dim % group_size != 0) return QX_STATUS_INVALID_SHAPE;
  if (x_dev == nullptr || codes_dev == nullptr || scales_dev == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  return launch_quantize_int8(x_dev, codes_dev, scales_dev, code_sums_dev, rows, dim, group_size,
                              static_cast<cudaStream_t>(stream));
}

// quantize_int8 with HOST pointers: shape -> null -> finite (quantization_ref.cpp:145-147)
qx_status qx_quantize_int8(const float* x, int8_t* codes, float* scales, long long rows,
                           long long dim, long long group_size) {
  if (!valid_product2(rows, dim)) return QX_STATUS_INVALID_SHAPE;
  if (group_size == 0) group_size = dim;
  if (group_size <= 0 || dim % group_size != 0) return QX_STATUS_INVALID_SHAPE;
  if (x == nullptr || codes == nullptr || scales == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  if (!finite_host(x, rows * dim)) return QX_STATUS_INVALID_ARGUMENT;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  std::lock_guard<std::mutex> lock(ctx->mutex);
  const size_t count = static_cast<size_t>(rows) * dim, groups = static_cast<size_t>(rows) * (dim / group_size);
  const size_t off_x = 0, off_c = align_up(count * 4, 256), off_s = off_c + align_up(count, 256);
  QX_TRY(ctx->ensure_staging(off_s + align_up(groups * 4, 256)));
  uint8_t* base = static_cast<uint8_t*>(ctx->staging);
  cudaStream_t s = ctx->stream;
  QX_CUDA_TRY(cudaMemcpyAsync(base + off_x, x, count * 4, cudaMemcpyHostToDevice, s));
  QX_TRY(launch_quantize_int8(reinterpret_cast<const float*>(base + off_x),
                              reinterpret_cast<int8_t*>(base + off_c),
                              reinterpret_cast<float*>(base + off_s), nullptr, rows, dim, group_size, s));
  QX_CUDA_TRY(cudaMemcpyAsync(codes, base + off_c, count, cudaMemcpyDeviceToHost, s));
  QX_CUDA_TRY(cudaMemcpyAsync(scales, base + off_s, groups * 4, cudaMemcpyDeviceToHost, s));
  QX_CUDA_TRY(cudaStreamSynchronize(s));
  return QX_STATUS_OK;
}

// lowbit_gemm_w8a8 on the device: x f32 [m][k]; scratch_dev holds the activation codes,
// scales and code sums: qx_lowbit_w8a8_scratch_bytes(m, k) bytes.
size_t qx_lowbit_w8a8_scratch_bytes(long long m, long long k) {
  if (m <= 0 || k <= 0) return 0;
  return align_up(static_cast<size_t>(m) * k, 256) + 2 * align_up(static_cast<size_t>(m) * 4, 256);
}

qx_status qx_lowbit_gemm_w8a8_dev(const uint8_t* packed_dev, const float* weight_scales_dev,
                                  const float* x_dev, float* y_dev, void* scratch_dev, long long m,
                                  long long n, long long k, void* stream) {
  if (!valid_product3(m, n, k)) return QX_STATUS_INVALID_SHAPE;
  if (packed_dev == nullptr || weight_scales_dev == nullptr || x_dev == nullptr || y_dev == nullptr ||
      scratch_dev == nullptr) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  if (k > 131000) {  // 15 * 127 * k must stay inside int32 (the reference's own guard)
    set_last_error_text("lowbit_gemm_w8a8: k beyond the exact int32 range");
    return QX_STATUS_INVALID_SHAPE;
  }
  uint8_t* base = static_cast<uint8_t*>(scratch_dev);
  int8_t* codes = reinterpret_cast<int8_t*>(base);
  float* scales = reinterpret_cast<float*>(base + align_up(static_cast<size_t>(m) * k, 256));
  int* sums = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(scales) + align_up(static_cast<size_t>(m) * 4, 256));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  QX_TRY(launch_quantize_int8(x_dev, codes, scales, sums, m, k, k, s));
  return launch_lowbit_w8a8(packed_dev, weight_scales_dev, codes, scales, sums, y_dev, m, n, k, s);
}

// lowbit_gemm_w8a8, src/dispatch/lowbit_w8a8.cpp:68-101 (HOST pointers): shape -> null ->
// packed-size status -> quantize_int8's own checks (finite activations)
qx_status qx_lowbit_gemm_w8a8(const uint8_t* packed_weights, const float* weight_scales,
                              const float* x, float* y, long long m, long long n, long long k) {
  if (!valid_product3(m, n, k)) return QX_STATUS_INVALID_SHAPE;
  if (packed_weights == nullptr || weight_scales == nullptr || x == nullptr || y == nullptr) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  size_t bytes = 0, scale_count = 0;
  QX_TRY(qx_lowbit_packed_size(kInt4Row, n, k, 0, &bytes, &scale_count));
  if (!finite_host(x, m * k)) return QX_STATUS_INVALID_ARGUMENT;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  std::lock_guard<std::mutex> lock(ctx->mutex);
  const size_t x_bytes = static_cast<size_t>(m) * k * 4, y_bytes = static_cast<size_t>(m) * n * 4;
  const size_t off_w = 0, off_ws = align_up(bytes, 256), off_x = off_ws + align_up(scale_count * 4, 256);
  const size_t off_y = off_x + align_up(x_bytes, 256), off_scratch = off_y + align_up(y_bytes, 256);
  QX_TRY(ctx->ensure_staging(off_scratch + qx_lowbit_w8a8_scratch_bytes(m, k)));
  uint8_t* base = static_cast<uint8_t*>(ctx->staging);
  cudaStream_t s = ctx->stream;
  QX_CUDA_TRY(cudaMemcpyAsync(base + off_w, packed_weights, bytes, cudaMemcpyHostToDevice, s));
  QX_CUDA_TRY(cudaMemcpyAsync(base + off_ws, weight_scales, scale_count * 4, cudaMemcpyHostToDevice, s));
  QX_CUDA_TRY(cudaMemcpyAsync(base + off_x, x, x_bytes, cudaMemcpyHostToDevice, s));
  QX_TRY(qx_lowbit_gemm_w8a8_dev(base + off_w, reinterpret_cast<const float*>(base + off_ws),
                                 reinterpret_cast<const float*>(base + off_x),
                                 reinterpret_cast<float*>(base + off_y), base + off_scratch, m, n, k, s));
  QX_CUDA_TRY(cudaMemcpyAsync(y, base + off_y, y_bytes, cudaMemcpyDeviceToHost, s));
  QX_CUDA_TRY(cudaStreamSynchronize(s));
  return QX_STATUS_OK;
}

const char* qx_lowbit_gemm_w8a8_variant(void) { return "sm100a_dp4a_stream"; }

const char* qx_lowbit_gemm_variant(int format) {
  return int4_format(format) ? "sm100a_digits_dp4a+stream_fma" : "unsupported";
}

// lowbit_gemm (int4 row / group formats), DEVICE pointers.
qx_status qx_lowbit_gemm_dev(int format, const uint8_t* packed_dev, const float* weight_scales_dev,
                             const float* x_dev, float* y_dev, long long m, long long n, long long k,
                             long long group_size, void* stream) {
  Layout layout;
  QX_TRY(validate_lowbit(format, packed_dev, weight_scales_dev, n, k, group_size, &layout));
  if (!int4_format(format)) return QX_STATUS_UNSUPPORTED_FORMAT;
  if (!valid_product2(m, k) || !valid_product2(m, n)) return QX_STATUS_INVALID_SHAPE;
  if (x_dev == nullptr || y_dev == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  return launch_lowbit_f32(packed_dev, weight_scales_dev, x_dev, y_dev, m, n, k, layout.groups,
                           layout.group_size, static_cast<cudaStream_t>(stream));
}

// lowbit_gemm, kernels/quantization/lowbit_ref.cpp:366-384 (HOST pointers): validate_lowbit
// (shape / null / sizes / finite scales) -> shapes with m -> null -> finite activations
qx_status qx_lowbit_gemm(int format, const uint8_t* packed_weights, const float* weight_scales,
                         const float* x, float* y, long long m, long long n, long long k,
                         long long group_size) {
  Layout layout;
  QX_TRY(validate_lowbit(format, packed_weights, weight_scales, n, k, group_size, &layout));
  if (!finite_host(weight_scales, n * layout.groups)) return QX_STATUS_INVALID_ARGUMENT;
  if (!valid_product2(m, k) || !valid_product2(m, n)) return QX_STATUS_INVALID_SHAPE;
  if (x == nullptr || y == nullptr || !finite_host(x, m * k)) return QX_STATUS_INVALID_ARGUMENT;
  if (!int4_format(format)) return QX_STATUS_UNSUPPORTED_FORMAT;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  std::lock_guard<std::mutex> lock(ctx->mutex);
  const size_t w_bytes = static_cast<size_t>(n) * layout.row_bytes, s_bytes = static_cast<size_t>(n) * layout.groups * 4;
  const size_t x_bytes = static_cast<size_t>(m) * k * 4, y_bytes = static_cast<size_t>(m) * n * 4;
  const size_t off_w = 0, off_s = align_up(w_bytes, 256), off_x = off_s + align_up(s_bytes, 256);
  const size_t off_y = off_x + align_up(x_bytes, 256);
  QX_TRY(ctx->ensure_staging(off_y + align_up(y_bytes, 256)));
  uint8_t* base = static_cast<uint8_t*>(ctx->staging);
  cudaStream_t s = ctx->stream;
  QX_CUDA_TRY(cudaMemcpyAsync(base + off_w, packed_weights, w_bytes, cudaMemcpyHostToDevice, s));
  QX_CUDA_TRY(cudaMemcpyAsync(base + off_s, weight_scales, s_bytes, cudaMemcpyHostToDevice, s));
  QX_CUDA_TRY(cudaMemcpyAsync(base + off_x, x, x_bytes, cudaMemcpyHostToDevice, s));
  QX_TRY(launch_lowbit_f32(base + off_w, reinterpret_cast<const float*>(base + off_s),
                           reinterpret_cast<const float*>(base + off_x),
                           reinterpret_cast<float*>(base + off_y), m, n, k, layout.groups,
                           layout.group_size, s));
  QX_CUDA_TRY(cudaMemcpyAsync(y, base + off_y, y_bytes, cudaMemcpyDeviceToHost, s));
  QX_CUDA_TRY(cudaStreamSynchronize(s));
  return QX_STATUS_OK;
}

// lowbit_pack, kernels/quantization/lowbit_ref.cpp:274-343 (int4 formats; HOST pointers)
qx_status qx_lowbit_pack(int format, const float* weights, uint8_t* packed, float* scales,
                         long long rows, long long dim, long long group_size) {
  Layout layout;
  if (!valid_product2(rows, dim) || !layout_for(format, dim, group_size, &layout)) return QX_STATUS_INVALID_SHAPE;
  if (weights == nullptr || packed == nullptr || scales == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  size_t w_bytes = 0, scale_count = 0;
  if (qx_lowbit_packed_size(format, rows, dim, group_size, &w_bytes, &scale_count) != QX_STATUS_OK) {
    return QX_STATUS_INVALID_SHAPE;
  }
  if (!int4_format(format)) return QX_STATUS_UNSUPPORTED_FORMAT;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  std::lock_guard<std::mutex> lock(ctx->mutex);
  const size_t f_bytes = static_cast<size_t>(rows) * dim * 4;
  const size_t off_f = 0, off_p = align_up(f_bytes, 256), off_s = off_p + align_up(w_bytes + 4, 256);
  QX_TRY(ctx->ensure_staging(off_s + align_up(scale_count * 4, 256)));
  uint8_t* base = static_cast<uint8_t*>(ctx->staging);
  cudaStream_t s = ctx->stream;
  QX_CUDA_TRY(cudaMemsetAsync(ctx->flag, 0, 4, s));
  QX_CUDA_TRY(cudaMemsetAsync(base + off_p, 0, align_up(w_bytes + 4, 256), s));
  QX_CUDA_TRY(cudaMemcpyAsync(base + off_f, weights, f_bytes, cudaMemcpyHostToDevice, s));
  const long long items = rows * layout.groups;
  int4_pack_kernel<<<static_cast<unsigned>((items + 7) / 8), 256, 0, s>>>(
      reinterpret_cast<const float*>(base + off_f), base + off_p, reinterpret_cast<float*>(base + off_s),
      rows, dim, layout.groups, layout.group_size, ctx->flag);
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  int bad = 0;
  QX_CUDA_TRY(cudaMemcpyAsync(&bad, ctx->flag, 4, cudaMemcpyDeviceToHost, s));
  QX_CUDA_TRY(cudaStreamSynchronize(s));
  if (bad != 0) return QX_STATUS_INVALID_ARGUMENT;  // non-finite weight
  QX_CUDA_TRY(cudaMemcpy(packed, base + off_p, w_bytes, cudaMemcpyDeviceToHost));
  QX_CUDA_TRY(cudaMemcpy(scales, base + off_s, scale_count * 4, cudaMemcpyDeviceToHost));
  return QX_STATUS_OK;
}

// lowbit_unpack, kernels/quantization/lowbit_ref.cpp:345-364 (int4 formats; HOST pointers)
qx_status qx_lowbit_unpack(int format, const uint8_t* packed, const float* scales, float* weights,
                           long long rows, long long dim, long long group_size) {
  Layout layout;
  QX_TRY(validate_lowbit(format, packed, scales, rows, dim, group_size, &layout));
  if (!finite_host(scales, rows * layout.groups)) return QX_STATUS_INVALID_ARGUMENT;
  if (weights == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  if (!int4_format(format)) return QX_STATUS_UNSUPPORTED_FORMAT;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  std::lock_guard<std::mutex> lock(ctx->mutex);
  const size_t w_bytes = static_cast<size_t>(rows) * layout.row_bytes, s_bytes = static_cast<size_t>(rows) * layout.groups * 4;
  const size_t f_bytes = static_cast<size_t>(rows) * dim * 4;
  const size_t off_p = 0, off_s = align_up(w_bytes, 256), off_f = off_s + align_up(s_bytes, 256);
  QX_TRY(ctx->ensure_staging(off_f + align_up(f_bytes, 256)));
  uint8_t* base = static_cast<uint8_t*>(ctx->staging);
  cudaStream_t s = ctx->stream;
  QX_CUDA_TRY(cudaMemcpyAsync(base + off_p, packed, w_bytes, cudaMemcpyHostToDevice, s));
  QX_CUDA_TRY(cudaMemcpyAsync(base + off_s, scales, s_bytes, cudaMemcpyHostToDevice, s));
  int4_unpack_kernel<<<static_cast<unsigned>((rows * dim + 255) / 256), 256, 0, s>>>(
      base + off_p, reinterpret_cast<const float*>(base + off_s), reinterpret_cast<float*>(base + off_f), rows,
      dim, layout.groups, layout.group_size);
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  QX_CUDA_TRY(cudaMemcpyAsync(weights, base + off_f, f_bytes, cudaMemcpyDeviceToHost, s));
  QX_CUDA_TRY(cudaStreamSynchronize(s));
  return QX_STATUS_OK;
}

}  // extern "C"
