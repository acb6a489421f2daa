// Canonical prepared projections for the integer layouts kInt8Symmetric, kInt4Symmetric and
// kUInt4Affine (zero points; GPTQ group index and act-order) with typed input / output, bias
// and activation epilogue, and the SmoothQuant, AWQ and GPTQ importers that produce such
// tensors.
//
// Replaces, for these layouts,
//   CpuPackedWeights::prepare(const CanonicalQuantTensor&)   src/memory/packed_weights.cpp:280-398
//   qgemm_prepacked_storage / qgemm_prepacked_epilogue_storage
//                                   kernels/quantization/qgemm_canonical.cpp:4460-4648
//   canonical_storage_panels (the portable schedule)         qgemm_canonical.cpp:2745-2863
//   store_projection_output / projection_activation          qgemm_canonical.cpp:361-379, 2570-2581
//   import_smoothquant_w8a8          kernels/quantization/quant_import_ref.cpp:1051-1116
//   import_awq_u4 / import_gptq_u4   kernels/quantization/quant_import_ref.cpp:840-999
//
// Arithmetic. The reference decodes a weight to f32 as scale * float(code) (one rounding,
// decode_prepared_chunk, qgemm_canonical.cpp:150-176) and multiplies it into one of four f32
// accumulators chosen by (column & 3); its AVX2 / NEON schedules order the same terms
// differently again, so its own test compares against a tolerance (4e-5 * (1 + |expected|))
// and so do this path's tests. Two paths here, both summing a lane's 16 columns first, scaling
// that partial sum by the weight scale once, and joining the 32 lane sums in a butterfly:
//   digits  (scale groups that are multiples of 16 columns, or one scale per row): the
//           activations of a span become exact 8-bit digits under a power-of-two envelope and
//           the sums are integer dot products; see "digit kernels" below;
//   floats  (a scale group boundary inside 16 columns, or a GPTQ group index): f32
//           multiply-adds on exactly converted codes, every weight decoded on its own as in
//           the reference (scale * code, or scale * (nibble - zero)).
// With an act-order map the activations are first gathered into packed column order.
//   tensor cores (int8 with one scale per row, five tokens or more): four digit planes under a
//           per-token envelope through the W8A8 GEMM; see "long prefills" below.
// Inputs stored as f16 / bf16 are widened exactly, the output is rounded once at the store.
// On the first two paths a token's result does not depend on the batch it is computed in; a
// batch that crosses five tokens changes route and with it the rounding (same tolerance).
//
// HBM layout. Codes stay in the canonical row-major byte order (a row of K int8 codes or
// K/2 nibble pairs is already what a warp wants to stream with 16-byte loads), followed by
// the f32 scale table [rows][groups]. Nothing is re-tiled, so prepared bytes = canonical
// bytes. The digit images of a call's activations (1792 bytes per token and 512 columns)
// live in the device's default workspace.
//
// Kernels. CUDA cores for decode-sized batches, the tcgen05 W8A8 GEMM for int8 prefills.
// Measured on 14336 x 4096 int8 with one bf16 token: 17 us per call for both launches (the
// digit kernel and the projection behind it), 3.4 TB/s of the weights' bytes, about half of
// the measured copy bandwidth; the float path ran the same shape in 24 us at 10 instructions
// per weight, bound by instruction issue.

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cmath>
#include <cstdlib>
#include <mutex>
#include <new>
#include <type_traits>
#include <vector>

#include "qx_common.cuh"
#include "qx_gemv.cuh"
#include "qx_int8_gemm.cuh"

struct qx_canonical_weights {
  int layout = 0;
  int scale_mode = 0;
  int device = -1;
  long long rows = 0;
  long long columns = 0;
  long long group_size = 0;     // columns per scale (== columns for row / channel scales)
  long long groups_per_row = 1;
  size_t data_bytes = 0;
  size_t scale_count = 0;
  uint8_t* data = nullptr;      // device: canonical codes
  float* scales = nullptr;      // device: [rows][groups_per_row]
  float* zeros = nullptr;       // device: [rows][groups_per_row] (kUInt4Affine), else null
  int* group_index = nullptr;   // device: [columns] packed column -> scale group, or null
  int* act_order = nullptr;     // device: [columns] packed column -> activation column, or null
  bool integral_zeros = false;  // every zero point is one of 0, 1, .. 15 (the usual case)
};

namespace qx {
namespace {

struct CanonicalParams {
  const uint8_t* data;
  const float* scales;
  const float* zeros;        // kUInt4Affine: zero point beside every scale
  const int* group_index;    // optional: packed column -> scale group
  int integral_zeros;        // every zero point is one of 0 .. 15: exact integer arithmetic
  const void* x;
  const float* bias;
  void* y;
  long long rows, columns, group_size, groups_per_row, m;
  long long ldy;     // row stride of y in elements (the tensor-core route; rows elsewhere)
  int x_type, y_type, activation;
  int vector_rows;   // 1: every row of codes starts on a 16-byte (int8) / 8-byte (int4) boundary
  int vector_x;      // 1: every activation row starts on a boundary of four elements
};

__device__ __forceinline__ float load_storage(const void* base, int type, long long index) {
  if (type == QX_STORAGE_F32) return static_cast<const float*>(base)[index];
  const uint16_t bits = static_cast<const uint16_t*>(base)[index];
  if (type == QX_STORAGE_F16) return __half2float(__ushort_as_half(bits));
  return __uint_as_float(static_cast<uint32_t>(bits) << 16);
}

// float_to_bf16 of the reference (kernels/utils/float_storage_ref.cpp:184-193): round to
// nearest even on the bit pattern; a NaN keeps its upper payload with the quiet bit set.
__device__ __forceinline__ uint16_t to_bf16_bits(float value) {
  const uint32_t bits = __float_as_uint(value);
  if ((bits & 0x7f800000u) == 0x7f800000u && (bits & 0x007fffffu) != 0) {
    return static_cast<uint16_t>((bits >> 16) | 0x0040u);
  }
  return static_cast<uint16_t>((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
}

__device__ __forceinline__ void store_storage(void* base, int type, long long index, float value) {
  if (type == QX_STORAGE_F32) {
    static_cast<float*>(base)[index] = value;
  } else if (type == QX_STORAGE_F16) {
    static_cast<uint16_t*>(base)[index] = __half_as_ushort(__float2half_rn(value));
  } else {
    static_cast<uint16_t*>(base)[index] = to_bf16_bits(value);
  }
}

// projection_activation, qgemm_canonical.cpp:361-379
__device__ __forceinline__ float apply_activation(float v, int activation) {
  switch (activation) {
    case QX_ACTIVATION_GELU_ERF:
      return 0.5f * v * (1.0f + erff(v * 0.7071067811865475f));
    case QX_ACTIVATION_GELU_TANH:
      return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    case QX_ACTIVATION_SILU:
      return v / (1.0f + expf(-v));
    case QX_ACTIVATION_RELU2:
      return v > 0.0f ? v * v : 0.0f;
    default:
      return v;
  }
}

// A lane owns 16 consecutive columns per K chunk (one 16-byte load of int8 codes, one 8-byte
// load of int4 codes); a chunk is 32 lanes x 16 = 512 columns, i.e. 128 float4 units of
// activations per token.
constexpr int kElems = 16;
constexpr int kChunk = 32 * kElems;
constexpr int kUnits = kChunk / 4;

struct LaneCodes {
  uint32_t w[4];  // int8: four words of four codes; int4: w[0], w[1] hold eight nibbles each
};

// The four codes of float4 group j (columns 4j .. 4j+3 of the lane's span) as floats, without
// the integer-to-float unit: a code is moved into the mantissa of 2^23 and the offset is
// subtracted, which is exact. int8: byte ^ 0x80 = code + 128; int4: nibble ^ 8 = code + 8
// (n >= 8 means n - 16), the lower column in the low nibble.
template <int LAYOUT>
__device__ __forceinline__ void decode4(const LaneCodes& codes, int j, float (&f)[4]) {
  if (LAYOUT == QX_CANONICAL_INT8_SYMMETRIC) {
    const uint32_t word = codes.w[j] ^ 0x80808080u;
    f[0] = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7440)) - 8388736.0f;
    f[1] = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7441)) - 8388736.0f;
    f[2] = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7442)) - 8388736.0f;
    f[3] = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7443)) - 8388736.0f;
  } else {
    // symmetric: nibble ^ 8 = code + 8; affine: the nibble itself, 0 .. 15
    constexpr bool kSigned = LAYOUT == QX_CANONICAL_INT4_SYMMETRIC;
    constexpr float kOffset = kSigned ? 8388616.0f : 8388608.0f;
    const uint32_t word = kSigned ? codes.w[j >> 1] ^ 0x88888888u : codes.w[j >> 1];
    const uint32_t lo = word & 0x0F0F0F0Fu, hi = (word >> 4) & 0x0F0F0F0Fu;
    if ((j & 1) == 0) {
      f[0] = __uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7440)) - kOffset;
      f[1] = __uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7440)) - kOffset;
      f[2] = __uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7441)) - kOffset;
      f[3] = __uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7441)) - kOffset;
    } else {
      f[0] = __uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7442)) - kOffset;
      f[1] = __uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7442)) - kOffset;
      f[2] = __uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7443)) - kOffset;
      f[3] = __uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7443)) - kOffset;
    }
  }
}

// Codes of columns k_lane .. k_lane + 15 of one row; `src` points at the row's byte for
// column k_lane. Columns at or past `columns` stay zero.
template <int LAYOUT>
__device__ __forceinline__ LaneCodes load_codes(const uint8_t* src, bool vector, int k_lane,
                                                int columns) {
  LaneCodes out = {{0u, 0u, 0u, 0u}};
  if (vector && k_lane + kElems <= columns) {
    if (LAYOUT == QX_CANONICAL_INT8_SYMMETRIC) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(src));
      out.w[0] = v.x; out.w[1] = v.y; out.w[2] = v.z; out.w[3] = v.w;
    } else {
      const uint2 v = __ldg(reinterpret_cast<const uint2*>(src));
      out.w[0] = v.x; out.w[1] = v.y;
    }
    return out;
  }
  // ragged tail or rows that do not start on a vector boundary: byte by byte
  const int left = columns - k_lane;
  const int span = left < kElems ? left : kElems;
  const int bytes = LAYOUT == QX_CANONICAL_INT8_SYMMETRIC ? span : (span + 1) / 2;
  uint32_t w0 = 0u, w1 = 0u, w2 = 0u, w3 = 0u;
  for (int b = 0; b < bytes; ++b) {
    const uint32_t v = static_cast<uint32_t>(src[b]) << (8 * (b & 3));
    if (b < 4) w0 |= v; else if (b < 8) w1 |= v; else if (b < 12) w2 |= v; else w3 |= v;
  }
  out.w[0] = w0; out.w[1] = w1; out.w[2] = w2; out.w[3] = w3;
  return out;  // a zero code decodes to zero in both layouts
}

// Four activations starting at element `index` (column k of a token's row), widened to f32.
__device__ __forceinline__ float4 load_x4(const CanonicalParams& p, long long index, int k,
                                          int columns) {
  if (p.vector_x && k + 4 <= columns) {
    if (p.x_type == QX_STORAGE_F32) return __ldg(reinterpret_cast<const float4*>(p.x) + (index >> 2));
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p.x) + (index >> 2));
    if (p.x_type == QX_STORAGE_F16) {
      const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
      const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
      return make_float4(lo.x, lo.y, hi.x, hi.y);
    }
    return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                       __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
  }
  float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    if (k + c < columns) v[c] = load_storage(p.x, p.x_type, index + c);
  }
  return make_float4(v[0], v[1], v[2], v[3]);
}

template <int LAYOUT, int TM, int ROWS, int WARPS>
__global__ void __launch_bounds__(32 * WARPS) canonical_gemm_kernel(const CanonicalParams p) {
  constexpr bool kInt8 = LAYOUT == QX_CANONICAL_INT8_SYMMETRIC;
  constexpr int kThreadsHere = 32 * WARPS;
  constexpr int kUnitsPerThread = (TM * kUnits + kThreadsHere - 1) / kThreadsHere;
  // two buffers of the chunk's activations: float4 unit (token, group g of lane `owner`) sits
  // at [token][g * 32 + owner], so that the 32 lanes read 32 consecutive float4
  __shared__ float4 xs[2][TM][kUnits];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int columns = static_cast<int>(p.columns);
  const long long row0 = (static_cast<long long>(blockIdx.x) * WARPS + warp) * ROWS;
  const long long token0 = static_cast<long long>(blockIdx.y) * TM;
  const int tokens = static_cast<int>(p.m - token0 < TM ? p.m - token0 : TM);
  const int group_size = static_cast<int>(p.group_size);
  const int chunks = (columns + kChunk - 1) / kChunk;

  // per row: where this lane's codes of chunk 0 start, and the row of the scale table
  const uint8_t* code_ptr[ROWS];
  const float* scale_row[ROWS];
  const float* zero_row[ROWS];
  bool row_ok[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const long long row = row0 + r;
    row_ok[r] = row < p.rows;
    const long long safe = row_ok[r] ? row : 0;
    code_ptr[r] = p.data + safe * (kInt8 ? p.columns : p.columns / 2) + lane * (kInt8 ? kElems : kElems / 2);
    scale_row[r] = p.scales + safe * p.groups_per_row;
    zero_row[r] = LAYOUT == QX_CANONICAL_UINT4_AFFINE ? p.zeros + safe * p.groups_per_row : nullptr;
  }
  // per staged unit of this thread: element index of chunk 0 and the shared-memory slot
  long long x_index[kUnitsPerThread];
  int x_column[kUnitsPerThread];  // column of chunk 0, or a column past the end when unused
  int x_slot[kUnitsPerThread];
#pragma unroll
  for (int i = 0; i < kUnitsPerThread; ++i) {
    const int u = threadIdx.x + i * kThreadsHere;
    const int token = u / kUnits, q = u % kUnits;
    const bool used = u < TM * kUnits && token < tokens;
    x_column[i] = used ? 4 * q : 0x40000000;
    x_index[i] = (token0 + (used ? token : 0)) * p.columns + 4 * q;
    x_slot[i] = u < TM * kUnits ? token * kUnits + (q & 3) * 32 + (q >> 2) : -1;
  }

  float acc[ROWS][TM];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
#pragma unroll
    for (int t = 0; t < TM; ++t) acc[r][t] = 0.0f;
  }

  LaneCodes codes[ROWS];
  float4 xr[kUnitsPerThread];
  auto fetch = [&](int chunk, LaneCodes (&into)[ROWS]) {
    const int k0 = chunk * kChunk;
    const int k_lane = k0 + lane * kElems;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      if (row_ok[r] && k_lane < columns) {
        into[r] = load_codes<LAYOUT>(code_ptr[r] + (kInt8 ? k0 : k0 / 2), p.vector_rows != 0,
                                     k_lane, columns);
      } else {
        into[r] = LaneCodes{{0u, 0u, 0u, 0u}};
      }
    }
#pragma unroll
    for (int i = 0; i < kUnitsPerThread; ++i) {
      xr[i] = x_column[i] + k0 < columns
                  ? load_x4(p, x_index[i] + k0, x_column[i] + k0, columns)
                  : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
  };
  fetch(0, codes);

  for (int chunk = 0; chunk < chunks; ++chunk) {
    float4* buf = &xs[chunk & 1][0][0];
#pragma unroll
    for (int i = 0; i < kUnitsPerThread; ++i) {
      if (x_slot[i] >= 0) buf[x_slot[i]] = xr[i];
    }
    // One barrier per chunk: a warp that writes buffer (chunk + 1) & 1 next has passed this
    // barrier, so every warp has finished the math of chunk - 1, the last reader of that buffer.
    __syncthreads();
    LaneCodes next_codes[ROWS];
    if (chunk + 1 < chunks) fetch(chunk + 1, next_codes);  // in flight under the math
    {
      // every weight is decoded on its own, as the reference does it: scale * float(code), or
      // scale * (float(nibble) - zero) for the affine layout (qgemm_canonical.cpp:150-176), the
      // group of a column from group_index when the tensor has one (scale_index, :86-115)
      const int k_lane = chunk * kChunk + lane * kElems;
#pragma unroll
      for (int j = 0; j < kElems / 4; ++j) {
        float4 xv[TM];
#pragma unroll
        for (int t = 0; t < TM; ++t) xv[t] = buf[t * kUnits + j * 32 + lane];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          float f[4];
          decode4<LAYOUT>(codes[r], j, f);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int k = k_lane + 4 * j + c;
            float s = 0.0f, z = 0.0f;
            if (row_ok[r] && k < columns) {
              const int group = p.group_index != nullptr ? p.group_index[k]
                                                         : (p.groups_per_row == 1 ? 0 : k / group_size);
              s = scale_row[r][group];
              if (LAYOUT == QX_CANONICAL_UINT4_AFFINE) z = zero_row[r][group];
            }
            f[c] = __fmul_rn(s, LAYOUT == QX_CANONICAL_UINT4_AFFINE ? __fsub_rn(f[c], z) : f[c]);
          }
#pragma unroll
          for (int t = 0; t < TM; ++t) {
            acc[r][t] = fmaf(f[0], xv[t].x, acc[r][t]);
            acc[r][t] = fmaf(f[1], xv[t].y, acc[r][t]);
            acc[r][t] = fmaf(f[2], xv[t].z, acc[r][t]);
            acc[r][t] = fmaf(f[3], xv[t].w, acc[r][t]);
          }
        }
      }
    }
    if (chunk + 1 < chunks) {
#pragma unroll
      for (int r = 0; r < ROWS; ++r) codes[r] = next_codes[r];
    }
  }

  // ---- the 32 partial sums of an output meet in a butterfly; lane (r * TM + t) % 32 stores it
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
#pragma unroll
    for (int t = 0; t < TM; ++t) {
      float v = acc[r][t];
#pragma unroll
      for (int h = 16; h >= 1; h >>= 1) v += __shfl_xor_sync(0xffffffffu, v, h);
      const long long row = row0 + r;
      if (lane == ((r * TM + t) & 31) && row_ok[r] && t < tokens) {
        if (p.bias != nullptr) v += p.bias[row];
        v = apply_activation(v, p.activation);
        store_storage(p.y, p.y_type, (token0 + t) * p.rows + row, v);
      }
    }
  }
}

// ---- digit kernels: the path of every tensor whose scale groups are multiples of 16 columns
//
// Activation digits. Per token and per span of 16 columns (one lane's columns of a chunk) the
// activations are written as 23-bit signed fixed point under the span's power-of-two
// envelope, x = e * t with |t| <= 2^22, and t is split into balanced base-256 digits
// t = 65536 * p2 + 256 * p1 + p0, each a signed byte. A span's dot product with 16 integer
// codes is then three exact integer dot products per four columns (dp4a), combined once per
// span in f32 and multiplied by e and by the weight scale: about one instruction per weight
// instead of the three or four of a float multiply-add on a decoded weight, which is what
// lets a single token run at memory speed. The only rounding on the activation side is the
// fixed-point step, at most 2^-23 of the span's envelope per element -- of the order of one
// f32 rounding in the reference's own sum; the integer sums are exact.
//
// A small kernel in front writes the digits of all tokens once per call (a few KB per token,
// read back by every warp through L1 / L2); the projection kernel is launched as its
// programmatic dependent: it fetches its first codes while the digits are still being
// written and waits for them itself.
//
// int4 without sign extension: a nibble n (meaning n - 16 when n >= 8) xor 8 is the unsigned
// u = code + 8, so sum(code * t) = sum(u * t) - 8 * sum(t); sum(t) of the span is stored with
// the digits. The even and odd nibbles of a word are two masked operands, and the digit
// words of a span are stored in that order (even columns of a word, then odd).
//
// Digit image of one (token, chunk): three planes of 128 words (word = span * 4 + g), then
// 32 envelopes, then 32 span sums.
constexpr int kImageWords = 3 * 128 + 32 + 32;

template <int LAYOUT>
__global__ void __launch_bounds__(128) canonical_digits_prepass(const CanonicalParams p,
                                                                uint32_t* __restrict__ image) {
  // Let the projection kernel behind start (it fetches weights first), then wait for the
  // work in front: the activations may be its output, and the projection of the previous
  // call may still be reading the images this kernel overwrites.
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  constexpr bool kInt8 = LAYOUT == QX_CANONICAL_INT8_SYMMETRIC;
  const int columns = static_cast<int>(p.columns);
  const int chunks = (columns + kChunk - 1) / kChunk;
  const int chunk = blockIdx.x % chunks;
  const long long token = blockIdx.x / chunks;
  const int word = threadIdx.x;  // span * 4 + g
  const int span_k = chunk * kChunk + (word >> 2) * kElems;
  const int g = word & 3;
  float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  if (span_k < columns) {
    const long long base = token * p.columns;
    if (kInt8) {
      v = load_x4(p, base + span_k + 4 * g, span_k + 4 * g, columns);
    } else {
      // even (g & 1 == 0) or odd columns of the eight columns of code word g >> 1
      const int k8 = span_k + 8 * (g >> 1);
      const float4 a = load_x4(p, base + k8, k8, columns);
      const float4 b = load_x4(p, base + k8 + 4, k8 + 4, columns);
      v = (g & 1) ? make_float4(a.y, a.w, b.y, b.w) : make_float4(a.x, a.z, b.x, b.z);
    }
  }
  // the span's largest magnitude: the four words of a span sit in four adjacent lanes
  float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
  // fmaxf drops a NaN operand: the sum of magnitudes keeps it
  if (!(fabsf(v.x) + fabsf(v.y) + fabsf(v.z) + fabsf(v.w) < __uint_as_float(0x7f800000u))) {
    amax = __uint_as_float(0x7f800000u);
  }
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  // envelope 2^E > amax; t = x * 2^22 / 2^E. Spans below 2^-103 count as zero; a NaN or
  // infinity makes the envelope NaN, which reaches every output of the token.
  int biased = static_cast<int>(__float_as_uint(amax) >> 23) + 1;  // exponent of 2^E
  biased = biased < 24 ? 24 : biased;
  const bool finite = biased < 256;
  const float to_fixed = finite ? __uint_as_float(static_cast<uint32_t>(276 - biased) << 23) : 0.0f;
  const float e = finite ? __uint_as_float(static_cast<uint32_t>(biased - 22) << 23)
                         : __uint_as_float(0x7fc00000u);
  const float xs[4] = {v.x, v.y, v.z, v.w};
  uint32_t w0 = 0u, w1 = 0u, w2 = 0u;
  int tsum = 0;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int t = finite ? __float2int_rn(xs[c] * to_fixed) : 0;
    const int p0 = ((t + 128) & 255) - 128;
    const int t1 = (t - p0) >> 8;
    const int p1 = ((t1 + 128) & 255) - 128;
    const int p2 = (t1 - p1) >> 8;
    w0 |= static_cast<uint32_t>(p0 & 255) << (8 * c);
    w1 |= static_cast<uint32_t>(p1 & 255) << (8 * c);
    w2 |= static_cast<uint32_t>(p2 & 255) << (8 * c);
    tsum += t;
  }
  tsum += __shfl_xor_sync(0xffffffffu, tsum, 1);
  tsum += __shfl_xor_sync(0xffffffffu, tsum, 2);
  uint32_t* out = image + static_cast<long long>(blockIdx.x) * kImageWords;
  out[word] = w0;
  out[128 + word] = w1;
  out[256 + word] = w2;
  if (g == 0) {
    out[384 + (word >> 2)] = __float_as_uint(e);
    out[416 + (word >> 2)] = static_cast<uint32_t>(tsum);
  }
}

// One (token, chunk) image as a lane uses it: its span's four digit words of every plane.
struct SpanDigits {
  uint4 d0, d1, d2;
  float e;
  int tsum;
};
__device__ __forceinline__ SpanDigits load_span(const uint32_t* image, int lane) {
  SpanDigits s;
  s.d0 = __ldg(reinterpret_cast<const uint4*>(image) + lane);
  s.d1 = __ldg(reinterpret_cast<const uint4*>(image + 128) + lane);
  s.d2 = __ldg(reinterpret_cast<const uint4*>(image + 256) + lane);
  s.e = __uint_as_float(__ldg(image + 384 + lane));
  s.tsum = static_cast<int>(__ldg(image + 416 + lane));
  return s;
}

// sum over the lane's 16 columns of code * t from the digit words; w: the span's four code
// words (int8), or its even / odd nibble words after the xor with 8 (int4)
template <int LAYOUT>
__device__ __forceinline__ float span_dot(const uint32_t (&w)[4], const uint4& d0, const uint4& d1,
                                          const uint4& d2, int tsum, float zero, bool integral_zero) {
  if (LAYOUT == QX_CANONICAL_INT8_SYMMETRIC) {
    int s0 = dp4a_ss(w[0], d0.x, 0), s1 = dp4a_ss(w[0], d1.x, 0), s2 = dp4a_ss(w[0], d2.x, 0);
    s0 = dp4a_ss(w[1], d0.y, s0); s1 = dp4a_ss(w[1], d1.y, s1); s2 = dp4a_ss(w[1], d2.y, s2);
    s0 = dp4a_ss(w[2], d0.z, s0); s1 = dp4a_ss(w[2], d1.z, s1); s2 = dp4a_ss(w[2], d2.z, s2);
    s0 = dp4a_ss(w[3], d0.w, s0); s1 = dp4a_ss(w[3], d1.w, s1); s2 = dp4a_ss(w[3], d2.w, s2);
    return block_sum(s0, s1, s2);  // |s_d| <= 16 * 128 * 128 < 2^21
  }
  int s0 = dp4a_us(w[0], d0.x, 0), s1 = dp4a_us(w[0], d1.x, 0), s2 = dp4a_us(w[0], d2.x, 0);
  s0 = dp4a_us(w[1], d0.y, s0); s1 = dp4a_us(w[1], d1.y, s1); s2 = dp4a_us(w[1], d2.y, s2);
  s0 = dp4a_us(w[2], d0.z, s0); s1 = dp4a_us(w[2], d1.z, s1); s2 = dp4a_us(w[2], d2.z, s2);
  s0 = dp4a_us(w[3], d0.w, s0); s1 = dp4a_us(w[3], d1.w, s1); s2 = dp4a_us(w[3], d2.w, s2);
  // sum(u * t): |.| <= 16 * 15 * 2^22 < 2^30, exact in int32
  const int ut = (s2 << 16) + (s1 << 8) + s0;
  if (LAYOUT == QX_CANONICAL_INT4_SYMMETRIC || LAYOUT == 3 /* kLayoutInt4Offset8 */) {
    return __int2float_rn(ut - 8 * tsum);  // u = code + 8
  }
  // affine: sum((u - zero) * t) = sum(u * t) - zero * sum(t); exact in int32 when the tensor's
  // zero points are the usual integers 0 .. 15 (|.| < 2^31), in f32 otherwise
  if (integral_zero) return __int2float_rn(ut - __float2int_rn(zero) * tsum);
  return fmaf(-zero, __int2float_rn(tsum), __int2float_rn(ut));
}

// Internal fourth layout of the digit kernels: adjacent nibbles meaning nibble - 8 (the compact
// int4 rows of lowbit_gemm, kernels/quantization/lowbit_ref.cpp:229-256): the symmetric path
// without the xor.
constexpr int kLayoutInt4Offset8 = 3;

constexpr int kDigitWarps = 4;  // independent warps per CTA: no shared memory, no barrier
constexpr int kStep = 1;       // chunks a lane requests at once (measured: 1 is as fast as 4)

template <int LAYOUT, int TM, int ROWS>
__global__ void __launch_bounds__(32 * kDigitWarps) canonical_digits_kernel(
    const CanonicalParams p, const uint32_t* __restrict__ image) {
  constexpr bool kInt8 = LAYOUT == QX_CANONICAL_INT8_SYMMETRIC;
  constexpr bool kAffine = LAYOUT == QX_CANONICAL_UINT4_AFFINE;
  constexpr uint32_t kNibbleXor = LAYOUT == QX_CANONICAL_INT4_SYMMETRIC ? 0x88888888u : 0u;
  const bool integral = p.integral_zeros != 0;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int columns = static_cast<int>(p.columns);
  const long long row0 = (static_cast<long long>(blockIdx.x) * kDigitWarps + warp) * ROWS;
  const long long token0 = static_cast<long long>(blockIdx.y) * TM;
  const int tokens = static_cast<int>(p.m - token0 < TM ? p.m - token0 : TM);
  const int group_size = static_cast<int>(p.group_size);
  const int chunks = (columns + kChunk - 1) / kChunk;

  const uint8_t* code_ptr[ROWS];
  const float* scale_row[ROWS];
  const float* zero_row[ROWS];
  bool row_ok[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const long long row = row0 + r;
    row_ok[r] = row < p.rows;
    const long long safe = row_ok[r] ? row : 0;
    code_ptr[r] = p.data + safe * (kInt8 ? p.columns : p.columns / 2) + lane * (kInt8 ? kElems : kElems / 2);
    scale_row[r] = p.scales + safe * p.groups_per_row;
    zero_row[r] = kAffine ? p.zeros + safe * p.groups_per_row : nullptr;
  }
  // the images of this CTA's tokens: [token][chunk]
  const uint32_t* token_image[TM];
#pragma unroll
  for (int t = 0; t < TM; ++t) {
    token_image[t] = image + (token0 + (t < tokens ? t : 0)) * chunks * kImageWords;
  }

  // A step is kStep consecutive chunks: a lane requests its 16 bytes of each of them at once.
  auto fetch_codes = [&](int step, LaneCodes (&into)[kStep][ROWS], float (&scales)[kStep][ROWS],
                         float (&zeros)[kStep][ROWS]) {
#pragma unroll
    for (int u = 0; u < kStep; ++u) {
      const int k0 = (step * kStep + u) * kChunk;
      const int k_lane = k0 + lane * kElems;
      const int group = p.groups_per_row == 1 ? 0 : k_lane / group_size;
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        zeros[u][r] = 0.0f;
        if (row_ok[r] && k_lane < columns) {
          into[u][r] = load_codes<LAYOUT>(code_ptr[r] + (kInt8 ? k0 : k0 / 2), p.vector_rows != 0,
                                          k_lane, columns);
          scales[u][r] = __ldg(scale_row[r] + group);
          if (kAffine) zeros[u][r] = __ldg(zero_row[r] + group);
        } else {
          into[u][r] = LaneCodes{{0u, 0u, 0u, 0u}};
          scales[u][r] = 0.0f;
        }
      }
    }
  };

  float acc[ROWS][TM];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
#pragma unroll
    for (int t = 0; t < TM; ++t) acc[r][t] = 0.0f;
  }
  // Whole rows, whole chunks, vector loads: the common shape, without a predicate in the loop.
  if (p.vector_rows != 0 && row0 + ROWS <= p.rows && columns % kChunk == 0) {
    using Vec = typename std::conditional<kInt8, uint4, uint2>::type;
    const Vec* vec_ptr[ROWS];
    float row_scale[ROWS], row_zero[ROWS];
    const bool single = p.groups_per_row == 1;
    const int spans_per_group = single ? 1 : group_size / kElems;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      vec_ptr[r] = reinterpret_cast<const Vec*>(code_ptr[r]);
      row_scale[r] = single ? __ldg(scale_row[r]) : 0.0f;
      row_zero[r] = (single && kAffine) ? __ldg(zero_row[r]) : 0.0f;
    }
    Vec current[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) current[r] = __ldg(vec_ptr[r]);  // independent of the kernel in front
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int chunk = 0; chunk < chunks; ++chunk) {
      Vec next[ROWS];
      if (chunk + 1 < chunks) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) next[r] = __ldg(vec_ptr[r] + (chunk + 1) * 32);
      }
      float s[ROWS], z[ROWS];
      if (single) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          s[r] = row_scale[r];
          z[r] = row_zero[r];
        }
      } else {
        const int group = (chunk * 32 + lane) / spans_per_group;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          s[r] = __ldg(scale_row[r] + group);
          z[r] = kAffine ? __ldg(zero_row[r] + group) : 0.0f;
        }
      }
      uint32_t w[ROWS][4];
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        if constexpr (kInt8) {
          w[r][0] = current[r].x; w[r][1] = current[r].y; w[r][2] = current[r].z; w[r][3] = current[r].w;
        } else {
          const uint32_t a = current[r].x ^ kNibbleXor, b = current[r].y ^ kNibbleXor;
          w[r][0] = a & 0x0F0F0F0Fu; w[r][1] = (a >> 4) & 0x0F0F0F0Fu;
          w[r][2] = b & 0x0F0F0F0Fu; w[r][3] = (b >> 4) & 0x0F0F0F0Fu;
        }
      }
#pragma unroll
      for (int t = 0; t < TM; ++t) {
        const SpanDigits span = load_span(token_image[t] + chunk * kImageWords, lane);
        const float e = t < tokens ? span.e : 0.0f;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          acc[r][t] = fmaf(s[r] * e, span_dot<LAYOUT>(w[r], span.d0, span.d1, span.d2, span.tsum, z[r], integral),
                           acc[r][t]);
        }
      }
      if (chunk + 1 < chunks) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) current[r] = next[r];
      }
    }
  } else {
  LaneCodes codes[kStep][ROWS];
  float scale[kStep][ROWS], zero[kStep][ROWS];
  fetch_codes(0, codes, scale, zero);  // weights do not depend on the kernel in front
  asm volatile("griddepcontrol.wait;" ::: "memory");

  const int steps = (chunks + kStep - 1) / kStep;
  for (int step = 0; step < steps; ++step) {
    const bool more = step + 1 < steps;
    LaneCodes next_codes[kStep][ROWS];
    float next_scale[kStep][ROWS], next_zero[kStep][ROWS];
    if (more) fetch_codes(step + 1, next_codes, next_scale, next_zero);  // HBM loads in flight under the math
#pragma unroll
    for (int u = 0; u < kStep; ++u) {
      const int chunk = step * kStep + u;
      if (chunk < chunks) {
        if (!kInt8) {
          // split every code word into its even and odd nibbles
#pragma unroll
          for (int r = 0; r < ROWS; ++r) {
            const uint32_t a = codes[u][r].w[0] ^ kNibbleXor, b = codes[u][r].w[1] ^ kNibbleXor;
            codes[u][r].w[0] = a & 0x0F0F0F0Fu;
            codes[u][r].w[1] = (a >> 4) & 0x0F0F0F0Fu;
            codes[u][r].w[2] = b & 0x0F0F0F0Fu;
            codes[u][r].w[3] = (b >> 4) & 0x0F0F0F0Fu;
          }
        }
#pragma unroll
        for (int t = 0; t < TM; ++t) {
          const SpanDigits span = load_span(token_image[t] + chunk * kImageWords, lane);
          const uint4 d0 = span.d0, d1 = span.d1, d2 = span.d2;
          const float e = t < tokens ? span.e : 0.0f;
#pragma unroll
          for (int r = 0; r < ROWS; ++r) {
            const float sum = span_dot<LAYOUT>(codes[u][r].w, d0, d1, d2, span.tsum, zero[u][r], integral);
            acc[r][t] = fmaf(scale[u][r] * e, sum, acc[r][t]);
          }
        }
      }
    }
    if (more) {
#pragma unroll
      for (int u = 0; u < kStep; ++u) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          codes[u][r] = next_codes[u][r];
          scale[u][r] = next_scale[u][r];
          zero[u][r] = next_zero[u][r];
        }
      }
    }
  }

  }  // general path

  // ---- the 32 span sums of an output meet in a butterfly; lane (r * TM + t) % 32 stores it
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
#pragma unroll
    for (int t = 0; t < TM; ++t) {
      float v = acc[r][t];
#pragma unroll
      for (int h = 16; h >= 1; h >>= 1) v += __shfl_xor_sync(0xffffffffu, v, h);
      const long long row = row0 + r;
      if (lane == ((r * TM + t) & 31) && row_ok[r] && t < tokens) {
        if (p.bias != nullptr) v += p.bias[row];
        v = apply_activation(v, p.activation);
        store_storage(p.y, p.y_type, (token0 + t) * p.rows + row, v);
      }
    }
  }
}

// bytes of digit images of a call
size_t digit_image_bytes(long long m, long long columns) {
  const long long chunks = (columns + kChunk - 1) / kChunk;
  return static_cast<size_t>(m) * static_cast<size_t>(chunks) * kImageWords * sizeof(uint32_t);
}

template <int LAYOUT, int TM, int ROWS>
qx_status launch_digits_one(const CanonicalParams& p, const uint32_t* image, cudaStream_t stream) {
  const long long gx = (p.rows + kDigitWarps * ROWS - 1) / (kDigitWarps * ROWS);
  const long long gy = (p.m + TM - 1) / TM;
  if (gx > 0x7fffffffLL || gy > 65535) {
    set_last_error_text("canonical projection: shape too large for one launch");
    return QX_STATUS_INVALID_SHAPE;
  }
  // programmatic dependent of the digit kernel in front: waits for it itself
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
  config.blockDim = dim3(32 * kDigitWarps);
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  QX_CUDA_TRY(cudaLaunchKernelEx(&config, canonical_digits_kernel<LAYOUT, TM, ROWS>, p, image));
  count_launch();
  return QX_STATUS_OK;
}

template <int LAYOUT, int TM>
qx_status launch_digits_tokens(const CanonicalParams& p, const uint32_t* image, int sm_count,
                               cudaStream_t stream) {
  // Two rows per warp: measured on 14336 x 4096 and 4096 x 4096 with 1 and 8 tokens, the more
  // warps the better (17.1 us against 18.5 us with four rows for one token, 20.6 against 21.9
  // for eight).
  (void)sm_count;
  int rows = 2;
  // developer switch: QX_B200_CANONICAL_ROWS=2|4
  if (const char* forced = std::getenv("QX_B200_CANONICAL_ROWS")) {
    const int asked = forced[0] - '0';
    if (asked == 2 || asked == 4) rows = asked;
  }
  if (rows == 4) return launch_digits_one<LAYOUT, TM, 4>(p, image, stream);
  return launch_digits_one<LAYOUT, TM, 2>(p, image, stream);
}

template <int LAYOUT>
qx_status launch_digits(const CanonicalParams& p, uint32_t* image, int sm_count,
                        cudaStream_t stream) {
  const long long chunks = (p.columns + kChunk - 1) / kChunk;
  const long long blocks = p.m * chunks;
  if (blocks > 0x7fffffffLL) {
    set_last_error_text("canonical projection: too many tokens for one launch");
    return QX_STATUS_INVALID_SHAPE;
  }
  {
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(static_cast<unsigned>(blocks));
    config.blockDim = dim3(128);
    config.stream = stream;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    QX_CUDA_TRY(cudaLaunchKernelEx(&config, canonical_digits_prepass<LAYOUT>, p, image));
    count_launch();
  }
  if (p.m == 1) return launch_digits_tokens<LAYOUT, 1>(p, image, sm_count, stream);
  if (p.m == 2) return launch_digits_tokens<LAYOUT, 2>(p, image, sm_count, stream);
  return launch_digits_tokens<LAYOUT, 4>(p, image, sm_count, stream);
}

template <int LAYOUT, int TM, int ROWS, int WARPS>
qx_status launch_one(const CanonicalParams& p, cudaStream_t stream) {
  const long long gx = (p.rows + WARPS * ROWS - 1) / (WARPS * ROWS);
  const long long gy = (p.m + TM - 1) / TM;
  if (gx > 0x7fffffffLL || gy > 65535) {
    set_last_error_text("canonical projection: shape too large for one launch");
    return QX_STATUS_INVALID_SHAPE;
  }
  canonical_gemm_kernel<LAYOUT, TM, ROWS, WARPS>
      <<<dim3(static_cast<unsigned>(gx), static_cast<unsigned>(gy)), 32 * WARPS, 0, stream>>>(p);
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  return QX_STATUS_OK;
}

// The float path is the rare one (a scale group boundary inside 16 columns, or a GPTQ group
// index): one tile shape, two rows per warp and four warps per CTA, which measured best or
// close to it on every shape tried when this kernel still served all tensors.
template <int LAYOUT, int TM>
qx_status launch_tokens(const CanonicalParams& p, int /*sm_count*/, cudaStream_t stream) {
  return launch_one<LAYOUT, TM, 2, 4>(p, stream);
}

template <int LAYOUT>
qx_status launch_layout(const CanonicalParams& p, int sm_count, cudaStream_t stream) {
  if (p.m == 1) return launch_tokens<LAYOUT, 1>(p, sm_count, stream);
  if (p.m <= 4) return launch_tokens<LAYOUT, 4>(p, sm_count, stream);
  return launch_tokens<LAYOUT, 8>(p, sm_count, stream);
}

bool known_storage(int type) {
  return type == QX_STORAGE_F32 || type == QX_STORAGE_F16 || type == QX_STORAGE_BF16;
}
size_t storage_bytes(int type) { return type == QX_STORAGE_F32 ? 4 : 2; }
bool known_activation(int activation) {
  return activation >= QX_ACTIVATION_NONE && activation <= QX_ACTIVATION_RELU2;
}

// GPTQ act-order: packed column k of the weights multiplies activation column order[k]
// (canonical_storage_panels, qgemm_canonical.cpp:2823-2840). The activations are gathered
// once per call into packed order (f32), so that the kernels read them in order.
__global__ void __launch_bounds__(256) gather_activations_kernel(const void* __restrict__ x,
                                                                 int x_type,
                                                                 const int* __restrict__ order,
                                                                 float* __restrict__ out,
                                                                 long long columns) {
  const long long token = blockIdx.y;
  for (long long k = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x; k < columns;
       k += 256LL * gridDim.x) {
    out[token * columns + k] = load_storage(x, x_type, token * columns + order[k]);
  }
}

// ---- five tokens or more of int8 tensors with one scale per row: the tensor cores ----------
// (Measured on 14336 x 4096 / 4096 x 4096: 4 tokens 23.7 / 18.1 us here against 34.4 / 14.8 us
// on the digit kernel, 8 tokens 21.7 / 16.3 against 56.5 / 19.5, 16 tokens 22.8 / 16.8 against
// 102.8 / 33.9.) Four digit planes of the activations become four int8 "token" rows each
// and the W8A8 tensor-core GEMM (qx_int8_gemm_tc.cu) forms the exact integer sums
//   A_d[t, o] = sum_k code[o, k] * p_d[t, k],      d = 0 .. 3,
// over the whole row. The envelope is therefore one power of two per TOKEN, not per 16
// columns, and the fixed point has 31 bits (x = e * t, |t| <= 2^30, t = sum_d 256^d p_d with
// balanced signed bytes): with three planes the fixed-point step of a whole row's envelope
// showed in outputs near zero at K = 4096 (errors of 1e-4 against a tolerance of 4e-5), with
// four it is below the f32 roundings that follow. The GEMM's own epilogue scales float(A_d) by
// the weight scale of the channel and by e * 256^d (two rounded multiplies), and a last kernel
// adds the four planes, the bias, applies the activation and stores the output type.
// |A_d| <= K * 128 * 128 fits int32 for K <= 131000 (the GEMM's own limit). Tokens whose
// largest magnitude is below 2^-70 count as zero.
constexpr long long kPrefillTokens = 5;
constexpr long long kPrefillChunk = 256;  // tokens per GEMM launch: bounds the scratch
constexpr int kPlanes = 4;

__global__ void __launch_bounds__(256) canonical_row_digits_kernel(
    const void* __restrict__ x, int x_type, long long columns, long long chunk_tokens,
    int8_t* __restrict__ planes, float* __restrict__ plane_scale) {
  __shared__ float warp_max[8];
  const long long token = blockIdx.x;
  const long long base = token * columns;
  float amax = 0.0f;
  bool finite = true;
  for (long long k = threadIdx.x; k < columns; k += 256) {
    const float v = fabsf(load_storage(x, x_type, base + k));
    finite = finite && v < __uint_as_float(0x7f800000u);  // false for NaN and infinity
    amax = fmaxf(amax, v);
  }
  if (!finite) amax = __uint_as_float(0x7f800000u);
#pragma unroll
  for (int h = 16; h >= 1; h >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, h));
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
  __syncthreads();
#pragma unroll
  for (int w = 0; w < 8; ++w) amax = fmaxf(amax, warp_max[w]);
  int biased = static_cast<int>(__float_as_uint(amax) >> 23) + 1;  // exponent of 2^E > amax
  biased = biased < 58 ? 58 : biased;                               // keeps e normal
  const bool ok = biased < 256;
  // t = x * 2^30 / 2^E: the factor's exponent 284 - biased is a normal float for 58 .. 255
  const float to_fixed = ok ? __uint_as_float(static_cast<uint32_t>(284 - biased) << 23) : 0.0f;
  const float e = ok ? __uint_as_float(static_cast<uint32_t>(biased - 30) << 23)
                     : __uint_as_float(0x7fc00000u);
  int8_t* out[kPlanes];
#pragma unroll
  for (int d = 0; d < kPlanes; ++d) out[d] = planes + (d * chunk_tokens + token) * columns;
  // a row's digits are written by gridDim.y CTAs, each its slice of the columns (every one of
  // them has scanned the whole row for the envelope)
  const long long slice = (columns + gridDim.y - 1) / gridDim.y;
  const long long k_begin = blockIdx.y * slice;
  const long long k_end = k_begin + slice < columns ? k_begin + slice : columns;
  for (long long k = k_begin + threadIdx.x; k < k_end; k += 256) {
    int t = ok ? __float2int_rn(load_storage(x, x_type, base + k) * to_fixed) : 0;
#pragma unroll
    for (int d = 0; d < kPlanes - 1; ++d) {
      const int digit = ((t + 128) & 255) - 128;
      out[d][k] = static_cast<int8_t>(digit);
      t = (t - digit) >> 8;
    }
    out[kPlanes - 1][k] = static_cast<int8_t>(t);
  }
  if (threadIdx.x == 0 && blockIdx.y == 0) {
    float weight = e;
#pragma unroll
    for (int d = 0; d < kPlanes; ++d) {
      plane_scale[d * chunk_tokens + token] = weight;
      weight *= 256.0f;
    }
  }
}

__global__ void __launch_bounds__(256) canonical_combine_kernel(
    const float* __restrict__ partial, long long chunk_tokens, long long tokens, long long rows,
    long long ldy, const float* __restrict__ bias, int activation, void* __restrict__ y, int y_type) {
  const long long total = tokens * rows;
  const long long plane = chunk_tokens * rows;
  for (long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x; i < total;
       i += 256LL * gridDim.x) {
    // largest plane first
    float v = partial[(kPlanes - 1) * plane + i];
#pragma unroll
    for (int d = kPlanes - 2; d >= 0; --d) v += partial[d * plane + i];
    const long long token = i / rows, row = i - token * rows;
    if (bias != nullptr) v += bias[row];
    store_storage(y, y_type, token * ldy + row, apply_activation(v, activation));
  }
}

size_t prefill_scratch_bytes(long long m, long long rows, long long columns) {
  const long long chunk = m < kPrefillChunk ? m : kPrefillChunk;
  return align_up(static_cast<size_t>(kPlanes * chunk * columns), 256) +
         align_up(static_cast<size_t>(kPlanes * chunk) * sizeof(float), 256) +
         static_cast<size_t>(kPlanes * chunk * rows) * sizeof(float);
}

qx_status launch_prefill_int8(const CanonicalParams& p, uint8_t* scratch, int sm_count,
                              cudaStream_t stream) {
  const long long chunk = p.m < kPrefillChunk ? p.m : kPrefillChunk;
  int8_t* planes = reinterpret_cast<int8_t*>(scratch);
  float* plane_scale = reinterpret_cast<float*>(scratch + align_up(static_cast<size_t>(kPlanes * chunk * p.columns), 256));
  float* partial = plane_scale + align_up(static_cast<size_t>(kPlanes * chunk) * sizeof(float), 256) / sizeof(float);
  const size_t x_bytes = p.x_type == QX_STORAGE_F32 ? 4 : 2, y_bytes = p.y_type == QX_STORAGE_F32 ? 4 : 2;
  for (long long t0 = 0; t0 < p.m; t0 += chunk) {
    const long long tokens = p.m - t0 < chunk ? p.m - t0 : chunk;
    const uint8_t* x = static_cast<const uint8_t*>(p.x) + static_cast<size_t>(t0 * p.columns) * x_bytes;
    // few tokens: several CTAs per row, so that the kernel is not one serial loop per row
    const long long wanted = (2LL * sm_count + tokens - 1) / tokens;
    const long long most = (p.columns + 1023) / 1024;
    const unsigned splits = static_cast<unsigned>(wanted < 1 ? 1 : (wanted > most ? most : (wanted > 16 ? 16 : wanted)));
    canonical_row_digits_kernel<<<dim3(static_cast<unsigned>(tokens), splits), 256, 0, stream>>>(
        x, p.x_type, p.columns, chunk, planes, plane_scale);
    count_launch();
    QX_CUDA_TRY(cudaGetLastError());
    if (tokens < chunk) {
      // the planes of a short last chunk are not contiguous token rows: run them one by one
      for (int d = 0; d < kPlanes; ++d) {
        Int8GemmArgs a{};
        a.w = reinterpret_cast<const int8_t*>(p.data);
        a.x = planes + d * chunk * p.columns;
        a.ws = p.scales;
        a.as = plane_scale + d * chunk;
        a.y = partial + d * chunk * p.rows;
        a.m = tokens;
        a.n = p.rows;
        a.k = p.columns;
        a.ldy = p.rows;
        QX_TRY(launch_int8_gemm(a, stream));
      }
    } else {
      Int8GemmArgs a{};
      a.w = reinterpret_cast<const int8_t*>(p.data);
      a.x = planes;
      a.ws = p.scales;
      a.as = plane_scale;
      a.y = partial;
      a.m = kPlanes * chunk;
      a.n = p.rows;
      a.k = p.columns;
      a.ldy = p.rows;
      QX_TRY(launch_int8_gemm(a, stream));
    }
    uint8_t* y = static_cast<uint8_t*>(p.y) + static_cast<size_t>(t0 * p.ldy) * y_bytes;
    const long long total = tokens * p.rows;
    const long long blocks = (total + 255) / 256;
    const long long cap = 8LL * sm_count;
    canonical_combine_kernel<<<static_cast<unsigned>(blocks < cap ? blocks : cap), 256, 0, stream>>>(
        partial, chunk, tokens, p.rows, p.ldy, p.bias, p.activation, y, p.y_type);
    count_launch();
    QX_CUDA_TRY(cudaGetLastError());
  }
  return QX_STATUS_OK;
}

template <int LAYOUT>
qx_status launch_any(const CanonicalParams& p, bool digits, uint32_t* image, int sm_count,
                     cudaStream_t stream) {
  if (digits) return launch_digits<LAYOUT>(p, image, sm_count, stream);
  return launch_layout<LAYOUT>(p, sm_count, stream);
}

qx_status launch_canonical(const qx_canonical_weights* w, const void* x, int x_type,
                           const float* bias, void* y, int y_type, long long m, int activation,
                           qx_workspace* workspace, cudaStream_t stream) {
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  if (workspace == nullptr) workspace = &ctx->workspace;
  if (ctx->device != w->device) {
    set_last_error_text("canonical projection: weights were prepared on another device");
    return QX_STATUS_INVALID_ARGUMENT;
  }
  if (w->columns > (1LL << 30) || m > 65535) {
    set_last_error_text("canonical projection: more than 2^30 columns or 65535 tokens");
    return QX_STATUS_INVALID_SHAPE;
  }
  CanonicalParams p{};
  p.data = w->data;
  p.scales = w->scales;
  p.zeros = w->zeros;
  p.group_index = w->group_index;
  p.integral_zeros = w->integral_zeros ? 1 : 0;
  p.x = x;
  p.bias = bias;
  p.y = y;
  p.rows = w->rows;
  p.ldy = w->rows;
  p.columns = w->columns;
  p.group_size = w->group_size;
  p.groups_per_row = w->groups_per_row;
  p.m = m;
  p.x_type = x_type;
  p.y_type = y_type;
  p.activation = activation;
  const bool int8 = w->layout == QX_CANONICAL_INT8_SYMMETRIC;
  const long long row_bytes = int8 ? w->columns : w->columns / 2;
  const int code_vector = int8 ? 16 : 8;
  p.vector_rows = (row_bytes % code_vector == 0 &&
                   reinterpret_cast<uintptr_t>(w->data) % code_vector == 0) ? 1 : 0;
  // digit path: one scale (and zero point) per 16 columns, groups in column order; otherwise
  // float multiply-adds on weights decoded one by one
  const bool digits = w->group_index == nullptr &&
                      (p.groups_per_row == 1 || p.group_size % kElems == 0);
  // workspace behind its counters: [gathered activations (act-order)][digit images]
  const size_t gather_bytes =
      w->act_order != nullptr ? align_up(static_cast<size_t>(m) * w->columns * sizeof(float), 256) : 0;
  // int8 with one scale per row, five tokens or more: the tensor-core route
  long long prefill_from = kPrefillTokens;
  // developer switch: QX_B200_CANONICAL_PREFILL_TOKENS=<n> moves the threshold
  if (const char* forced = std::getenv("QX_B200_CANONICAL_PREFILL_TOKENS")) {
    const long long asked = std::atoll(forced);
    if (asked > 0) prefill_from = asked;
  }
  const bool prefill = int8 && p.groups_per_row == 1 && m >= prefill_from && w->columns <= 131000;
  const size_t image_bytes = prefill ? prefill_scratch_bytes(m, w->rows, w->columns)
                                     : (digits ? digit_image_bytes(m, w->columns) : 0);
  uint32_t* image = nullptr;
  if (gather_bytes + image_bytes != 0) {
    QX_TRY(workspace->reserve(kWorkspaceCounterBytes + gather_bytes + image_bytes));
    uint8_t* scratch = static_cast<uint8_t*>(workspace->base) + kWorkspaceCounterBytes;
    image = reinterpret_cast<uint32_t*>(scratch + gather_bytes);
    if (prefill) {
      return launch_prefill_int8(p, scratch + gather_bytes, ctx->prop.multiProcessorCount, stream);
    }
    if (w->act_order != nullptr) {
      float* gathered = reinterpret_cast<float*>(scratch);
      const unsigned gx = static_cast<unsigned>(w->columns + 255) / 256;
      gather_activations_kernel<<<dim3(gx < 64 ? gx : 64, static_cast<unsigned>(m)), 256, 0, stream>>>(
          x, x_type, w->act_order, gathered, w->columns);
      count_launch();
      QX_CUDA_TRY(cudaGetLastError());
      p.x = gathered;
      p.x_type = QX_STORAGE_F32;
    }
  }
  const int x_vector = p.x_type == QX_STORAGE_F32 ? 16 : 8;
  p.vector_x = (w->columns % 4 == 0 && reinterpret_cast<uintptr_t>(p.x) % x_vector == 0) ? 1 : 0;
  const int sm_count = ctx->prop.multiProcessorCount;
  switch (w->layout) {
    case QX_CANONICAL_INT8_SYMMETRIC:
      return launch_any<QX_CANONICAL_INT8_SYMMETRIC>(p, digits, image, sm_count, stream);
    case QX_CANONICAL_INT4_SYMMETRIC:
      return launch_any<QX_CANONICAL_INT4_SYMMETRIC>(p, digits, image, sm_count, stream);
    default:
      return launch_any<QX_CANONICAL_UINT4_AFFINE>(p, digits, image, sm_count, stream);
  }
}

bool finite_nonnegative(const float* v, size_t count) {
  for (size_t i = 0; i < count; ++i) {
    if (!std::isfinite(v[i]) || v[i] < 0.0f) return false;
  }
  return true;
}
bool finite_all(const float* v, size_t count) {
  for (size_t i = 0; i < count; ++i) {
    if (!std::isfinite(v[i])) return false;
  }
  return true;
}

// Shape checks shared by prepare and the entry points.
qx_status validate_tensor(const qx_canonical_tensor* t, long long* groups_per_row,
                          long long* group_size) {
  if (t->layout != QX_CANONICAL_INT8_SYMMETRIC && t->layout != QX_CANONICAL_INT4_SYMMETRIC &&
      t->layout != QX_CANONICAL_UINT4_AFFINE) {
    return QX_STATUS_UNSUPPORTED_FORMAT;
  }
  const bool four_bit = t->layout != QX_CANONICAL_INT8_SYMMETRIC;
  if (!valid_product2(t->rows, t->columns)) return QX_STATUS_INVALID_SHAPE;
  if (t->group_size < 0 || (t->group_size > 0 && t->columns % t->group_size != 0)) {
    return QX_STATUS_INVALID_SHAPE;
  }
  // the optional column maps (src/memory/quant_contract.cpp:120-137): full length, and only
  // for the 4-bit layouts
  if ((t->act_order_count != 0 && t->act_order_count != static_cast<size_t>(t->columns)) ||
      (t->group_index_count != 0 && t->group_index_count != static_cast<size_t>(t->columns))) {
    return QX_STATUS_INVALID_SHAPE;
  }
  if ((t->group_index_count != 0 || t->act_order_count != 0) && !four_bit) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  // validate_quant_metadata counts the scales its mode implies first
  // (src/memory/quant_contract.cpp:176-208) ...
  const size_t rows = static_cast<size_t>(t->rows), columns = static_cast<size_t>(t->columns);
  size_t expected_scales = 0;
  long long groups = 1, size = t->columns;
  switch (t->scale_mode) {
    case QX_SCALE_NONE: break;
    case QX_SCALE_TENSOR: expected_scales = 1; break;
    case QX_SCALE_ROW:
    case QX_SCALE_CHANNEL: expected_scales = rows; break;
    case QX_SCALE_GROUP:
      if (t->group_size <= 0) return QX_STATUS_INVALID_SHAPE;
      groups = t->columns / t->group_size;
      size = t->group_size;
      expected_scales = rows * static_cast<size_t>(groups);
      break;
    case 5:  // kBlock
      if (t->scale_count == 0) return QX_STATUS_INVALID_SHAPE;
      expected_scales = t->scale_count;
      break;
    case 6:  // kMicroscaleK32
    case 8:  // kTurboQuantK32
      expected_scales = rows * (columns / 32);
      break;
    case 7:  // kNVFP4K16
      expected_scales = rows * (columns / 16);
      break;
    default: return QX_STATUS_INVALID_ARGUMENT;
  }
  if (t->scale_count != expected_scales) return QX_STATUS_INVALID_SHAPE;
  // one zero point per scale for the affine layout, none otherwise (quant_contract.cpp:213-218)
  if (t->zero_point_count != (t->layout == QX_CANONICAL_UINT4_AFFINE ? expected_scales : 0)) {
    return QX_STATUS_INVALID_SHAPE;
  }
  // ... then validate_canonical_quant_tensor accepts row, channel and group scales for the
  // integer layouts (kernels/quantization/quant_import_ref.cpp:406-421)
  if (t->scale_mode != QX_SCALE_ROW && t->scale_mode != QX_SCALE_CHANNEL &&
      t->scale_mode != QX_SCALE_GROUP) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  size_t expected = rows * columns;
  if (four_bit) {
    if ((t->columns & 1) != 0) return QX_STATUS_INVALID_SHAPE;
    expected /= 2;
  }
  if (t->data_bytes != expected) return QX_STATUS_INVALID_SHAPE;
  if (t->data == nullptr || t->scales == nullptr ||
      (t->zero_point_count != 0 && t->zero_points == nullptr) ||
      (t->group_index_count != 0 && t->group_index == nullptr) ||
      (t->act_order_count != 0 && t->act_order == nullptr)) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  if (!finite_nonnegative(t->scales, t->scale_count) ||
      !finite_all(t->zero_points, t->zero_point_count)) {
    return QX_STATUS_INVALID_SHAPE;
  }
  // act_order is a permutation of the columns, group_index names existing groups
  // (quant_import_ref.cpp:477-490)
  if (t->act_order_count != 0) {
    std::vector<uint8_t> seen(static_cast<size_t>(t->columns), 0);
    for (size_t i = 0; i < t->act_order_count; ++i) {
      const int v = t->act_order[i];
      if (v < 0 || v >= t->columns || seen[static_cast<size_t>(v)] != 0) return QX_STATUS_INVALID_ARGUMENT;
      seen[static_cast<size_t>(v)] = 1;
    }
  }
  for (size_t i = 0; i < t->group_index_count; ++i) {
    if (t->group_index[i] < 0 || t->group_index[i] >= groups) return QX_STATUS_INVALID_ARGUMENT;
  }
  *groups_per_row = groups;
  *group_size = size;
  return QX_STATUS_OK;
}

}  // namespace

// lowbit_gemm on compact int4 rows (value = nibble - 8, one f32 scale per row or per group of a
// multiple of 16 columns, even column count): the digit kernels.
bool int4_offset8_digits_serves(long long m, long long k, long long groups, long long group_size) {
  return m <= 65535 && k % 2 == 0 && k <= (1LL << 30) &&
         (groups == 1 || (group_size % kElems == 0 && k % group_size == 0));
}
qx_status launch_int4_offset8_digits(const uint8_t* packed, const float* scales, const float* x,
                                     float* y, long long m, long long n, long long k,
                                     long long groups, long long group_size, cudaStream_t stream) {
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  CanonicalParams p{};
  p.data = packed;
  p.scales = scales;
  p.x = x;
  p.y = y;
  p.rows = n;
  p.ldy = n;
  p.columns = k;
  p.group_size = groups == 1 ? k : group_size;
  p.groups_per_row = groups;
  p.m = m;
  p.x_type = QX_STORAGE_F32;
  p.y_type = QX_STORAGE_F32;
  p.activation = QX_ACTIVATION_NONE;
  p.vector_rows = ((k / 2) % 8 == 0 && reinterpret_cast<uintptr_t>(packed) % 8 == 0) ? 1 : 0;
  p.vector_x = (k % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0) ? 1 : 0;
  QX_TRY(ctx->workspace.reserve(kWorkspaceCounterBytes + digit_image_bytes(m, k)));
  uint32_t* image = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(ctx->workspace.base) +
                                                kWorkspaceCounterBytes);
  return launch_digits<kLayoutInt4Offset8>(p, image, ctx->prop.multiProcessorCount, stream);
}

// qgemm_w8a32 (int8 weights, one f32 scale per row, f32 in and out) from five tokens on: the
// same digit planes through the W8A8 tensor-core GEMM.
bool w8a32_planes_serves(long long m, long long k) { return m >= kPrefillTokens && k <= 131000 && m <= 65535; }
qx_status launch_w8a32_planes(const int8_t* w, const float* ws, const float* x, float* y,
                              long long m, long long n, long long k, long long ldy,
                              qx_workspace* workspace, cudaStream_t stream) {
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  if (workspace == nullptr) workspace = &ctx->workspace;
  CanonicalParams p{};
  p.data = reinterpret_cast<const uint8_t*>(w);
  p.scales = ws;
  p.x = x;
  p.y = y;
  p.rows = n;
  p.ldy = ldy;
  p.columns = k;
  p.group_size = k;
  p.groups_per_row = 1;
  p.m = m;
  p.x_type = QX_STORAGE_F32;
  p.y_type = QX_STORAGE_F32;
  p.activation = QX_ACTIVATION_NONE;
  QX_TRY(workspace->reserve(kWorkspaceCounterBytes + prefill_scratch_bytes(m, n, k)));
  return launch_prefill_int8(p, static_cast<uint8_t*>(workspace->base) + kWorkspaceCounterBytes,
                             ctx->prop.multiProcessorCount, stream);
}

}  // namespace qx

using namespace qx;

extern "C" {

qx_status qx_canonical_prepare(const qx_canonical_tensor* tensor, qx_canonical_weights** out) {
  if (tensor == nullptr || out == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  *out = nullptr;
  long long groups = 1, size = 0;
  QX_TRY(validate_tensor(tensor, &groups, &size));
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  qx_canonical_weights* w = new (std::nothrow) qx_canonical_weights();
  if (w == nullptr) return QX_STATUS_OUT_OF_MEMORY;
  w->layout = tensor->layout;
  w->scale_mode = tensor->scale_mode;
  w->device = ctx->device;
  w->rows = tensor->rows;
  w->columns = tensor->columns;
  w->group_size = size;
  w->groups_per_row = groups;
  w->data_bytes = tensor->data_bytes;
  w->scale_count = tensor->scale_count;
  w->integral_zeros = tensor->zero_point_count != 0;
  for (size_t i = 0; i < tensor->zero_point_count; ++i) {
    const float z = tensor->zero_points[i];
    if (!(z >= 0.0f && z <= 15.0f && z == static_cast<float>(static_cast<int>(z)))) {
      w->integral_zeros = false;
      break;
    }
  }
  // one allocation: codes, then every table on a 256-byte boundary
  const size_t scale_offset = align_up(tensor->data_bytes, 256);
  const size_t zero_offset = scale_offset + align_up(tensor->scale_count * sizeof(float), 256);
  const size_t group_offset = zero_offset + align_up(tensor->zero_point_count * sizeof(float), 256);
  const size_t order_offset = group_offset + align_up(tensor->group_index_count * sizeof(int), 256);
  const size_t total = order_offset + align_up(tensor->act_order_count * sizeof(int), 256);
  void* block = nullptr;
  cudaError_t err = cudaMalloc(&block, total);
  if (err != cudaSuccess) {
    set_last_error("cudaMalloc(canonical weights)", err);
    delete w;
    return err == cudaErrorMemoryAllocation ? QX_STATUS_OUT_OF_MEMORY : QX_STATUS_DEVICE_ERROR;
  }
  w->data = static_cast<uint8_t*>(block);
  w->scales = reinterpret_cast<float*>(w->data + scale_offset);
  if (tensor->zero_point_count != 0) w->zeros = reinterpret_cast<float*>(w->data + zero_offset);
  if (tensor->group_index_count != 0) w->group_index = reinterpret_cast<int*>(w->data + group_offset);
  if (tensor->act_order_count != 0) w->act_order = reinterpret_cast<int*>(w->data + order_offset);
  std::lock_guard<std::mutex> lock(ctx->mutex);
  auto upload = [&](void* dst, const void* src, size_t bytes) {
    if (err == cudaSuccess && bytes != 0) {
      err = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream);
    }
  };
  upload(w->data, tensor->data, tensor->data_bytes);
  upload(w->scales, tensor->scales, tensor->scale_count * sizeof(float));
  upload(w->zeros, tensor->zero_points, tensor->zero_point_count * sizeof(float));
  upload(w->group_index, tensor->group_index, tensor->group_index_count * sizeof(int));
  upload(w->act_order, tensor->act_order, tensor->act_order_count * sizeof(int));
  if (err == cudaSuccess) err = cudaStreamSynchronize(ctx->stream);
  if (err != cudaSuccess) {
    set_last_error("upload of canonical weights", err);
    (void)cudaFree(block);
    delete w;
    return QX_STATUS_DEVICE_ERROR;
  }
  *out = w;
  return QX_STATUS_OK;
}

void qx_canonical_destroy(qx_canonical_weights* weights) {
  if (weights == nullptr) return;
  if (weights->data != nullptr) (void)cudaFree(weights->data);
  delete weights;
}

qx_status qx_qgemm_prepacked_epilogue_storage_dev(const qx_canonical_weights* weights,
                                                  const void* x_dev, int x_type,
                                                  const float* bias_dev, void* y_dev, int y_type,
                                                  long long m, int activation,
                                                  qx_workspace* workspace, void* stream) {
  if (!known_activation(activation)) return QX_STATUS_INVALID_ARGUMENT;
  if (weights == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  if (!valid_product2(m, weights->columns) || !valid_product2(m, weights->rows)) {
    return QX_STATUS_INVALID_SHAPE;
  }
  if (!known_storage(x_type) || !known_storage(y_type)) return QX_STATUS_UNSUPPORTED_FORMAT;
  if (x_dev == nullptr || y_dev == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  return launch_canonical(weights, x_dev, x_type, bias_dev, y_dev, y_type, m, activation, workspace,
                          static_cast<cudaStream_t>(stream));
}

qx_status qx_qgemm_prepacked_epilogue_storage(const qx_canonical_weights* weights, const void* x,
                                              int x_type, long long x_count, const float* bias,
                                              void* y, int y_type, long long y_count, long long m,
                                              int activation) {
  // validation order of qgemm_prepacked_storage_impl, qgemm_canonical.cpp:4460-4481
  if (!known_activation(activation)) return QX_STATUS_INVALID_ARGUMENT;
  if (weights == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  if (!valid_product2(m, weights->columns) || !valid_product2(m, weights->rows) ||
      x_count != m * weights->columns || y_count != m * weights->rows) {
    return QX_STATUS_INVALID_SHAPE;
  }
  if (!known_storage(x_type) || !known_storage(y_type)) return QX_STATUS_UNSUPPORTED_FORMAT;
  if (x == nullptr || y == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  std::lock_guard<std::mutex> lock(ctx->mutex);
  const size_t x_bytes = static_cast<size_t>(x_count) * storage_bytes(x_type);
  const size_t y_bytes = static_cast<size_t>(y_count) * storage_bytes(y_type);
  const size_t bias_bytes = bias != nullptr ? static_cast<size_t>(weights->rows) * 4 : 0;
  const size_t off_x = 0, off_bias = align_up(x_bytes, 256);
  const size_t off_y = off_bias + align_up(bias_bytes == 0 ? 1 : bias_bytes, 256);
  QX_TRY(ctx->ensure_staging(off_y + align_up(y_bytes, 256)));
  uint8_t* stage = static_cast<uint8_t*>(ctx->staging);
  cudaStream_t s = ctx->stream;
  QX_CUDA_TRY(cudaMemcpyAsync(stage + off_x, x, x_bytes, cudaMemcpyHostToDevice, s));
  if (bias != nullptr) {
    QX_CUDA_TRY(cudaMemcpyAsync(stage + off_bias, bias, bias_bytes, cudaMemcpyHostToDevice, s));
  }
  QX_TRY(launch_canonical(weights, stage + off_x, x_type,
                          bias != nullptr ? reinterpret_cast<const float*>(stage + off_bias)
                                          : nullptr,
                          stage + off_y, y_type, m, activation, nullptr, s));
  QX_CUDA_TRY(cudaMemcpyAsync(y, stage + off_y, y_bytes, cudaMemcpyDeviceToHost, s));
  QX_CUDA_TRY(cudaStreamSynchronize(s));
  return QX_STATUS_OK;
}

qx_status qx_qgemm_prepacked_storage(const qx_canonical_weights* weights, const void* x,
                                     int x_type, long long x_count, void* y, int y_type,
                                     long long y_count, long long m) {
  return qx_qgemm_prepacked_epilogue_storage(weights, x, x_type, x_count, nullptr, y, y_type,
                                             y_count, m, QX_ACTIVATION_NONE);
}

const char* qx_canonical_gemm_variant(void) { return "sm100a_stream_fma_typed"; }

qx_status qx_import_smoothquant_w8a8(const qx_smoothquant_source* source,
                                     qx_canonical_tensor* tensor, int32_t* row_sums_out) {
  // check order of import_smoothquant_w8a8, quant_import_ref.cpp:1053-1074
  if (source == nullptr || tensor == nullptr || row_sums_out == nullptr ||
      source->weights == nullptr || source->weight_scales == nullptr ||
      source->activation_scales == nullptr || !valid_product2(source->rows, source->columns)) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  const size_t elements =
      static_cast<size_t>(source->rows) * static_cast<size_t>(source->columns);
  if (source->weight_count != elements ||
      source->weight_scale_count != static_cast<size_t>(source->rows) ||
      source->activation_scale_count == 0 ||
      (source->activation_zero_point_count != 0 &&
       (source->activation_zero_points == nullptr ||
        source->activation_zero_point_count != source->activation_scale_count)) ||
      (source->row_sum_count != 0 &&
       (source->row_sums == nullptr ||
        source->row_sum_count != static_cast<size_t>(source->rows))) ||
      !finite_all(source->weight_scales, source->weight_scale_count) ||
      !finite_all(source->activation_scales, source->activation_scale_count)) {
    return QX_STATUS_INVALID_SHAPE;
  }
  // validate_canonical_quant_tensor rejects a negative scale (quant_import_ref.cpp:470-476)
  if (!finite_nonnegative(source->weight_scales, source->weight_scale_count)) {
    return QX_STATUS_INVALID_SHAPE;
  }
  for (long long row = 0; row < source->rows; ++row) {
    if (source->row_sum_count != 0) {
      row_sums_out[row] = source->row_sums[row];
    } else {
      int32_t sum = 0;
      const int8_t* codes = source->weights + row * source->columns;
      for (long long column = 0; column < source->columns; ++column) sum += codes[column];
      row_sums_out[row] = sum;
    }
  }
  tensor->layout = QX_CANONICAL_INT8_SYMMETRIC;
  tensor->scale_mode = QX_SCALE_CHANNEL;
  tensor->rows = source->rows;
  tensor->columns = source->columns;
  tensor->group_size = source->columns;
  tensor->data = reinterpret_cast<const uint8_t*>(source->weights);
  tensor->data_bytes = elements;
  tensor->scales = source->weight_scales;
  tensor->scale_count = source->weight_scale_count;
  tensor->zero_points = nullptr;
  tensor->zero_point_count = 0;
  tensor->group_index = nullptr;
  tensor->group_index_count = 0;
  tensor->act_order = nullptr;
  tensor->act_order_count = 0;
  return QX_STATUS_OK;
}

namespace {
void put_nibble(uint8_t* bytes, size_t element, unsigned code) {
  const int shift = static_cast<int>(4 * (element & 1));
  bytes[element / 2] = static_cast<uint8_t>((bytes[element / 2] & ~(0x0fu << shift)) |
                                            ((code & 0x0fu) << shift));
}
// the view a 4-bit importer returns over the caller's output arrays
void fill_view(qx_canonical_tensor* t, int layout, long long n, long long k, long long group,
               const uint8_t* data, const float* scales, const float* zeros, size_t groups) {
  t->layout = layout;
  t->scale_mode = QX_SCALE_GROUP;
  t->rows = n;
  t->columns = k;
  t->group_size = group;
  t->data = data;
  t->data_bytes = static_cast<size_t>(n) * static_cast<size_t>(k) / 2;
  t->scales = scales;
  t->scale_count = static_cast<size_t>(n) * groups;
  t->zero_points = zeros;
  t->zero_point_count = zeros != nullptr ? static_cast<size_t>(n) * groups : 0;
  t->group_index = nullptr;
  t->group_index_count = 0;
  t->act_order = nullptr;
  t->act_order_count = 0;
}
}  // namespace

qx_status qx_import_awq_u4(const qx_awq_u4_source* source, qx_canonical_tensor* tensor,
                           uint8_t* data_out, float* scales_out, float* zero_points_out) {
  // checks of import_awq_u4, quant_import_ref.cpp:842-860
  if (source == nullptr || tensor == nullptr || data_out == nullptr || scales_out == nullptr ||
      zero_points_out == nullptr || source->qweight == nullptr || source->qzeros == nullptr ||
      source->scales == nullptr || source->input_features <= 0 || source->output_features <= 0 ||
      source->group_size <= 0 || source->input_features % source->group_size != 0 ||
      source->output_features % 8 != 0 || source->input_features % 2 != 0) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  const size_t k = static_cast<size_t>(source->input_features);
  const size_t n = static_cast<size_t>(source->output_features);
  const size_t groups = k / static_cast<size_t>(source->group_size);
  if (source->qweight_words != k * (n / 8) || source->qzero_words != groups * (n / 8) ||
      source->scale_count != groups * n || !finite_all(source->scales, source->scale_count)) {
    return QX_STATUS_INVALID_SHAPE;
  }
  // a negative scale fails validate_canonical_quant_tensor (quant_import_ref.cpp:470-476)
  if (!finite_nonnegative(source->scales, source->scale_count)) return QX_STATUS_INVALID_SHAPE;
  // AWQ packs output channel o of a word at nibble kAwqReverseOrder[o & 7] (:17, :869-880)
  static const int kAwqReverseOrder[8] = {0, 4, 1, 5, 2, 6, 3, 7};
  for (size_t i = 0; i < n * k / 2; ++i) data_out[i] = 0;
  for (size_t output = 0; output < n; ++output) {
    const size_t word_column = output / 8;
    const int lane = kAwqReverseOrder[output & 7];
    for (size_t input = 0; input < k; ++input) {
      const uint32_t word = source->qweight[input * (n / 8) + word_column];
      put_nibble(data_out, output * k + input, (word >> (4 * lane)) & 0x0fu);
    }
    for (size_t group = 0; group < groups; ++group) {
      const uint32_t word = source->qzeros[group * (n / 8) + word_column];
      scales_out[output * groups + group] = source->scales[group * n + output];
      zero_points_out[output * groups + group] = static_cast<float>((word >> (4 * lane)) & 0x0fu);
    }
  }
  fill_view(tensor, QX_CANONICAL_UINT4_AFFINE, source->output_features, source->input_features,
            source->group_size, data_out, scales_out, zero_points_out, groups);
  return QX_STATUS_OK;
}

qx_status qx_import_gptq_u4(const qx_gptq_u4_source* source, qx_canonical_tensor* tensor,
                            uint8_t* data_out, float* scales_out, float* zero_points_out) {
  // checks of import_gptq_u4, quant_import_ref.cpp:907-930
  if (source == nullptr || tensor == nullptr || data_out == nullptr || scales_out == nullptr ||
      source->qweight == nullptr || source->qzeros == nullptr || source->scales == nullptr ||
      source->input_features <= 0 || source->output_features <= 0 ||
      source->input_features % 8 != 0 || source->output_features % 8 != 0 ||
      source->group_size <= 0 || source->input_features % source->group_size != 0 ||
      (source->symmetric == 0 && zero_points_out == nullptr)) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  const size_t k = static_cast<size_t>(source->input_features);
  const size_t n = static_cast<size_t>(source->output_features);
  const size_t groups = k / static_cast<size_t>(source->group_size);
  if (source->qweight_words != (k / 8) * n || source->qzero_words != groups * (n / 8) ||
      source->scale_count != groups * n ||
      (source->group_index_count != 0 &&
       (source->group_index == nullptr || source->group_index_count != k)) ||
      (source->act_order_count != 0 &&
       (source->act_order == nullptr || source->act_order_count != k)) ||
      !finite_all(source->scales, source->scale_count)) {
    return QX_STATUS_INVALID_SHAPE;
  }
  const bool symmetric = source->symmetric != 0;
  auto zero_of = [&](size_t group, size_t output) {
    const uint32_t word = source->qzeros[group * (n / 8) + output / 8];
    int zero = static_cast<int>((word >> (4 * (output & 7))) & 0x0fu);
    if (source->gptq_v2 == 0) zero = (zero + 1) & 0x0f;  // V1 checkpoints store zero - 1
    return zero;
  };
  for (size_t i = 0; i < n * k / 2; ++i) data_out[i] = 0;
  for (size_t output = 0; output < n; ++output) {
    for (size_t input = 0; input < k; ++input) {
      const uint32_t word = source->qweight[(input / 8) * n + output];
      const int raw = static_cast<int>((word >> (4 * (input & 7))) & 0x0fu);
      int code = raw;
      if (symmetric) {
        // the zero point is folded into a signed code (:947-959)
        const size_t zero_group = source->group_index_count == 0
                                      ? input / static_cast<size_t>(source->group_size)
                                      : static_cast<size_t>(source->group_index[input]);
        if (zero_group >= groups) return QX_STATUS_INVALID_ARGUMENT;
        int folded = raw - zero_of(zero_group, output);
        folded = folded < -8 ? -8 : (folded > 7 ? 7 : folded);
        code = folded & 0x0f;
      }
      put_nibble(data_out, output * k + input, static_cast<unsigned>(code));
    }
    for (size_t group = 0; group < groups; ++group) {
      scales_out[output * groups + group] = source->scales[group * n + output];
      if (!symmetric) zero_points_out[output * groups + group] = static_cast<float>(zero_of(group, output));
    }
  }
  fill_view(tensor, symmetric ? QX_CANONICAL_INT4_SYMMETRIC : QX_CANONICAL_UINT4_AFFINE,
            source->output_features, source->input_features, source->group_size, data_out,
            scales_out, symmetric ? nullptr : zero_points_out, groups);
  if (source->group_index_count != 0) {
    tensor->group_index = source->group_index;
    tensor->group_index_count = k;
  }
  if (source->act_order_count != 0) {
    tensor->act_order = source->act_order;
    tensor->act_order_count = k;
  }
  // what validate_canonical_quant_tensor then rejects (quant_import_ref.cpp:470-490)
  long long groups_checked = 0, size_checked = 0;
  return validate_tensor(tensor, &groups_checked, &size_checked);
}

}  // extern "C"
