// Device-resident prepared weights (the B200 counterpart of CpuPackedWeights,
// src/memory/packed_weights.cpp:141-278).
//
// HBM layout ("row-tile panels"). The canonical GGUF bytes interleave a 2-byte fp16 scale
// with 32 (q8_0) or 16 (q4_0) code bytes, so no block starts on a 16-byte boundary. At
// prepare time one pass re-lays the rows kept on this device out as tiles of 128 rows by
// K-slabs of 8 blocks (256 elements), the unit one CTA pipeline stage consumes:
//   panel [tile][slab]{ codes  [row 0..127][8 blocks x (32 | 16) code bytes]  32 KiB | 16 KiB
//                       scales [row 0..127][block 0..7] fp16 bits             2 KiB }
// Each (tile, slab) is one contiguous span of 34 KiB (q8_0) or 18 KiB (q4_0), so a stage
// is ONE fully coalesced bulk read; code rows are 128 bytes with their 16-byte chunks
// already permuted into the 128-byte swizzle of the tensor-core operand (qx_gemv.cuh).
// Same byte count as the canonical layout (34 / 18 bytes per block) whenever
// rows % 128 == 0 and columns % 256 == 0 -- every benchmark shape -- otherwise the last
// tile / slab is zero padded (a zero scale contributes 0).
// This is the device counterpart of the reference's [row_panel, k_block, row_lane,
// block_bytes] CPU panel (src/memory/packed_weights.cpp:253-266).
#pragma once

#include "qx_common.cuh"
#include "qx_gemv.cuh"

struct qx_weights {
  int format = 0;
  int device = -1;
  long long rows_total = 0;  // rows of the full matrix
  long long row_begin = 0;   // first row kept on this device
  long long rows = 0;        // rows kept
  long long columns = 0;
  long long blocks_per_row = 0;
  long long tiles = 0;       // ceil(rows / 128)
  long long slabs = 0;       // ceil(blocks_per_row / 8)
  size_t block_bytes = 0;
  size_t contract_bytes = 0;
  size_t prepared_bytes = 0;
  uint64_t preparation_ns = 0;
  uint8_t* panel = nullptr;  // device: [tile][slab]{codes, scales}
  // A handle may hold several matrices with the same column count back to back ("fused"
  // projections: up + gate, q + k + v), each starting on a tile boundary, so that one GEMV
  // launch streams all of them. segment s covers tiles [seg_tile_begin[s], ...) and has
  // seg_rows[s] rows; `rows` is their sum. Ordinary handles have one segment.
  static constexpr int kMaxSegments = 4;
  int segments = 1;
  long long seg_tile_begin[kMaxSegments] = {0, 0, 0, 0};
  long long seg_rows[kMaxSegments] = {0, 0, 0, 0};
  // Lazily built by the prefill GEMM (see qx_q4_gemm.cu); not part of prepared_bytes
  // until built.
  void* dense_cache = nullptr;
  size_t dense_cache_bytes = 0;

  size_t code_bytes_per_block() const { return block_bytes - 2; }
  // bytes of the whole span of one (tile, slab)
  size_t slab_bytes() const { return static_cast<size_t>(qx::slab_span_bytes(format)); }
  size_t panel_bytes() const { return static_cast<size_t>(tiles) * slabs * slab_bytes(); }
};

namespace qx {

// Re-layout canonical blocks [rows][nb][block_bytes] -> panels. `src` points at the first
// kept row's first block (device memory, 2-byte aligned).
// Same for one segment of a fused handle: `rows` rows into the tiles from `tile_begin` on.
qx_status launch_relayout(const qx_weights* w, const uint8_t* src, cudaStream_t stream);
qx_status launch_relayout_segment(const qx_weights* w, const uint8_t* src, long long rows,
                                  long long tile_begin, cudaStream_t stream);

// y[m][ldy] (+ row offset already applied by the caller) = x[m][k] . dequant(W)^T
// `push` (qx_gemv_tc.cuh): also store the results on the other ranks (m <= 32 only).
struct GemvPush;
// Extras of a GEMV launch: where a fused handle's segments write their outputs (dense
// [m][seg_rows[s]] each; null: the y argument, one segment) and how the in-kernel quantizer
// treats the activations.
struct GemvOptions {
  float* segment_y[qx_weights::kMaxSegments] = {nullptr, nullptr, nullptr, nullptr};
  // false: 23-bit fixed point under a power-of-two block envelope (the f32 path).
  // true: the activation quantisation of qgemv_w8a8 (per 32-block scale amax / 127, codes
  // nearbyint(x / scale) clamped to +-127; kernels/quantization/qgemv_w8a8_ref.cpp:18-41);
  // single activation row only.
  bool int8_activations = false;
};
qx_status launch_qgemm_f32(const qx_weights* w, const float* x_dev, float* y_dev,
                           long long m, long long ldy, qx_workspace* ws,
                           cudaStream_t stream, const GemvPush* push = nullptr,
                           const GemvOptions* options = nullptr);

}  // namespace qx
