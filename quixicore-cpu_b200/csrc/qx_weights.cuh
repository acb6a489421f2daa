// Device-resident prepared weights (the B200 counterpart of CpuPackedWeights,
// src/memory/packed_weights.cpp:141-278).
//
// HBM layout ("split planes"). The canonical GGUF bytes interleave a 2-byte fp16 scale
// with 32 (q8_0) or 16 (q4_0) code bytes, so no block starts on a 16-byte boundary. At
// prepare time one pass re-lays them out, for the rows kept on this device, as
//   codes  [rows][blocks_per_row][32 | 16] bytes   16-byte aligned, row-major
//   scales [rows][blocks_per_row]          fp16 bits
// which is byte-for-byte the same amount of data (34 or 18 bytes per block) but lets a
// warp read 32 consecutive blocks of a row as one contiguous, 128-bit-vectorised span.
#pragma once

#include "qx_common.cuh"

struct qx_weights {
  int format = 0;
  int device = -1;
  long long rows_total = 0;  // rows of the full matrix
  long long row_begin = 0;   // first row kept on this device
  long long rows = 0;        // rows kept
  long long columns = 0;
  long long blocks_per_row = 0;
  size_t block_bytes = 0;
  size_t contract_bytes = 0;
  size_t prepared_bytes = 0;
  uint64_t preparation_ns = 0;
  uint8_t* codes = nullptr;         // device
  unsigned short* scales = nullptr; // device, fp16 bits
  // Lazily built by the prefill GEMM (see qx_q4_gemm.cu); not part of prepared_bytes
  // until built.
  void* dense_cache = nullptr;
  size_t dense_cache_bytes = 0;
};

namespace qx {

// Re-layout canonical blocks [rows][nb][block_bytes] -> split planes. `src` points at
// the first kept row's first block (device memory, 2-byte aligned).
qx_status launch_relayout(int format, const uint8_t* src, long long rows, long long nb,
                          uint8_t* codes, unsigned short* scales, cudaStream_t stream);

// y[m][ldy] (+ row offset already applied by the caller) = x[m][k] . dequant(W)^T
qx_status launch_qgemm_f32(const qx_weights* w, const float* x_dev, float* y_dev,
                           long long m, long long ldy, qx_workspace* ws,
                           cudaStream_t stream);

}  // namespace qx
