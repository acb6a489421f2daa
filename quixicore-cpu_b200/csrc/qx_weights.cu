// Prepared weights: load-time re-layout of canonical GGUF blocks into device planes.
// Counterpart of CpuPackedWeights::prepare (src/memory/packed_weights.cpp:197-278); like
// the reference's panel build it runs once per weight matrix, outside any timed region.

#include <chrono>
#include <new>

#include "qx_weights.cuh"

namespace qx {
namespace {

// One thread per panel block slot (tile, slab, row-in-tile, block-in-slab). Canonical
// blocks are only 2-byte aligned (34 / 18 byte stride), so they are read as 16-bit words;
// slots past the last row or block are written as zeros.
template <int FMT>
__global__ void __launch_bounds__(256) relayout_kernel(const unsigned short* __restrict__ src,
                                                       long long rows, long long nb,
                                                       long long slabs, long long total_slots,
                                                       uint8_t* __restrict__ panel) {
  constexpr int kWords = FMT == QX_FORMAT_Q8_0 ? 17 : 9;  // 16-bit words per block
  const long long slot = blockIdx.x * 256LL + threadIdx.x;
  if (slot >= total_slots) return;
  const int j = static_cast<int>(slot % kSlabBlocks);
  const int r = static_cast<int>((slot / kSlabBlocks) % kTileRows);
  const long long ts = slot / (kSlabBlocks * kTileRows);  // tile * slabs + slab
  const long long s = ts % slabs, tile = ts / slabs;
  const long long row = tile * kTileRows + r, b = s * kSlabBlocks + j;
  uint32_t w[(kWords - 1) / 2];
  unsigned short scale = 0;
#pragma unroll
  for (int i = 0; i < (kWords - 1) / 2; ++i) w[i] = 0;
  if (row < rows && b < nb) {
    const unsigned short* in = src + (row * nb + b) * kWords;
    scale = in[0];
#pragma unroll
    for (int i = 0; i < (kWords - 1) / 2; ++i) {
      w[i] = static_cast<uint32_t>(in[1 + 2 * i]) | (static_cast<uint32_t>(in[2 + 2 * i]) << 16);
    }
  }
  uint8_t* span = panel + ts * slab_span_bytes(FMT);
  *reinterpret_cast<unsigned short*>(span + panel_scale_offset(FMT, r, j)) = scale;
  if constexpr (FMT == QX_FORMAT_Q8_0) {
    *reinterpret_cast<uint4*>(span + panel_code_offset_q8(r, j, 0)) = make_uint4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<uint4*>(span + panel_code_offset_q8(r, j, 1)) = make_uint4(w[4], w[5], w[6], w[7]);
  } else {
    *reinterpret_cast<uint4*>(span + panel_code_offset_q4(r, j)) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

}  // namespace

qx_status launch_relayout(const qx_weights* w, const uint8_t* src, cudaStream_t stream) {
  return launch_relayout_segment(w, src, w->rows, 0, stream);
}

qx_status launch_relayout_segment(const qx_weights* w, const uint8_t* src, long long rows,
                                  long long tile_begin, cudaStream_t stream) {
  const long long tiles = (rows + kTileRows - 1) / kTileRows;
  const long long total = tiles * w->slabs * kTileRows * kSlabBlocks;
  const unsigned grid = static_cast<unsigned>((total + 255) / 256);
  const auto* in = reinterpret_cast<const unsigned short*>(src);
  uint8_t* panel = w->panel + static_cast<size_t>(tile_begin) * w->slabs * w->slab_bytes();
  if (w->format == QX_FORMAT_Q8_0) {
    relayout_kernel<QX_FORMAT_Q8_0><<<grid, 256, 0, stream>>>(
        in, rows, w->blocks_per_row, w->slabs, total, panel);
  } else {
    relayout_kernel<QX_FORMAT_Q4_0><<<grid, 256, 0, stream>>>(
        in, rows, w->blocks_per_row, w->slabs, total, panel);
  }
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  return QX_STATUS_OK;
}

namespace {

qx_status prepare_common(int format, const void* contract, bool contract_on_device,
                         long long rows, long long columns, long long row_begin,
                         long long row_count, cudaStream_t stream, bool sync,
                         qx_weights** out) {
  const auto t0 = std::chrono::steady_clock::now();
  if (out == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  *out = nullptr;
  // CpuPackedWeights::prepare: null check first, then the packed-size validation
  // (packed_weights.cpp:201-208).
  if (contract == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  size_t contract_bytes = 0;
  QX_TRY(validate_nk(format, rows, columns));
  QX_TRY(packed_bytes(format, rows, columns, &contract_bytes));
  if (row_begin < 0 || row_count <= 0 || row_begin > rows - row_count) {
    return QX_STATUS_INVALID_SHAPE;
  }
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));

  size_t block_bytes = 0;
  format_info(format, &block_bytes);
  const long long nb = columns / kBlockK;
  const size_t shard_bytes = static_cast<size_t>(row_count) * nb * block_bytes;

  auto* w = new (std::nothrow) qx_weights();
  if (w == nullptr) return QX_STATUS_OUT_OF_MEMORY;
  w->format = format;
  w->device = ctx->device;
  w->rows_total = rows;
  w->row_begin = row_begin;
  w->rows = row_count;
  w->columns = columns;
  w->blocks_per_row = nb;
  w->block_bytes = block_bytes;
  w->contract_bytes = shard_bytes;
  w->tiles = (row_count + kTileRows - 1) / kTileRows;
  w->slabs = (nb + kSlabBlocks - 1) / kSlabBlocks;
  w->seg_rows[0] = row_count;
  const size_t panel_bytes = w->panel_bytes();

  auto fail = [&](qx_status status) {
    qx_weights_destroy(w);
    return status;
  };
  cudaError_t err = cudaMalloc(reinterpret_cast<void**>(&w->panel), align_up(panel_bytes, 256));
  if (err != cudaSuccess) {
    set_last_error("cudaMalloc(prepared planes)", err);
    return fail(err == cudaErrorMemoryAllocation ? QX_STATUS_OUT_OF_MEMORY
                                                 : QX_STATUS_DEVICE_ERROR);
  }
  w->prepared_bytes = panel_bytes;

  const uint8_t* shard_src = static_cast<const uint8_t*>(contract) +
                             static_cast<size_t>(row_begin) * nb * block_bytes;
  void* temp = nullptr;
  const uint8_t* device_src = shard_src;
  if (!contract_on_device) {
    err = cudaMalloc(&temp, align_up(shard_bytes, 256));
    if (err != cudaSuccess) {
      set_last_error("cudaMalloc(canonical staging)", err);
      return fail(err == cudaErrorMemoryAllocation ? QX_STATUS_OUT_OF_MEMORY
                                                   : QX_STATUS_DEVICE_ERROR);
    }
    err = cudaMemcpyAsync(temp, shard_src, shard_bytes, cudaMemcpyHostToDevice, stream);
    if (err != cudaSuccess) {
      set_last_error("cudaMemcpyAsync(canonical bytes)", err);
      (void)cudaFree(temp);
      return fail(QX_STATUS_DEVICE_ERROR);
    }
    device_src = static_cast<const uint8_t*>(temp);
  }
  qx_status status =
      launch_relayout(w, device_src, stream);
  if (status == QX_STATUS_OK && (sync || temp != nullptr)) {
    err = cudaStreamSynchronize(stream);
    if (err != cudaSuccess) {
      set_last_error("cudaStreamSynchronize(prepare)", err);
      status = QX_STATUS_DEVICE_ERROR;
    }
  }
  if (temp != nullptr) (void)cudaFree(temp);
  if (status != QX_STATUS_OK) return fail(status);
  w->preparation_ns = static_cast<uint64_t>(
      std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - t0)
          .count());
  *out = w;
  return QX_STATUS_OK;
}

}  // namespace
}  // namespace qx

extern "C" {

qx_status qx_weights_prepare(int format, const void* contract_packed, long long rows,
                             long long columns, long long row_begin, long long row_count,
                             qx_weights** out) {
  qx::DeviceContext* ctx = nullptr;
  if (out == nullptr || contract_packed == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  QX_TRY(qx::validate_nk(format, rows, columns));
  QX_TRY(qx::current_context(&ctx));
  std::lock_guard<std::mutex> lock(ctx->mutex);
  return qx::prepare_common(format, contract_packed, false, rows, columns, row_begin, row_count,
                            ctx->stream, true, out);
}

qx_status qx_weights_prepare_fused(int format, const void* const* contract_packed,
                                   const long long* rows, int count, long long columns,
                                   qx_weights** out) {
  using namespace qx;
  const auto t0 = std::chrono::steady_clock::now();
  if (out == nullptr || contract_packed == nullptr || rows == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  *out = nullptr;
  if (count < 1 || count > qx_weights::kMaxSegments) return QX_STATUS_INVALID_ARGUMENT;
  size_t block_bytes = 0;
  if (!format_info(format, &block_bytes)) return QX_STATUS_UNSUPPORTED_FORMAT;
  long long total_rows = 0;
  for (int s = 0; s < count; ++s) {
    if (contract_packed[s] == nullptr) return QX_STATUS_INVALID_ARGUMENT;
    QX_TRY(validate_nk(format, rows[s], columns));
    size_t bytes = 0;
    QX_TRY(packed_bytes(format, rows[s], columns, &bytes));
    total_rows += rows[s];
  }
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  std::lock_guard<std::mutex> lock(ctx->mutex);
  const long long nb = columns / kBlockK;
  auto* w = new (std::nothrow) qx_weights();
  if (w == nullptr) return QX_STATUS_OUT_OF_MEMORY;
  w->format = format;
  w->device = ctx->device;
  w->rows_total = total_rows;
  w->rows = total_rows;
  w->columns = columns;
  w->blocks_per_row = nb;
  w->block_bytes = block_bytes;
  w->slabs = (nb + kSlabBlocks - 1) / kSlabBlocks;
  w->segments = count;
  size_t largest = 0;
  for (int s = 0; s < count; ++s) {
    w->seg_tile_begin[s] = w->tiles;
    w->seg_rows[s] = rows[s];
    w->tiles += (rows[s] + kTileRows - 1) / kTileRows;
    const size_t bytes = static_cast<size_t>(rows[s]) * nb * block_bytes;
    w->contract_bytes += bytes;
    largest = bytes > largest ? bytes : largest;
  }
  const size_t panel_bytes = w->panel_bytes();
  void* temp = nullptr;
  auto fail = [&](const char* what, cudaError_t err) {
    set_last_error(what, err);
    if (temp != nullptr) (void)cudaFree(temp);
    qx_weights_destroy(w);
    return err == cudaErrorMemoryAllocation ? QX_STATUS_OUT_OF_MEMORY : QX_STATUS_DEVICE_ERROR;
  };
  cudaError_t err = cudaMalloc(reinterpret_cast<void**>(&w->panel), align_up(panel_bytes, 256));
  if (err != cudaSuccess) return fail("cudaMalloc(prepared planes)", err);
  w->prepared_bytes = panel_bytes;
  err = cudaMalloc(&temp, align_up(largest, 256));
  if (err != cudaSuccess) return fail("cudaMalloc(canonical staging)", err);
  for (int s = 0; s < count; ++s) {
    const size_t bytes = static_cast<size_t>(rows[s]) * nb * block_bytes;
    err = cudaMemcpyAsync(temp, contract_packed[s], bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (err != cudaSuccess) return fail("cudaMemcpyAsync(canonical bytes)", err);
    const qx_status status = launch_relayout_segment(w, static_cast<const uint8_t*>(temp), rows[s],
                                                     w->seg_tile_begin[s], ctx->stream);
    if (status != QX_STATUS_OK) {
      (void)cudaFree(temp);
      qx_weights_destroy(w);
      return status;
    }
    // the staging buffer is reused by the next segment
    err = cudaStreamSynchronize(ctx->stream);
    if (err != cudaSuccess) return fail("cudaStreamSynchronize(prepare)", err);
  }
  (void)cudaFree(temp);
  w->preparation_ns = static_cast<uint64_t>(
      std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - t0)
          .count());
  *out = w;
  return QX_STATUS_OK;
}

qx_status qx_weights_prepare_dev(int format, const void* contract_packed_dev, long long rows,
                                 long long columns, long long row_begin, long long row_count,
                                 void* stream, qx_weights** out) {
  return qx::prepare_common(format, contract_packed_dev, true, rows, columns, row_begin,
                            row_count, static_cast<cudaStream_t>(stream), false, out);
}

qx_status qx_weights_get_info(const qx_weights* w, qx_weights_info* info) {
  if (w == nullptr || info == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  info->format = w->format;
  info->rows = w->rows;
  info->columns = w->columns;
  info->block_size = qx::kBlockK;
  info->blocks_per_row = w->blocks_per_row;
  info->block_bytes = w->block_bytes;
  info->contract_bytes = w->contract_bytes;
  info->prepared_bytes = w->prepared_bytes + w->dense_cache_bytes;
  info->memory_amplification =
      w->contract_bytes == 0 ? 0.0
                             : static_cast<double>(info->prepared_bytes) /
                                   static_cast<double>(w->contract_bytes);
  info->preparation_ns = w->preparation_ns;
  info->device = w->device;
  info->has_dense_bf16 = w->dense_cache != nullptr ? 1 : 0;
  info->row_tile = qx::kTileRows;
  info->panel_bytes = w->panel_bytes();
  return QX_STATUS_OK;
}

const void* qx_weights_panel_dev(const qx_weights* w) { return w == nullptr ? nullptr : w->panel; }

void qx_weights_destroy(qx_weights* w) {
  if (w == nullptr) return;
  if (w->panel != nullptr) (void)cudaFree(w->panel);
  if (w->dense_cache != nullptr) (void)cudaFree(w->dense_cache);
  delete w;
}

}  // extern "C"
