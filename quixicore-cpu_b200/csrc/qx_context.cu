// Per-device context, device discovery, workspace arena and shape validation.
//
// Device discovery replaces the reference's CPUID/hwcap probing
// (src/runtime/cpu_features_x86_64.cpp:66-104): it reports the compute capability, SM
// count, memory sizes and which peers this device can map over NVLink / PCIe.

#include <cstring>
#include <limits>
#include <memory>
#include <string>

#include "qx_common.cuh"

namespace qx {

std::atomic<unsigned long long> g_launches{0};

namespace {
thread_local std::string tl_error;
std::mutex g_ctx_mutex;
std::unique_ptr<DeviceContext> g_contexts[64];
std::atomic<int> g_threads{1};
}  // namespace

void set_last_error(const char* where, cudaError_t code) {
  tl_error = std::string(where) + ": " + cudaGetErrorName(code) + " (" +
             cudaGetErrorString(code) + ")";
}
void set_last_error_text(const char* text) { tl_error = text; }

qx_status DeviceContext::ensure_staging(size_t bytes) {
  if (bytes <= staging_bytes) return QX_STATUS_OK;
  if (staging != nullptr) {
    QX_CUDA_TRY(cudaStreamSynchronize(stream));
    QX_CUDA_TRY(cudaFree(staging));
    staging = nullptr;
    staging_bytes = 0;
  }
  const size_t want = align_up(bytes + bytes / 4, 1 << 20);
  QX_CUDA_TRY(cudaMalloc(&staging, want));
  staging_bytes = want;
  return QX_STATUS_OK;
}

qx_status current_context(DeviceContext** out) {
  int device = -1;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
    (void)cudaGetLastError();
    set_last_error_text("no CUDA device is visible; this library has no CPU fallback");
    return QX_STATUS_DEVICE_ERROR;
  }
  QX_CUDA_TRY(cudaGetDevice(&device));
  if (device < 0 || device >= 64) {
    set_last_error_text("device ordinal out of range");
    return QX_STATUS_DEVICE_ERROR;
  }
  std::lock_guard<std::mutex> lock(g_ctx_mutex);
  if (!g_contexts[device]) {
    auto ctx = std::make_unique<DeviceContext>();
    ctx->device = device;
    QX_CUDA_TRY(cudaGetDeviceProperties(&ctx->prop, device));
    if (ctx->prop.major != 10) {
      set_last_error_text("device is not compute capability 10.x (B200); kernels are sm_100a only");
      return QX_STATUS_DEVICE_ERROR;
    }
    QX_CUDA_TRY(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
    QX_CUDA_TRY(cudaMalloc(&ctx->flag, 256));
    QX_CUDA_TRY(cudaMemset(ctx->flag, 0, 256));
    QX_CUDA_TRY(cudaHostAlloc(reinterpret_cast<void**>(&ctx->error_host), 64, cudaHostAllocMapped));
    ctx->error_host[0] = 0;
    QX_CUDA_TRY(cudaHostGetDevicePointer(reinterpret_cast<void**>(&ctx->error_dev), ctx->error_host, 0));
    ctx->workspace.device = device;
    g_contexts[device] = std::move(ctx);
  }
  *out = g_contexts[device].get();
  return QX_STATUS_OK;
}

DeviceContext* existing_context(int device) {
  if (device < 0 || device >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_ctx_mutex);
  return g_contexts[device].get();
}

bool valid_product3(long long a, long long b, long long c) {
  const long long dims[3] = {a, b, c};
  long long product = 1;
  for (long long d : dims) {
    if (d <= 0 || product > std::numeric_limits<long long>::max() / d) return false;
    product *= d;
  }
  return true;
}
bool valid_product2(long long a, long long b) { return valid_product3(a, b, 1); }

bool format_info(int format, size_t* block_bytes) {
  if (format == QX_FORMAT_Q8_0) { *block_bytes = 34; return true; }
  if (format == QX_FORMAT_Q4_0) { *block_bytes = 18; return true; }
  return false;
}

// src/dispatch/qgemv.cpp:125-141
qx_status validate_nk(int format, long long n, long long k) {
  size_t bytes = 0;
  if (!format_info(format, &bytes)) return QX_STATUS_UNSUPPORTED_FORMAT;
  if (n <= 0 || k <= 0 || k % kBlockK != 0) return QX_STATUS_INVALID_SHAPE;
  const long long max = std::numeric_limits<long long>::max();
  if (n > max / k || n > max / (k / kBlockK)) return QX_STATUS_INVALID_SHAPE;
  return QX_STATUS_OK;
}

// src/dispatch/qgemv.cpp:143-164
qx_status packed_bytes(int format, long long n, long long k, size_t* size) {
  size_t bytes = 0;
  if (!format_info(format, &bytes)) return QX_STATUS_UNSUPPORTED_FORMAT;
  const size_t rows = static_cast<size_t>(n);
  const size_t blocks_per_row = static_cast<size_t>(k / kBlockK);
  const size_t max = std::numeric_limits<size_t>::max();
  if (rows != 0 && blocks_per_row > max / rows) return QX_STATUS_INVALID_SHAPE;
  const size_t blocks = rows * blocks_per_row;
  if (blocks != 0 && bytes > max / blocks) return QX_STATUS_INVALID_SHAPE;
  *size = blocks * bytes;
  return QX_STATUS_OK;
}

}  // namespace qx

qx_status qx_workspace::reserve(size_t bytes) {
  if (bytes <= capacity) return QX_STATUS_OK;
  if (base != nullptr) {
    QX_CUDA_TRY(cudaDeviceSynchronize());
    QX_CUDA_TRY(cudaFree(base));
    base = nullptr;
    capacity = 0;
  }
  const size_t want = qx::align_up(bytes + bytes / 8, 1 << 20);
  QX_CUDA_TRY(cudaMalloc(&base, want));
  capacity = want;
  QX_CUDA_TRY(cudaMemset(base, 0, qx::kWorkspaceCounterBytes));
  return QX_STATUS_OK;
}

qx_workspace::~qx_workspace() {
  if (base != nullptr) (void)cudaFree(base);
}

extern "C" {

qx_status qx_workspace_create(size_t reserve_bytes, qx_workspace** out) {
  if (out == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  qx::DeviceContext* ctx = nullptr;
  QX_TRY(qx::current_context(&ctx));
  auto* ws = new (std::nothrow) qx_workspace();
  if (ws == nullptr) return QX_STATUS_OUT_OF_MEMORY;
  ws->device = ctx->device;
  const qx_status status = ws->reserve(reserve_bytes);
  if (status != QX_STATUS_OK) {
    delete ws;
    return status;
  }
  *out = ws;
  return QX_STATUS_OK;
}

size_t qx_workspace_capacity(const qx_workspace* workspace) {
  return workspace == nullptr ? 0 : workspace->capacity;
}

void qx_workspace_destroy(qx_workspace* workspace) { delete workspace; }

qx_status qx_device_query(qx_device_info* info) {
  if (info == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  std::memset(info, 0, sizeof *info);
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
    (void)cudaGetLastError();
    qx::set_last_error_text("no CUDA device is visible");
    return QX_STATUS_DEVICE_ERROR;
  }
  int device = 0;
  QX_CUDA_TRY(cudaGetDevice(&device));
  cudaDeviceProp prop{};
  QX_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
  info->device = device;
  info->sm_major = prop.major;
  info->sm_minor = prop.minor;
  info->sm_count = prop.multiProcessorCount;
  info->max_smem_per_block = static_cast<int>(prop.sharedMemPerBlockOptin);
  info->l2_bytes = prop.l2CacheSize;
  info->hbm_bytes = prop.totalGlobalMem;
  info->visible_devices = count;
  for (int peer = 0; peer < count && peer < 31; ++peer) {
    int can = peer == device ? 1 : 0;
    if (peer != device) (void)cudaDeviceCanAccessPeer(&can, device, peer);
    if (can) info->peer_access_mask |= 1 << peer;
    if (peer == device || !can || peer >= 16) continue;
    // Link class of the pair as the driver reports it (read-only queries): native atomics
    // over the link exist on NVLink / NVSwitch paths and not across PCIe; the performance
    // rank orders a device's peers by link quality (0 = best).
    int atomics = 0, rank = -1;
    if (cudaDeviceGetP2PAttribute(&atomics, cudaDevP2PAttrNativeAtomicSupported, device, peer) != cudaSuccess) {
      (void)cudaGetLastError();
      atomics = 0;
    }
    if (cudaDeviceGetP2PAttribute(&rank, cudaDevP2PAttrPerformanceRank, device, peer) != cudaSuccess) {
      (void)cudaGetLastError();
      rank = -1;
    }
    if (atomics) info->nvlink_peer_mask |= 1 << peer;
    info->peer_performance_rank[peer] = static_cast<signed char>(rank);
  }
  for (int peer = 0; peer < 16; ++peer) {
    if (!(info->peer_access_mask & (1 << peer)) || peer == device) info->peer_performance_rank[peer] = -1;
  }
  {
    int bits = 0;
    for (int peer = 0; peer < 31; ++peer) bits += (info->nvlink_peer_mask >> peer) & 1;
    info->nvlink_peers = bits;
    // every NVLink peer at the same (best) rank: a switched fabric, uniform bandwidth to all
    int uniform = bits > 0 ? 1 : 0;
    for (int peer = 0; peer < 16; ++peer) {
      if ((info->nvlink_peer_mask & (1 << peer)) && info->peer_performance_rank[peer] != 0) uniform = 0;
    }
    info->nvlink_uniform = uniform;
  }
  std::strncpy(info->name, prop.name, sizeof(info->name) - 1);
  return QX_STATUS_OK;
}

const char* qx_last_error_string(void) { return qx::tl_error.c_str(); }

void qx_set_num_threads(int n) { qx::g_threads.store(n < 1 ? 1 : (n > 512 ? 512 : n)); }
int qx_num_threads(void) { return qx::g_threads.load(); }

unsigned long long qx_kernel_launch_count(void) { return qx::g_launches.load(); }

}  // extern "C"
