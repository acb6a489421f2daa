// Shared declarations of the qx_b200 library: status helpers, the per-device context
// (stream + default workspace), launch accounting and small device utilities.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <mutex>

#include "qx_b200.h"

namespace qx {

constexpr int kBlockK = 32;  // elements per q8_0 / q4_0 block
// Every workspace starts with this many bytes of arrival counters that kernels leave at
// zero when they finish; reserve() zeroes them whenever it (re)allocates.
constexpr size_t kWorkspaceCounterBytes = 1 << 20;

// ---- error reporting -------------------------------------------------------------
void set_last_error(const char* where, cudaError_t code);
void set_last_error_text(const char* text);

#define QX_CUDA_TRY(expr)                                  \
  do {                                                     \
    const cudaError_t qx_err_ = (expr);                    \
    if (qx_err_ != cudaSuccess) {                          \
      ::qx::set_last_error(#expr, qx_err_);                \
      return qx_err_ == cudaErrorMemoryAllocation          \
                 ? QX_STATUS_OUT_OF_MEMORY                 \
                 : QX_STATUS_DEVICE_ERROR;                 \
    }                                                      \
  } while (0)

#define QX_TRY(expr)                                       \
  do {                                                     \
    const qx_status qx_st_ = (expr);                       \
    if (qx_st_ != QX_STATUS_OK) return qx_st_;             \
  } while (0)

// Every kernel launch goes through this counter (qx_kernel_launch_count()).
extern std::atomic<unsigned long long> g_launches;
inline void count_launch(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// ---- device workspace (grow-only arena, mirrors quixicore_cpu::Workspace) ----------
}  // namespace qx

struct qx_workspace {
  int device = -1;
  void* base = nullptr;
  size_t capacity = 0;
  // Returns a 256-byte aligned device pointer valid until the next reserve() that
  // grows the arena. Growing synchronises the device (cudaFree of the old block).
  qx_status reserve(size_t bytes);
  ~qx_workspace();
};

namespace qx {

struct DeviceContext {
  int device = -1;
  cudaDeviceProp prop{};
  cudaStream_t stream = nullptr;  // used by the host-pointer entry points
  qx_workspace workspace;         // default workspace (NULL workspace argument)
  std::mutex mutex;               // serialises host-pointer calls on this device
  // staging buffers for host-pointer calls (grow-only)
  void* staging = nullptr;
  size_t staging_bytes = 0;
  int* flag = nullptr;            // device word for scale / finiteness checks
  // Error word of the tensor-core kernels (a bounded wait that gave up leaves its role code
  // there): pinned host memory the GPU can address, written only on that path, so the host
  // reads it after a synchronisation without a copy.
  int* error_host = nullptr;      // host address
  int* error_dev = nullptr;       // device address of the same word
  qx_status ensure_staging(size_t bytes);
};

// Context of the current CUDA device; creates it on first use. Fails with
// QX_STATUS_DEVICE_ERROR when no sm_100 device is usable.
qx_status current_context(DeviceContext** out);

// ---- shape validation shared by the entry points ------------------------------------
bool valid_product3(long long a, long long b, long long c);
bool valid_product2(long long a, long long b);
bool format_info(int format, size_t* block_bytes);
qx_status validate_nk(int format, long long n, long long k);
qx_status packed_bytes(int format, long long n, long long k, size_t* size);

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device attribute of a kernel: every
// device of the process that launches it needs its own opt-in. One instance of this guard
// per kernel (a function-local static at the launch site) remembers which devices have it.
struct SmemOptIn {
  std::mutex mutex;
  bool done[64] = {};
  template <class Kernel>
  qx_status ensure(Kernel kernel, size_t bytes) {
    int device = -1;
    QX_CUDA_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= 64) return QX_STATUS_DEVICE_ERROR;
    std::lock_guard<std::mutex> lock(mutex);
    if (!done[device]) {
      QX_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(bytes)));
      done[device] = true;
    }
    return QX_STATUS_OK;
  }
};

// Context of `device` if one exists already; never creates (and so never allocates).
DeviceContext* existing_context(int device);

}  // namespace qx
