// Row-sharded decode across the GPUs of one node with the all-gather fused into the GEMV:
// peer-mappable buffers (CUDA IPC, one process per GPU), the pushing GEMV entry point and
// the kernel that waits for all ranks' slices. Semantics of all_gather in
// kernels/collectives/collectives_ref.cpp:26-37; the transport is plain peer stores from
// the GEMV's row finishers (qx_gemv_tc.cu), no cluster multicast and no remote loads.

#include <cstdlib>
#include <cstring>

#include "qx_gemv_tc.cuh"
#include "qx_sm100.cuh"
#include "qx_weights.cuh"

namespace qx {
namespace {

// control block of a rank: [0..7] slice-complete words (one per rank, written by that
// rank), [16] pushes completed here, [17] waits completed here, [18] CTAs done in the
// current launch
constexpr int kFlagWords = 8, kPushCountWord = 16, kWaitCountWord = 17, kLaunchCounterWord = 18;
constexpr size_t kControlBytes = 256;

// Lane r waits until rank r's slice of the next step has arrived (bounded), then lane 0
// advances the local wait counter.
__global__ void __launch_bounds__(32) allgather_wait_kernel(int* control, int world, int* error,
                                                            unsigned long long limit_ns) {
  // Launched programmatically: it may start while the GEMV in front of it still runs (it only
  // polls), and the kernel behind it may start its own set-up at once; whatever that kernel
  // reads of the gathered results it guards with griddepcontrol.wait, which returns when
  // this kernel has finished.
  asm volatile("griddepcontrol.launch_dependents;");
  // The wait counter is advanced by the previous wait kernel of this chain, which may still
  // be polling for a late peer when this one starts (the GEMV between the two triggers its
  // dependents at its start): read it only after everything in front has finished. The GEMV
  // in front sets this rank's own word at its very end, so this costs next to nothing.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int lane = threadIdx.x;
  const int expected = control[kWaitCountWord] + 1;
  bool ok = true;
  if (lane < world) {
    const unsigned long long start = sm100::global_timer_ns();
    for (;;) {
      int seen;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(control + lane) : "memory");
      if (seen - expected >= 0) break;
      if (sm100::global_timer_ns() - start > limit_ns) {
        ok = false;
        break;
      }
      // poll tightly while the slices are expected any moment, back off afterwards
      if (sm100::global_timer_ns() - start > 20000ull) __nanosleep(200);
    }
  }
  if (!ok) sm100::report_error(error, 31);
  __syncwarp();
  if (lane == 0) control[kWaitCountWord] = expected;
}

// Time limit of the wait kernel: 2 s, or QX_B200_WAIT_LIMIT_MS milliseconds (1..10000) when
// that is set in the environment (tests of the give-up path use a few milliseconds).
unsigned long long wait_limit_ns() {
  static const unsigned long long limit = []() -> unsigned long long {
    const char* text = std::getenv("QX_B200_WAIT_LIMIT_MS");
    if (text != nullptr) {
      const long ms = std::strtol(text, nullptr, 10);
      if (ms >= 1 && ms <= 10000) return static_cast<unsigned long long>(ms) * 1000000ull;
    }
    return sm100::kWaitLimitNs;
  }();
  return limit;
}

qx_status check_plan(const qx_push_plan* plan) {
  if (plan == nullptr || plan->world < 2 || plan->world > 8 || plan->rank < 0 ||
      plan->rank >= plan->world || plan->rows_per_rank <= 0 || plan->results_local == nullptr ||
      plan->control_local == nullptr) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  for (int r = 0; r < plan->world; ++r) {
    if (r != plan->rank && (plan->results_peer[r] == nullptr || plan->control_peer[r] == nullptr)) {
      return QX_STATUS_INVALID_ARGUMENT;
    }
  }
  return QX_STATUS_OK;
}

}  // namespace
}  // namespace qx

extern "C" {

size_t qx_push_control_bytes(void) { return qx::kControlBytes; }

qx_status qx_peer_alloc(size_t bytes, void** dev_ptr, unsigned char handle[64]) {
  using namespace qx;
  if (dev_ptr == nullptr || handle == nullptr || bytes == 0) return QX_STATUS_INVALID_ARGUMENT;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* ptr = nullptr;
  cudaError_t err = cudaMalloc(&ptr, align_up(bytes, 256));
  if (err != cudaSuccess) {
    set_last_error("cudaMalloc(peer buffer)", err);
    return err == cudaErrorMemoryAllocation ? QX_STATUS_OUT_OF_MEMORY : QX_STATUS_DEVICE_ERROR;
  }
  cudaIpcMemHandle_t ipc;
  if ((err = cudaMemset(ptr, 0, align_up(bytes, 256))) != cudaSuccess ||
      (err = cudaIpcGetMemHandle(&ipc, ptr)) != cudaSuccess) {
    set_last_error("cudaIpcGetMemHandle", err);
    (void)cudaFree(ptr);
    return QX_STATUS_DEVICE_ERROR;
  }
  memcpy(handle, &ipc, 64);
  *dev_ptr = ptr;
  return QX_STATUS_OK;
}

qx_status qx_peer_open(const unsigned char handle[64], void** dev_ptr) {
  using namespace qx;
  if (dev_ptr == nullptr || handle == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  cudaIpcMemHandle_t ipc;
  memcpy(&ipc, handle, 64);
  void* ptr = nullptr;
  const cudaError_t err = cudaIpcOpenMemHandle(&ptr, ipc, cudaIpcMemLazyEnablePeerAccess);
  if (err != cudaSuccess) {
    set_last_error("cudaIpcOpenMemHandle", err);
    return QX_STATUS_DEVICE_ERROR;
  }
  *dev_ptr = ptr;
  return QX_STATUS_OK;
}

qx_status qx_peer_close(void* dev_ptr) {
  if (dev_ptr == nullptr) return QX_STATUS_OK;
  const cudaError_t err = cudaIpcCloseMemHandle(dev_ptr);
  if (err != cudaSuccess) {
    qx::set_last_error("cudaIpcCloseMemHandle", err);
    return QX_STATUS_DEVICE_ERROR;
  }
  return QX_STATUS_OK;
}

qx_status qx_peer_free(void* dev_ptr) {
  if (dev_ptr == nullptr) return QX_STATUS_OK;
  const cudaError_t err = cudaFree(dev_ptr);
  if (err != cudaSuccess) {
    qx::set_last_error("cudaFree(peer buffer)", err);
    return QX_STATUS_DEVICE_ERROR;
  }
  return QX_STATUS_OK;
}

qx_status qx_qgemm_prepacked_push_dev(const qx_weights* weights, const float* x_dev, long long m,
                                      const qx_push_plan* plan, qx_workspace* workspace,
                                      void* stream) {
  using namespace qx;
  if (weights == nullptr || x_dev == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  QX_TRY(check_plan(plan));
  if (m <= 0 || m > kGemvMaxBatch || weights->rows != plan->rows_per_rank) return QX_STATUS_INVALID_SHAPE;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  // result buffer: [parity][world][m][rows_per_rank]; this rank writes slice `rank`
  const long long slice = m * plan->rows_per_rank;
  const long long parity_stride = static_cast<long long>(plan->world) * slice;
  const long long offset = static_cast<long long>(plan->rank) * slice;
  GemvPush push;
  push.peers = plan->world - 1;
  int* control = static_cast<int*>(plan->control_local);
  push.push_count = control + kPushCountWord;
  push.launch_counter = control + kLaunchCounterWord;
  push.own_flag = control + plan->rank;
  push.y_odd = plan->results_local + parity_stride + offset;
  int slot = 0;
  for (int r = 0; r < plan->world; ++r) {
    if (r == plan->rank) continue;
    push.y_peer[slot] = plan->results_peer[r] + offset;
    push.y_peer_odd[slot] = plan->results_peer[r] + parity_stride + offset;
    push.peer_flag[slot] = static_cast<int*>(plan->control_peer[r]) + plan->rank;
    ++slot;
  }
  return launch_qgemm_f32(weights, x_dev, plan->results_local + offset, m, plan->rows_per_rank,
                          workspace != nullptr ? workspace : &ctx->workspace,
                          static_cast<cudaStream_t>(stream), &push);
}

qx_status qx_allgather_wait_dev(const qx_push_plan* plan, long long m, long long step,
                                const float** results_dev, void* stream) {
  using namespace qx;
  QX_TRY(check_plan(plan));
  if (m <= 0 || step <= 0) return QX_STATUS_INVALID_ARGUMENT;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(1);
  config.blockDim = dim3(32);
  config.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  QX_CUDA_TRY(cudaLaunchKernelEx(&config, allgather_wait_kernel, static_cast<int*>(plan->control_local),
                                 plan->world, ctx->error_dev, wait_limit_ns()));
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  if (results_dev != nullptr) {
    const long long parity_stride = static_cast<long long>(plan->world) * m * plan->rows_per_rank;
    *results_dev = plan->results_local + (step & 1) * parity_stride;
  }
  return QX_STATUS_OK;
}

}  // extern "C"
