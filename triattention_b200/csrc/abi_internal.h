// Error plumbing shared by the C-ABI entry points.  Every entry point returns 0 on success or a
// negative code; the message is kept per host thread and read with tri_last_error().
// The reference raises RuntimeError from TORCH_CHECK / C10_CUDA_KERNEL_LAUNCH_CHECK
// (triattention/kernels/cuda/common_host.cuh:4-13,24); the Python shim turns these codes into the
// same exception type.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

enum TriStatus : int { TRI_OK = 0, TRI_ERR_ARGUMENT = -1, TRI_ERR_CUDA = -2, TRI_ERR_DEVICE = -3 };

void tri_set_error(const char* what);
int tri_launch_status(const char* where);

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

#define TRI_CHECK(cond, msg)             \
  do {                                   \
    if (!(cond)) {                       \
      tri_set_error(msg);                \
      return TRI_ERR_ARGUMENT;           \
    }                                    \
  } while (0)

#define TRI_CUDA(call, where)                 \
  do {                                        \
    cudaError_t e_ = (call);                  \
    if (e_ != cudaSuccess) {                  \
      tri_set_error(cudaGetErrorString(e_));  \
      (void)where;                            \
      return TRI_ERR_CUDA;                    \
    }                                         \
  } while (0)

// One-time configuration that CUDA keeps per device and context (the opt-in to more than 48 KB of dynamic shared
// memory of a kernel): remembered per device ordinal, so that a process driving several GPUs configures each of
// them.  Two host threads making their first call on a device at the same time both set the same attribute
// value, which is harmless; the flags are atomics so that neither reads a torn value.
#include <atomic>
struct TriPerDevice {
  static constexpr int MaxDevices = 64;
  std::atomic<bool> done[MaxDevices];
  // returns the current device's ordinal if it still needs configuring, -1 if it is configured, -2 on error
  int pending() {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MaxDevices) return -2;
    return done[device].load(std::memory_order_acquire) ? -1 : device;
  }
  void mark(int device) { done[device].store(true, std::memory_order_release); }
};

// Launch with programmatic stream serialisation: the kernel may become resident while its predecessor in
// the stream is still running and orders itself with grid_dependency_wait() (common.cuh).  Hides the
// launch latency between kernels that follow one another in a stream.
template <typename... Params, typename... Args>
static inline cudaError_t launch_chained(void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared, cudaStream_t stream,
                                         Args... args) {
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = shared; cfg.stream = stream;
  cfg.attrs = &attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}
