// Shared host-side helpers of the C-ABI library: thread-local error text,
// CUDA error mapping, launch counting.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/mac_b200.h"

namespace mac_b200 {

// Text behind mac_b200_last_error(); one buffer per host thread.
char* error_buffer();
constexpr int kErrorBufferBytes = 512;

int fail(int code, const char* fmt, ...);

inline int cuda_fail(cudaError_t err, const char* what) {
  return fail(MAC_B200_ECUDA, "%s: %s (%s)", what, cudaGetErrorString(err),
              cudaGetErrorName(err));
}

// Reads and clears the sticky status bits of the prefill ring-build kernels on
// the current device (the caller has synchronised the device).
int take_prefill_build_status(unsigned* bits);

// The same for the tensor-memory variant of the sink-exclusive build.
int take_prefill_sink_tc_status(unsigned* bits);

// Sink-exclusive prefill build on tcgen05 / tensor memory (validated arguments); sets
// *launched when it ran, leaves it false when this step has to take the mma.sync kernel.
int launch_prefill_sink_exclusive_tc(const ::MacB200PrefillBuildArgs& a, int sms, cudaStream_t stream,
                                     bool* launched);

// Multiprocessor count of a device, looked up once per device.
int device_sm_count(int device);

// Kernels launched by this process through the library (all entry points).
extern std::atomic<int64_t> g_kernel_launches;

#define MAC_REQUIRE(cond, ...)                        \
  do {                                                \
    if (!(cond)) return ::mac_b200::fail(MAC_B200_EINVAL, __VA_ARGS__); \
  } while (0)

#define MAC_CUDA(call)                                              \
  do {                                                              \
    cudaError_t _e = (call);                                        \
    if (_e != cudaSuccess) return ::mac_b200::cuda_fail(_e, #call); \
  } while (0)

}  // namespace mac_b200
