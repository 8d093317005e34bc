// Error text, ABI version and launch counter shared by the entry points.
#include "mac_b200_common.h"

#include <cstring>

namespace mac_b200 {

std::atomic<int64_t> g_kernel_launches{0};

char* error_buffer() {
  static thread_local char buf[kErrorBufferBytes] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), kErrorBufferBytes, fmt, ap);
  va_end(ap);
  return code;
}

int device_sm_count(int device) {
  static std::atomic<int> cached[64];
  if (device < 0 || device >= 64) return 148;
  int v = cached[device].load(std::memory_order_relaxed);
  if (v <= 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || v <= 0)
      v = 148;   // B200; only used to cap grids
    cached[device].store(v, std::memory_order_relaxed);
  }
  return v;
}

}  // namespace mac_b200

extern "C" const char* mac_b200_last_error(void) { return mac_b200::error_buffer(); }

extern "C" int mac_b200_abi_version(void) { return MAC_B200_ABI_VERSION; }
