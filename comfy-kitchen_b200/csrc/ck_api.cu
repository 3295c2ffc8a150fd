// Library-level entry points: version, error text, device probe.
#include "ck_common.cuh"

#include <cstdlib>
#include <mutex>

namespace ck {

char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("CK_PDL");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

}  // namespace ck

extern "C" int ck_abi_version(void) { return CK_ABI_VERSION; }

extern "C" const char* ck_last_error(void) { return ck::last_error_buffer(); }

extern "C" int ck_device_supported(int device) {
  int major = 0;
  cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  if (e != cudaSuccess) {
    ck::fail(CK_ERR_CUDA, "cudaDeviceGetAttribute failed: %s", cudaGetErrorString(e));
    return -CK_ERR_CUDA;
  }
  return major == 10 ? 1 : 0;
}
