// Library-level entry points: version, error text, device check, launch counter.
#include "common.cuh"

namespace ulm {

std::atomic<uint64_t> g_launches{0};

char* err_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(err_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}

}  // namespace ulm

extern "C" {

int ulm_abi_version(void) { return ULM_ABI_VERSION; }

const char* ulm_last_error(void) { return ulm::err_buf(); }

uint64_t ulm_launch_count(void) { return ulm::g_launches.load(std::memory_order_relaxed); }

int ulm_device_ok(int device) {
  cudaDeviceProp p;
  cudaError_t e = cudaGetDeviceProperties(&p, device);
  if (e != cudaSuccess) return ulm::fail(ULM_ERR_CUDA, "cudaGetDeviceProperties(%d): %s", device, cudaGetErrorString(e));
  if (p.major != 10 || p.minor != 0)
    return ulm::fail(ULM_ERR_DEVICE, "device %d is sm_%d%d; this library holds sm_100a code only", device, p.major, p.minor);
  return ULM_OK;
}

}  // extern "C"
