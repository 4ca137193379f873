// Error reporting and device queries shared by every entry point of the C ABI.
#include "common.cuh"

#include <map>
#include <mutex>
#include <utility>

namespace lq {

char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(LQ_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  }
  return LQ_OK;
}

int sm_count() {
  static thread_local int cached_dev = -1, cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return kSmCount;
  if (dev != cached_dev) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = kSmCount;
    cached = n;
    cached_dev = dev;
  }
  return cached;
}

int ensure_smem_limit(const void* kernel, int bytes, const char* what) {
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, int> raised;  // (kernel, device) -> bytes granted
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return fail(LQ_ERR_LAUNCH, "%s: no current device", what);
  }
  std::lock_guard<std::mutex> lock(mu);
  auto key = std::make_pair(kernel, dev);
  auto it = raised.find(key);
  if (it != raised.end() && it->second >= bytes) return LQ_OK;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
    cudaGetLastError();
    return fail(LQ_ERR_LAUNCH, "%s: cannot raise the dynamic shared memory limit to %d bytes", what, bytes);
  }
  raised[key] = bytes;
  return LQ_OK;
}

}  // namespace lq

extern "C" int lq_version(void) { return 3; }
extern "C" const char* lq_last_error(void) { return lq::error_buffer(); }
