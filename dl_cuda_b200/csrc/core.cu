// Library-level pieces of the C ABI: status strings, the per-thread error
// text, the launch counter and the cached SM count.
#include "common.cuh"

#include <cstring>

namespace dlb {

std::atomic<uint64_t> g_launches{0};

namespace {
thread_local char t_error[512] = "";
}

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
}

int sm_count() {
  constexpr int kMaxDev = 64;
  static std::atomic<int> cached[kMaxDev];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

}  // namespace dlb

extern "C" int dlb_version(void) { return 100; }

extern "C" const char *dlb_status_string(int status) {
  switch (status) {
    case DLB_OK: return "ok";
    case DLB_ERR_INVALID_ARG: return "invalid argument";
    case DLB_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case DLB_ERR_UNSUPPORTED: return "unsupported shape";
    case DLB_ERR_CUDA: return "CUDA error";
    case DLB_ERR_NO_DEVICE: return "no CUDA device (there is no CPU fallback)";
    default: return "unknown status";
  }
}

extern "C" const char *dlb_last_error(void) { return dlb::t_error; }

extern "C" uint64_t dlb_launch_count(void) {
  return dlb::g_launches.load(std::memory_order_relaxed);
}
