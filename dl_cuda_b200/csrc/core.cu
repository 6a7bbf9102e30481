// Library-level pieces of the C ABI: status strings, the per-thread error
// text, the launch counter and the cached SM count.
#include "common.cuh"
#include "tma.cuh"

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

// Tuning options (dlb_set_option): 0 = the built-in heuristic decides.
namespace {
struct Option {
  const char *name;
  std::atomic<int> value;
};
Option g_options[] = {
    {"gather_rows_in_flight", {0}},     // 4 or 8 table rows loaded per thread before the first store
    {"gather_variant", {0}},            // 1: rows in registers, 2: the bulk-copy (TMA) pipeline
    {"gather_bulk_waves", {0}},         // grid of the bulk-copy gather in units of the CTAs that fit the GPU (default 4)
    {"gather_bulk_ctas_per_sm", {0}},   // 1: one CTA per SM with a deeper ring (default 2)
    {"ln_bwd_pipe", {0}},               // 1: never the bulk-copy pipeline, 2: whenever the shape allows
    {"ln_bwd_pipe_threads", {0}},       // column threads per CTA: 128, 256 or 512
    {"ln_bwd_pipe_ctas_per_sm", {0}},   // 1 or 2
    {"ln_bwd_pipe_rows_per_tile", {0}}, // 1, 2, 4 or 8
    {"act_bwd_partial_rows", {0}},      // upper bound of the partial rows of a fused bias gradient
    {"scatter_variant", {0}},           // 1: rows in registers, 2: the bulk-copy (TMA) pipeline
    {"scatter_bulk_ctas_per_sm", {0}},  // ring sized for this many CTAs per SM (default 3)
    {"scatter_zero_kernel", {0}},       // 1: empty rows are cleared by a kernel of their own before the scatter-add
    {"embed_push_period", {0}},         // one CTA in this many pushes rows over NVLink, the others clear rows
    {"embed_peer_phases", {0}},         // 1: only the local sums, 2: only the push of dlb_embed_scatter_bwd_peer
};
}  // namespace

int get_option(const char *name) {
  for (Option &o : g_options)
    if (strcmp(o.name, name) == 0) return o.value.load(std::memory_order_relaxed);
  return 0;
}

__device__ unsigned int g_wait_timeouts = 0;

unsigned int *wait_timeouts_counter() {
  constexpr int kMaxDev = 64;
  static std::atomic<unsigned int *> cached[kMaxDev];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
  unsigned int *p = cached[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    void *addr = nullptr;
    if (cudaGetSymbolAddress(&addr, g_wait_timeouts) != cudaSuccess) return nullptr;
    p = static_cast<unsigned int *>(addr);
    cached[dev].store(p, std::memory_order_release);
  }
  return p;
}

}  // namespace dlb

extern "C" int dlb_pipeline_timeouts(unsigned int *h_count) {
  DLB_REQUIRE(h_count != nullptr, DLB_ERR_INVALID_ARG, "pipeline_timeouts: null pointer");
  unsigned int *p = dlb::wait_timeouts_counter();
  DLB_REQUIRE(p != nullptr, DLB_ERR_NO_DEVICE, "pipeline_timeouts: no CUDA device");
  // Every stream of the device, non-blocking ones included, has to drain first: a plain
  // cudaMemcpy only orders itself after the legacy default stream.
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(h_count, p, sizeof(unsigned int), cudaMemcpyDeviceToHost);
  DLB_REQUIRE(e == cudaSuccess, DLB_ERR_CUDA, "pipeline_timeouts: %s", cudaGetErrorString(e));
  return DLB_OK;
}

extern "C" int dlb_set_option(const char *name, int value) {
  DLB_REQUIRE(name != nullptr, DLB_ERR_INVALID_ARG, "set_option: null name");
  for (dlb::Option &o : dlb::g_options) {
    if (strcmp(o.name, name) == 0) {
      o.value.store(value, std::memory_order_relaxed);
      return DLB_OK;
    }
  }
  dlb::set_error("set_option: unknown option '%s'", name);
  return DLB_ERR_INVALID_ARG;
}

extern "C" int dlb_version(void) { return 101; }

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
