// Shared device/host helpers for the sm_100a layer kernels: 16-byte vector
// access with streaming cache hints, storage-type traits (fp32 / bf16 storage,
// fp32 arithmetic), warp reductions, and the status/launch bookkeeping that
// the C ABI reports through.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "../../include/dlcuda_b200.h"

namespace dlb {

// ---------------------------------------------------------------- host side
void set_error(const char *fmt, ...);
extern std::atomic<uint64_t> g_launches;
int sm_count();  // SMs of the current device (cached per device)
int get_option(const char *name);  // value set through dlb_set_option, 0 if unset

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

inline bool aligned16(const void *p) {
  return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

// Every launch goes through this: counts it and turns a launch error into a
// status instead of leaving it for the next runtime call to trip over.
#define DLB_LAUNCH_CHECK(name)                                                  \
  do {                                                                          \
    ::dlb::g_launches.fetch_add(1, std::memory_order_relaxed);                  \
    cudaError_t e__ = cudaGetLastError();                                       \
    if (e__ != cudaSuccess) {                                                   \
      ::dlb::set_error("%s: launch failed: %s", name, cudaGetErrorString(e__)); \
      return DLB_ERR_CUDA;                                                      \
    }                                                                           \
  } while (0)

#define DLB_REQUIRE(cond, status, ...) \
  do {                                 \
    if (!(cond)) {                     \
      ::dlb::set_error(__VA_ARGS__);   \
      return status;                   \
    }                                  \
  } while (0)

// Launch with programmatic dependent launch allowed: the launch is set up while
// the previous kernel of the stream runs and the grid starts as that kernel's
// CTAs exit.  Every kernel of this library starts with pdl_prologue(), which
// waits until all earlier work of the stream has completed and is visible, so
// only launch latency overlaps, never data.
//
// One rule follows for every kernel launched this way: it lives while earlier
// kernels of the stream still write, so it must not read anything a kernel may
// have written through the non-coherent path (ld.global.nc: __ldg, or any load
// through a `const T *__restrict__` parameter, which the compiler turns into
// one).  Such a load is not ordered by griddepcontrol.wait and was seen to
// return the previous contents of a buffer.  Activations, gradients, partial
// sums, sort plans AND parameters (the optimizer kernels write them) are read
// with ordinary loads; only tables that no kernel ever writes (the positional
// encoding) use ld_const_f4.
template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                       Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  (void)cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);  // errors surface in DLB_LAUNCH_CHECK
}

// Plain stream-ordered launch (no programmatic overlap with the previous kernel).
template <typename... KArgs, typename... Args>
inline void launch_plain(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                         Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  (void)cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

template <typename T>
inline T ceil_div(T a, T b) {
  return (a + b - 1) / b;
}

// -------------------------------------------------------------- device side
constexpr int kWarp = 32;
constexpr int kMaxPeers = DLB_MAX_PEERS;  // most ranks (GPUs of one node) the peer-memory entry points take

// First statement of every kernel: wait for everything launched before this
// kernel.  A kernel does NOT release its successor early
// (griddepcontrol.launch_dependents): the successor's CTAs then become resident,
// waiting, while this grid still has CTAs to start, and hold the slots those
// need.  On B200 the early release cost the ten-kernel block chain 5 % (1.653
// against 1.566 ms per step at 32768 x 4096, bf16) and made every kernel with
// a shared-memory ring slower inside the chain than the form it replaces.
// Releasing early only from grids no larger than the SM count (whose CTAs are
// all running by then) was slower as well: 0.511 against 0.493 ms per step of
// the same chain at 8192 token rows.
__device__ __forceinline__ void pdl_prologue() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Storage traits: a 16-byte vector holds kPerVec elements of storage type T.
template <typename T>
struct Store;

template <>
struct Store<float> {
  static constexpr int kPerVec = 4;
  __device__ __forceinline__ static void unpack(const uint4 &v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
  }
  __device__ __forceinline__ static uint4 pack(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]),
                      __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  __device__ __forceinline__ static float to_float(float v) { return v; }
  __device__ __forceinline__ static float from_float(float v) { return v; }
};

template <>
struct Store<__nv_bfloat16> {
  static constexpr int kPerVec = 8;
  __device__ __forceinline__ static void unpack(const uint4 &v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      // bf16 -> fp32 is a 16-bit shift; the low half of the word is element 2i.
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ __forceinline__ static uint4 pack(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t *>(&p);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  __device__ __forceinline__ static float to_float(__nv_bfloat16 v) {
    return __bfloat162float(v);
  }
  __device__ __forceinline__ static __nv_bfloat16 from_float(float v) {
    return __float2bfloat16_rn(v);
  }
};

// Streaming (touch-once) 16-byte accesses: evict-first in L1/L2 so that the
// small reused operands (gamma, beta, bias, PE rows, hot table rows) stay put.
__device__ __forceinline__ uint4 ld_stream(const void *p) {
  return __ldcs(reinterpret_cast<const uint4 *>(p));
}
__device__ __forceinline__ void st_stream(void *p, const uint4 &v) {
  __stcs(reinterpret_cast<uint4 *>(p), v);
}
// 32-byte streaming store (sm_100 256-bit global access): one lane writes a whole
// 32-byte sector, where two 16-byte stores with a 32-byte lane stride would each
// write half of it.  p must be 32-byte aligned.
__device__ __forceinline__ void st_stream32(float *p, const float (&f)[8]) {
  asm volatile("st.global.cs.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(f[0]), "f"(f[1]),
               "f"(f[2]), "f"(f[3]), "f"(f[4]), "f"(f[5]), "f"(f[6]), "f"(f[7])
               : "memory");
}
inline bool aligned32(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }

// Cached (L1-allocating, coherent) 16-byte access for operands that are reused across rows.
__device__ __forceinline__ uint4 ld_keep(const void *p) {
  return *reinterpret_cast<const uint4 *>(p);
}
__device__ __forceinline__ float4 ld_keep_f4(const float *p) {
  return *reinterpret_cast<const float4 *>(p);
}
// Coherent scalar load of data another kernel of the stream produced.
template <typename V>
__device__ __forceinline__ V ld_co(const V *p) {
  return *p;
}
// Non-coherent 16-byte load: ONLY for tables no kernel writes (see launch_pdl).
__device__ __forceinline__ float4 ld_const_f4(const float *p) {
  return __ldg(reinterpret_cast<const float4 *>(p));
}

// Nanoseconds of the GPU's wall clock, for bounding waits.
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace dlb
