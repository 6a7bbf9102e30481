// Bias + ReLU / Sigmoid / Tanh / GELU epilogues, forward and backward, for
// sm_100a.  Pure streaming kernels: each thread owns one 16-byte column vector
// of a [rows, cols] tensor and walks down its rows four at a time, so the bias
// stays in registers, the bias gradient is a register accumulator, and four
// independent 16-byte loads per operand are in flight per thread.
//
// What backward needs is written by forward in the same pass instead of by a
// device-to-device copy: ReLU keeps one bit per element (bit i of the cache is
// element i, little-endian inside each byte), Sigmoid/Tanh keep y, GELU keeps
// the pre-activation.
//
// The arithmetic is spelled exactly as in dl-cuda's kernels
// (src/activation.cuh:5-55, 203-226) so that fp32 results carry the same bits.
#include "common.cuh"
#include "reduce.cuh"

namespace dlb {
namespace {

constexpr int kBlock = 256;
constexpr int kUnroll = 4;
constexpr int kActNone = -1;  // identity: used for the stand-alone bias gradient

template <int KIND>
__device__ __forceinline__ float act_forward(float x) {
  if constexpr (KIND == DLB_ACT_RELU) {
    return (x > 0.0f) ? x : 0.0f;
  } else if constexpr (KIND == DLB_ACT_SIGMOID) {
    return 1.0f / (1.0f + expf(-x));
  } else if constexpr (KIND == DLB_ACT_TANH) {
    return tanhf(x);
  } else {
    float cdf = 0.5f * (1.0f + tanhf(0.7978845608f * (x + 0.044715f * x * x * x)));
    return x * cdf;
  }
}

// c is what forward cached: y for Sigmoid/Tanh, the pre-activation for GELU,
// 1.0f/0.0f (from the bit) for ReLU.
template <int KIND>
__device__ __forceinline__ float act_backward(float dy, float c) {
  if constexpr (KIND == kActNone) {
    return dy;
  } else if constexpr (KIND == DLB_ACT_RELU) {
    return dy * c;
  } else if constexpr (KIND == DLB_ACT_SIGMOID) {
    float s = c;
    return dy * s * (1.0f - s);
  } else if constexpr (KIND == DLB_ACT_TANH) {
    float t = c;
    return dy * (1.0f - t * t);
  } else {
    float x = c;
    float x3 = x * x * x;
    float inner = 0.7978845608f * (x + 0.044715f * x3);
    float tanh_val = tanhf(inner);
    float sech2 = 1.0f - tanh_val * tanh_val;
    float d_inner = 0.7978845608f * (1.0f + 0.134145f * x * x);
    float cdf = 0.5f * (1.0f + tanh_val);
    return dy * (cdf + x * 0.5f * sech2 * d_inner);
  }
}

// Geometry shared by forward and backward.  blockDim = (tx, ty), tx*ty = 256:
// tx adjacent threads cover tx adjacent column vectors of one row, ty rows are
// in flight per step, kUnroll steps are unrolled.  grid = (column blocks, row
// chunks); a CTA owns rows [by*rows_per_cta, (by+1)*rows_per_cta).
struct Tiling {
  dim3 block, grid;
  int64_t rows_per_cta;
};

// ctas_per_sm: how many CTAs per SM the grid aims at (more, smaller CTAs stream better).
// tx_cap: widest CTA in column vectors.  With a bias gradient every CTA row adds a partial row of
// column sums to write and reduce, so backward uses narrow CTAs (64 vectors wide, 4 rows deep):
// the same number of CTAs then makes 4x fewer partial rows (measured at 32768 x 16384 bf16:
// 374 us with 256-wide CTAs, 351 us with 64-wide ones).
// max_gy > 0 bounds the CTA rows (= partial rows of a fused bias gradient).
Tiling make_tiling(int64_t rows, int64_t ncv, int ctas_per_sm, int tx_cap = kBlock, int64_t gy_cap = 0) {
  Tiling t;
  int tx = 2;  // never 1: fp32 ReLU pairs adjacent lanes to build one mask byte
  while (tx < tx_cap && tx < ncv) tx *= 2;
  const int ty = kBlock / tx;
  t.block = dim3(tx, ty);
  const int64_t gx = ceil_div<int64_t>(ncv, tx);
  const int64_t step = static_cast<int64_t>(ty) * kUnroll;
  const int64_t max_gy = ceil_div<int64_t>(rows, step);
  int64_t gy = ceil_div<int64_t>(static_cast<int64_t>(sm_count()) * ctas_per_sm, gx);
  if (gy > max_gy) gy = max_gy;
  if (gy_cap > 0 && gy > gy_cap) gy = gy_cap;
  if (gy > 65535) gy = 65535;
  if (gy < 1) gy = 1;
  t.rows_per_cta = ceil_div<int64_t>(ceil_div<int64_t>(rows, gy), step) * step;
  gy = ceil_div<int64_t>(rows, t.rows_per_cta);
  t.grid = dim3(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
  return t;
}

// Mask byte for the 8 elements starting at element offset `off` (a multiple of
// the vector width).  bf16: a thread's vector is 8 elements, one byte.  fp32: a
// thread holds 4 bits; the even lane of each pair stores both nibbles.
template <int E>
__device__ __forceinline__ void store_mask(uint8_t *mask, size_t off, uint32_t bits, bool valid) {
  if constexpr (E == 8) {
    if (valid) mask[off >> 3] = static_cast<uint8_t>(bits);
  } else {
    const uint32_t other = __shfl_xor_sync(0xffffffffu, bits, 1);
    if (valid && (threadIdx.x & 1) == 0) mask[off >> 3] = static_cast<uint8_t>(bits | (other << 4));
  }
}

template <int E>
__device__ __forceinline__ uint32_t load_mask(const uint8_t *mask, size_t off) {
  const uint32_t byte = __ldcs(mask + (off >> 3));
  if constexpr (E == 8) return byte;
  return (byte >> ((off & 4) ? 4 : 0)) & 0xfu;
}

// I is the element-index type: int when every index fits 31 bits (fewer registers), else int64_t.
template <typename T, int KIND, typename I>
__global__ void __launch_bounds__(kBlock, 4)
act_fwd_kernel(const T *x, const float *bias, T *y, void *cache, I rows,
               I cols, I n, I rows_per_cta) {
  pdl_prologue();
  using S = Store<T>;
  constexpr int E = S::kPerVec;
  const I ncv = cols / E;
  const I cv = static_cast<I>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool col_ok = cv < ncv;
  const int ty = blockDim.y;

  const bool has_bias = bias != nullptr;
  float bv[E];
#pragma unroll
  for (int e = 0; e < E; e++) bv[e] = 0.f;
  if (has_bias && col_ok) {
#pragma unroll
    for (int q = 0; q < E / 4; q++) {
      const float4 b4 = ld_keep_f4(bias + cv * E + 4 * q);
      bv[4 * q] = b4.x; bv[4 * q + 1] = b4.y; bv[4 * q + 2] = b4.z; bv[4 * q + 3] = b4.w;
    }
  }

  const I r_begin = static_cast<I>(blockIdx.y) * rows_per_cta;
  const I r_end = (rows < r_begin + rows_per_cta ? rows : r_begin + rows_per_cta);
  for (I r0 = r_begin; r0 < r_end; r0 += static_cast<I>(ty) * kUnroll) {
    uint4 in[kUnroll];
    I off[kUnroll];
    bool ok[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; u++) {
      const I r = r0 + u * ty + threadIdx.y;
      off[u] = r * cols + cv * E;
      ok[u] = col_ok && r < r_end && off[u] + E <= n;
      if (ok[u]) in[u] = ld_stream(x + off[u]);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; u++) {
      float v[E], out[E];
      uint32_t bits = 0;
      if (ok[u]) {
        S::unpack(in[u], v);
#pragma unroll
        for (int e = 0; e < E; e++) {
          // Without a bias the value passes through untouched (x + 0.0f would turn -0.0f into +0.0f).
          const float pre = has_bias ? v[e] + bv[e] : v[e];
          v[e] = pre;
          out[e] = act_forward<KIND>(pre);
          if (KIND == DLB_ACT_RELU && pre > 0.0f) bits |= 1u << e;
        }
        st_stream(y + off[u], S::pack(out));
      }
      if (cache != nullptr) {
        if constexpr (KIND == DLB_ACT_RELU) {
          store_mask<E>(static_cast<uint8_t *>(cache), off[u], bits, ok[u]);
        } else if constexpr (KIND == DLB_ACT_GELU) {
          if (ok[u]) st_stream(static_cast<T *>(cache) + off[u], S::pack(v));
        } else {
          if (ok[u]) st_stream(static_cast<T *>(cache) + off[u], S::pack(out));
        }
      }
    }
  }
}

// partial (when non-null) is [gridDim.y][cols]: the CTA's column sums of dx.
template <typename T, int KIND, typename I>
__global__ void __launch_bounds__(kBlock, 4)
act_bwd_kernel(const T *dy, const void *cache, T *dx, float *__restrict__ partial, I rows,
               I cols, I n, I rows_per_cta) {
  pdl_prologue();
  using S = Store<T>;
  constexpr int E = S::kPerVec;
  __shared__ float colacc[kBlock * E];  // [ty][tx*E]
  const I ncv = cols / E;
  const I cv = static_cast<I>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool col_ok = cv < ncv;
  const int ty = blockDim.y;

  float acc[E];
#pragma unroll
  for (int e = 0; e < E; e++) acc[e] = 0.f;

  const I r_begin = static_cast<I>(blockIdx.y) * rows_per_cta;
  const I r_end = (rows < r_begin + rows_per_cta ? rows : r_begin + rows_per_cta);
  for (I r0 = r_begin; r0 < r_end; r0 += static_cast<I>(ty) * kUnroll) {
    uint4 g[kUnroll], c[kUnroll];
    uint32_t bits[kUnroll];
    I off[kUnroll];
    bool ok[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; u++) {
      const I r = r0 + u * ty + threadIdx.y;
      off[u] = r * cols + cv * E;
      ok[u] = col_ok && r < r_end && off[u] + E <= n;
      if (ok[u]) {
        g[u] = ld_stream(dy + off[u]);
        if constexpr (KIND == DLB_ACT_RELU) {
          bits[u] = load_mask<E>(static_cast<const uint8_t *>(cache), off[u]);
        } else if constexpr (KIND != kActNone) {
          c[u] = ld_stream(static_cast<const T *>(cache) + off[u]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; u++) {
      if (ok[u]) {
        float gv[E], cvv[E], out[E];
        S::unpack(g[u], gv);
        if constexpr (KIND == DLB_ACT_RELU) {
#pragma unroll
          for (int e = 0; e < E; e++) cvv[e] = ((bits[u] >> e) & 1u) ? 1.0f : 0.0f;
        } else if constexpr (KIND != kActNone) {
          S::unpack(c[u], cvv);
        } else {
#pragma unroll
          for (int e = 0; e < E; e++) cvv[e] = 0.f;
        }
#pragma unroll
        for (int e = 0; e < E; e++) {
          out[e] = act_backward<KIND>(gv[e], cvv[e]);
          acc[e] += out[e];
        }
        if (dx != nullptr) st_stream(dx + off[u], S::pack(out));
      }
    }
  }

  if (partial != nullptr) {
    const int tx = blockDim.x;
#pragma unroll
    for (int e = 0; e < E; e++) colacc[(threadIdx.y * tx + threadIdx.x) * E + e] = acc[e];
    __syncthreads();
    if (threadIdx.y == 0 && col_ok) {
#pragma unroll
      for (int e = 0; e < E; e++) {
        float t = 0.f;
        for (int yy = 0; yy < ty; yy++) t += colacc[(yy * tx + threadIdx.x) * E + e];
        partial[static_cast<size_t>(blockIdx.y) * cols + cv * E + e] = t;
      }
    }
  }
}

// Any shape, any alignment: a thread owns 8 consecutive elements (one mask
// byte) and handles them one at a time.
template <typename T, int KIND>
__global__ void __launch_bounds__(kBlock)
act_fwd_scalar_kernel(const T *x, const float *bias, T *y, void *cache, int64_t cols,
                      int64_t n) {
  pdl_prologue();
  using S = Store<T>;
  const int64_t i0 = (static_cast<int64_t>(blockIdx.x) * kBlock + threadIdx.x) * 8;
  if (i0 >= n) return;
  uint32_t bits = 0;
  for (int e = 0; e < 8 && i0 + e < n; e++) {
    const int64_t i = i0 + e;
    float pre = S::to_float(x[i]);
    if (bias != nullptr) pre = pre + bias[i % cols];
    const float out = act_forward<KIND>(pre);
    if (pre > 0.0f) bits |= 1u << e;
    y[i] = S::from_float(out);
    if (cache != nullptr) {
      if constexpr (KIND == DLB_ACT_GELU) static_cast<T *>(cache)[i] = S::from_float(pre);
      if constexpr (KIND == DLB_ACT_SIGMOID || KIND == DLB_ACT_TANH)
        static_cast<T *>(cache)[i] = S::from_float(out);
    }
  }
  if (KIND == DLB_ACT_RELU && cache != nullptr)
    static_cast<uint8_t *>(cache)[i0 >> 3] = static_cast<uint8_t>(bits);
}

template <typename T, int KIND>
__global__ void __launch_bounds__(kBlock)
act_bwd_scalar_kernel(const T *dy, const void *cache, T *dx, int64_t n) {
  pdl_prologue();
  using S = Store<T>;
  const int64_t i0 = (static_cast<int64_t>(blockIdx.x) * kBlock + threadIdx.x) * 8;
  if (i0 >= n) return;
  uint32_t bits = 0;
  if (KIND == DLB_ACT_RELU) bits = static_cast<const uint8_t *>(cache)[i0 >> 3];
  for (int e = 0; e < 8 && i0 + e < n; e++) {
    const int64_t i = i0 + e;
    float c;
    if constexpr (KIND == DLB_ACT_RELU)
      c = ((bits >> e) & 1u) ? 1.0f : 0.0f;
    else
      c = S::to_float(static_cast<const T *>(cache)[i]);
    dx[i] = S::from_float(act_backward<KIND>(S::to_float(dy[i]), c));
  }
}

// Column sums of a [rows, cols] tensor for shapes the vector path cannot take:
// one thread per column, a CTA row chunk summed top to bottom.
template <typename T>
__global__ void __launch_bounds__(kBlock)
colsum_scalar_kernel(const T *v, float *__restrict__ partial, int64_t rows,
                     int64_t cols, int64_t rows_per_chunk) {
  pdl_prologue();
  using S = Store<T>;
  const int64_t col = static_cast<int64_t>(blockIdx.x) * kBlock + threadIdx.x;
  if (col >= cols) return;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * rows_per_chunk;
  const int64_t r1 = min(rows, r0 + rows_per_chunk);
  float t = 0.f;
  for (int64_t r = r0; r < r1; r++) t += S::to_float(v[r * cols + col]);
  partial[static_cast<size_t>(blockIdx.y) * cols + col] = t;
}

constexpr int64_t kScalarRowsPerChunk = 256;
constexpr int64_t kFlatCols = 4096;  // virtual row width for tensors without bias

int64_t partial_rows_bound(int64_t rows) {
  // Vector path: gy <= sm*64/gx <= sm*64; scalar path: rows/256.  Bound both.
  const int64_t a = static_cast<int64_t>(sm_count()) * 64;
  const int64_t b = ceil_div<int64_t>(rows, kScalarRowsPerChunk);
  return a > b ? a : b;
}

template <typename T>
bool vector_ok(bool flat, int64_t cols, int64_t n, const void *p0, const void *p1, const void *p2,
               const void *p3) {
  // Multiples of 8: whole vectors per row, and (fp32) lane pairs share a mask
  // byte.  A flat tensor (no bias, no dbias) is re-tiled, so only n matters.
  return (flat || cols % 8 == 0) && n % 8 == 0 && aligned16(p0) && aligned16(p1) &&
         (p2 == nullptr || aligned16(p2)) && (p3 == nullptr || aligned16(p3));
}

template <typename T, int KIND>
int act_fwd_typed(const void *x, const float *bias, void *y, void *cache, int64_t rows,
                  int64_t cols, cudaStream_t st) {
  constexpr int E = Store<T>::kPerVec;
  const int64_t n = rows * cols;
  if (vector_ok<T>(bias == nullptr, cols, n, x, y, bias, cache)) {
    int64_t vr = rows, vc = cols;
    if (bias == nullptr) {  // flat: any row width works, take a wide one
      vc = kFlatCols;
      vr = ceil_div<int64_t>(n, vc);
    }
    const Tiling t = make_tiling(vr, vc / E, 64);
    if (n + vc * 4 * kBlock < INT32_MAX)
      launch_pdl(act_fwd_kernel<T, KIND, int>, t.grid, t.block, 0, st, static_cast<const T *>(x), bias,
                 static_cast<T *>(y), cache, vr, vc, n, t.rows_per_cta);
    else
      launch_pdl(act_fwd_kernel<T, KIND, int64_t>, t.grid, t.block, 0, st, static_cast<const T *>(x), bias,
                 static_cast<T *>(y), cache, vr, vc, n, t.rows_per_cta);
    DLB_LAUNCH_CHECK("act_fwd");
    return DLB_OK;
  }
  const int64_t threads = ceil_div<int64_t>(n, 8);
  launch_pdl(act_fwd_scalar_kernel<T, KIND>, static_cast<unsigned>(ceil_div<int64_t>(threads, kBlock)), kBlock, 0, st, 
      static_cast<const T *>(x), bias, static_cast<T *>(y), cache, cols, n);
  DLB_LAUNCH_CHECK("act_fwd_scalar");
  return DLB_OK;
}

template <typename T, int KIND>
int act_bwd_typed(const void *dy, const void *cache, void *dx, float *dbias, float *partial,
                  int64_t rows, int64_t cols, cudaStream_t st) {
  constexpr int E = Store<T>::kPerVec;
  const int64_t n = rows * cols;
  if (vector_ok<T>(dbias == nullptr, cols, n, dy, dy, dx, cache)) {
    int64_t vr = rows, vc = cols;
    if (dbias == nullptr) {
      vc = kFlatCols;
      vr = ceil_div<int64_t>(n, vc);
    }
    // A CTA row of the grid costs one partial row of column sums (written, then read by the second
    // stage): with few data rows keep those to a few percent of the payload (one per 64 data rows).
    int64_t gy_cap = 0;
    if (dbias != nullptr) {
      gy_cap = vr / 64 > 32 ? vr / 64 : 32;
      const int want = get_option("act_bwd_partial_rows");
      if (want > 0) gy_cap = want;
    }
    const Tiling t = make_tiling(vr, vc / E, 64, dbias != nullptr ? 64 : kBlock, gy_cap);
    if (n + vc * 4 * kBlock < INT32_MAX)
      launch_pdl(act_bwd_kernel<T, KIND, int>, t.grid, t.block, 0, st, 
        static_cast<const T *>(dy), cache, static_cast<T *>(dx), dbias ? partial : nullptr, vr, vc,
        n, t.rows_per_cta);
    else
      launch_pdl(act_bwd_kernel<T, KIND, int64_t>, t.grid, t.block, 0, st, 
        static_cast<const T *>(dy), cache, static_cast<T *>(dx), dbias ? partial : nullptr, vr, vc,
        n, t.rows_per_cta);
    DLB_LAUNCH_CHECK("act_bwd");
    if (dbias != nullptr)
      return colsum_finalize(partial, static_cast<int>(t.grid.y), static_cast<int>(cols), dbias,
                             static_cast<int>(cols), nullptr, st);
    return DLB_OK;
  }
  if constexpr (KIND != kActNone) {
    const int64_t threads = ceil_div<int64_t>(n, 8);
    launch_pdl(act_bwd_scalar_kernel<T, KIND>, static_cast<unsigned>(ceil_div<int64_t>(threads, kBlock)), kBlock, 0, st, 
        static_cast<const T *>(dy), cache, static_cast<T *>(dx), n);
    DLB_LAUNCH_CHECK("act_bwd_scalar");
  }
  if (dbias != nullptr) {
    const void *src = (KIND == kActNone) ? dy : dx;
    const int64_t chunks = ceil_div<int64_t>(rows, kScalarRowsPerChunk);
    dim3 grid(static_cast<unsigned>(ceil_div<int64_t>(cols, kBlock)), static_cast<unsigned>(chunks));
    launch_pdl(colsum_scalar_kernel<T>, grid, kBlock, 0, st, static_cast<const T *>(src), partial, rows,
                                                     cols, kScalarRowsPerChunk);
    DLB_LAUNCH_CHECK("colsum_scalar");
    return colsum_finalize(partial, static_cast<int>(chunks), static_cast<int>(cols), dbias,
                           static_cast<int>(cols), nullptr, st);
  }
  return DLB_OK;
}

template <typename T>
int act_fwd_kind(int kind, const void *x, const float *bias, void *y, void *cache, int64_t rows,
                 int64_t cols, cudaStream_t st) {
  switch (kind) {
    case DLB_ACT_RELU: return act_fwd_typed<T, DLB_ACT_RELU>(x, bias, y, cache, rows, cols, st);
    case DLB_ACT_SIGMOID: return act_fwd_typed<T, DLB_ACT_SIGMOID>(x, bias, y, cache, rows, cols, st);
    case DLB_ACT_TANH: return act_fwd_typed<T, DLB_ACT_TANH>(x, bias, y, cache, rows, cols, st);
    case DLB_ACT_GELU: return act_fwd_typed<T, DLB_ACT_GELU>(x, bias, y, cache, rows, cols, st);
  }
  set_error("act_fwd: unknown activation %d", kind);
  return DLB_ERR_INVALID_ARG;
}

template <typename T>
int act_bwd_kind(int kind, const void *dy, const void *cache, void *dx, float *dbias,
                 float *partial, int64_t rows, int64_t cols, cudaStream_t st) {
  switch (kind) {
    case DLB_ACT_RELU: return act_bwd_typed<T, DLB_ACT_RELU>(dy, cache, dx, dbias, partial, rows, cols, st);
    case DLB_ACT_SIGMOID: return act_bwd_typed<T, DLB_ACT_SIGMOID>(dy, cache, dx, dbias, partial, rows, cols, st);
    case DLB_ACT_TANH: return act_bwd_typed<T, DLB_ACT_TANH>(dy, cache, dx, dbias, partial, rows, cols, st);
    case DLB_ACT_GELU: return act_bwd_typed<T, DLB_ACT_GELU>(dy, cache, dx, dbias, partial, rows, cols, st);
    case kActNone: return act_bwd_typed<T, kActNone>(dy, cache, dx, dbias, partial, rows, cols, st);
  }
  set_error("act_bwd: unknown activation %d", kind);
  return DLB_ERR_INVALID_ARG;
}

bool shape_ok(int64_t rows, int64_t cols) {
  return rows >= 0 && cols > 0 && rows <= (INT64_MAX / 8) / cols && cols <= INT32_MAX;
}

}  // namespace
}  // namespace dlb

using namespace dlb;

extern "C" size_t dlb_act_cache_bytes(int kind, int64_t n, int dtype) {
  if (n <= 0) return 0;
  if (kind == DLB_ACT_RELU) return static_cast<size_t>((n + 7) / 8);
  return static_cast<size_t>(n) * (dtype == DLB_BF16 ? 2 : 4);
}

extern "C" int dlb_act_fwd(int kind, const void *x, const float *bias, void *y, void *cache,
                           int64_t rows, int64_t cols, int dtype, void *stream) {
  DLB_REQUIRE(shape_ok(rows, cols), DLB_ERR_INVALID_ARG, "act_fwd: rows=%lld cols=%lld",
              static_cast<long long>(rows), static_cast<long long>(cols));
  if (rows == 0) return DLB_OK;
  DLB_REQUIRE(x && y, DLB_ERR_INVALID_ARG, "act_fwd: null pointer");
  if (dtype == DLB_F32) return act_fwd_kind<float>(kind, x, bias, y, cache, rows, cols, as_stream(stream));
  if (dtype == DLB_BF16)
    return act_fwd_kind<__nv_bfloat16>(kind, x, bias, y, cache, rows, cols, as_stream(stream));
  set_error("act_fwd: unknown dtype %d", dtype);
  return DLB_ERR_INVALID_ARG;
}

extern "C" size_t dlb_act_bwd_workspace_bytes(int kind, int64_t rows, int64_t cols) {
  (void)kind;
  if (rows <= 0 || cols <= 0) return 0;
  return static_cast<size_t>(partial_rows_bound(rows)) * static_cast<size_t>(cols) * sizeof(float);
}

extern "C" int dlb_act_bwd(int kind, const void *dy, const void *cache, void *dx, float *dbias,
                           void *workspace, size_t workspace_bytes, int64_t rows, int64_t cols,
                           int dtype, void *stream) {
  DLB_REQUIRE(shape_ok(rows, cols), DLB_ERR_INVALID_ARG, "act_bwd: rows=%lld cols=%lld",
              static_cast<long long>(rows), static_cast<long long>(cols));
  DLB_REQUIRE(kind >= DLB_ACT_RELU && kind <= DLB_ACT_GELU, DLB_ERR_INVALID_ARG,
              "act_bwd: unknown activation %d", kind);
  if (rows == 0) {
    if (dbias != nullptr) {
      cudaError_t e = cudaMemsetAsync(dbias, 0, sizeof(float) * cols, as_stream(stream));
      DLB_REQUIRE(e == cudaSuccess, DLB_ERR_CUDA, "act_bwd: memset: %s", cudaGetErrorString(e));
    }
    return DLB_OK;
  }
  DLB_REQUIRE(dy && cache && dx, DLB_ERR_INVALID_ARG, "act_bwd: null pointer");
  if (dbias != nullptr)
    DLB_REQUIRE(workspace && aligned16(workspace) &&
                    workspace_bytes >= dlb_act_bwd_workspace_bytes(kind, rows, cols),
                DLB_ERR_WORKSPACE, "act_bwd: dbias needs a 16-byte aligned workspace of %zu bytes",
                dlb_act_bwd_workspace_bytes(kind, rows, cols));
  float *partial = static_cast<float *>(workspace);
  if (dtype == DLB_F32)
    return act_bwd_kind<float>(kind, dy, cache, dx, dbias, partial, rows, cols, as_stream(stream));
  if (dtype == DLB_BF16)
    return act_bwd_kind<__nv_bfloat16>(kind, dy, cache, dx, dbias, partial, rows, cols,
                                       as_stream(stream));
  set_error("act_bwd: unknown dtype %d", dtype);
  return DLB_ERR_INVALID_ARG;
}

extern "C" size_t dlb_bias_grad_workspace_bytes(int64_t rows, int64_t cols) {
  return dlb_act_bwd_workspace_bytes(kActNone, rows, cols);
}

extern "C" int dlb_bias_grad(const void *dy, float *dbias, void *workspace, size_t workspace_bytes,
                             int64_t rows, int64_t cols, int dtype, void *stream) {
  DLB_REQUIRE(shape_ok(rows, cols) && dbias, DLB_ERR_INVALID_ARG, "bias_grad: bad arguments");
  if (rows == 0) {
    cudaError_t e = cudaMemsetAsync(dbias, 0, sizeof(float) * cols, as_stream(stream));
    DLB_REQUIRE(e == cudaSuccess, DLB_ERR_CUDA, "bias_grad: memset: %s", cudaGetErrorString(e));
    return DLB_OK;
  }
  DLB_REQUIRE(dy, DLB_ERR_INVALID_ARG, "bias_grad: null pointer");
  DLB_REQUIRE(workspace && aligned16(workspace) &&
                  workspace_bytes >= dlb_bias_grad_workspace_bytes(rows, cols),
              DLB_ERR_WORKSPACE, "bias_grad: 16-byte aligned workspace of %zu bytes required",
              dlb_bias_grad_workspace_bytes(rows, cols));
  float *partial = static_cast<float *>(workspace);
  if (dtype == DLB_F32)
    return act_bwd_kind<float>(kActNone, dy, nullptr, nullptr, dbias, partial, rows, cols,
                               as_stream(stream));
  if (dtype == DLB_BF16)
    return act_bwd_kind<__nv_bfloat16>(kActNone, dy, nullptr, nullptr, dbias, partial, rows, cols,
                                       as_stream(stream));
  set_error("bias_grad: unknown dtype %d", dtype);
  return DLB_ERR_INVALID_ARG;
}
