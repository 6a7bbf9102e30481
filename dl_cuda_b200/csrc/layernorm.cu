// Layer norm with the transformer's residual add folded in, forward and
// backward, for sm_100a.  Bandwidth-bound: every activation byte crosses HBM
// once.  A row is owned by TPR threads (a sub-warp, a warp or several warps)
// that hold it in registers, so mean and variance are the same two-pass sums
// the reference kernel computes (src/transformer.cuh:145-156 in dl-cuda) at the
// cost of a single read.  Backward produces dx and the per-CTA column partials
// of dgamma/dbeta in the same pass; a second small kernel adds the partials in
// a fixed order.
#include "common.cuh"
#include "ln_bwd_pipe.cuh"
#include "reduce.cuh"

namespace dlb {
namespace {

constexpr int kBlock = 256;

// Sum over the TPR threads that own one row.  TPR <= 32: xor-shuffles inside
// the sub-warp.  TPR > 32: warp shuffles, then one shared-memory exchange
// between the row's warps (scratch holds kBlock/32 floats per value).
template <int TPR, int N>
__device__ __forceinline__ void row_sum(float (&v)[N], float *scratch, int slot) {
  constexpr int kLanes = TPR < 32 ? TPR : 32;
#pragma unroll
  for (int i = 0; i < N; i++) {
#pragma unroll
    for (int o = kLanes / 2; o > 0; o >>= 1) v[i] += __shfl_xor_sync(0xffffffffu, v[i], o);
  }
  if constexpr (TPR > 32) {
    constexpr int kWarpsPerRow = TPR / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();  // scratch may still be read from the previous use
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < N; i++) scratch[i * (kBlock / 32) + warp] = v[i];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < N; i++) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < kWarpsPerRow; w++) t += scratch[i * (kBlock / 32) + slot * kWarpsPerRow + w];
      v[i] = t;
    }
  }
}

// ------------------------------------------------------------------ forward
template <typename T, int TPR, int VPT>
__global__ void __launch_bounds__(kBlock)
ln_fwd_kernel(const T *a, const T *b, const float *gamma,
              const float *beta, T *y, T *xhat, float *__restrict__ inv_std,
              int rows, int d, float eps) {
  pdl_prologue();
  using S = Store<T>;
  constexpr int E = S::kPerVec;
  constexpr int kRowsPerCta = kBlock / TPR;
  __shared__ float scratch[(kBlock / 32)];

  const int slot = threadIdx.x / TPR;
  const int tir = threadIdx.x % TPR;
  const int row = blockIdx.x * kRowsPerCta + slot;
  const int nvec = d / E;
  const bool live = row < rows;
  const size_t base = static_cast<size_t>(row) * d;

  float s[VPT][E];
#pragma unroll
  for (int j = 0; j < VPT; j++) {
    const int vi = j * TPR + tir;
    if (live && vi < nvec) {
      uint4 va = ld_stream(a + base + static_cast<size_t>(vi) * E);
      S::unpack(va, s[j]);
    } else {
#pragma unroll
      for (int e = 0; e < E; e++) s[j][e] = 0.f;
    }
  }
  if (b != nullptr) {
#pragma unroll
    for (int j = 0; j < VPT; j++) {
      const int vi = j * TPR + tir;
      if (live && vi < nvec) {
        float t[E];
        uint4 vb = ld_stream(b + base + static_cast<size_t>(vi) * E);
        S::unpack(vb, t);
#pragma unroll
        for (int e = 0; e < E; e++) s[j][e] += t[e];
      }
    }
  }

  float acc[1] = {0.f};
#pragma unroll
  for (int j = 0; j < VPT; j++)
#pragma unroll
    for (int e = 0; e < E; e++) acc[0] += s[j][e];
  row_sum<TPR>(acc, scratch, slot);
  const float mean = acc[0] / d;

  acc[0] = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; j++) {
    const int vi = j * TPR + tir;
    if (vi < nvec) {
#pragma unroll
      for (int e = 0; e < E; e++) {
        const float diff = s[j][e] - mean;
        acc[0] += diff * diff;
      }
    }
  }
  row_sum<TPR>(acc, scratch, slot);
  const float var = acc[0] / d;
  const float is = 1.0f / sqrtf(var + eps);
  if (live && tir == 0 && inv_std != nullptr) inv_std[row] = is;

#pragma unroll
  for (int j = 0; j < VPT; j++) {
    const int vi = j * TPR + tir;
    if (live && vi < nvec) {
      const size_t off = base + static_cast<size_t>(vi) * E;
      float g[E], bt[E], xh[E], out[E];
#pragma unroll
      for (int q = 0; q < E / 4; q++) {
        const float4 g4 = ld_keep_f4(gamma + vi * E + 4 * q);
        const float4 b4 = ld_keep_f4(beta + vi * E + 4 * q);
        g[4 * q] = g4.x; g[4 * q + 1] = g4.y; g[4 * q + 2] = g4.z; g[4 * q + 3] = g4.w;
        bt[4 * q] = b4.x; bt[4 * q + 1] = b4.y; bt[4 * q + 2] = b4.z; bt[4 * q + 3] = b4.w;
      }
#pragma unroll
      for (int e = 0; e < E; e++) {
        xh[e] = (s[j][e] - mean) * is;
        out[e] = g[e] * xh[e] + bt[e];
      }
      if (xhat != nullptr) st_stream(xhat + off, S::pack(xh));
      st_stream(y + off, S::pack(out));
    }
  }
}

// Any d, any alignment: one CTA per row, scalar accesses, the row is read
// three times (the second and third reads come from L1/L2).
template <typename T>
__global__ void __launch_bounds__(kBlock)
ln_fwd_generic_kernel(const T *a, const T *b,
                      const float *gamma, const float *beta,
                      T *y, T *xhat, float *__restrict__ inv_std, int rows, int d,
                      float eps) {
  pdl_prologue();
  using S = Store<T>;
  __shared__ float red[kBlock / 32];
  const size_t base = static_cast<size_t>(blockIdx.x) * d;
  auto load = [&](int i) {
    float v = S::to_float(a[base + i]);
    if (b != nullptr) v += S::to_float(b[base + i]);
    return v;
  };
  float part = 0.f;
  for (int i = threadIdx.x; i < d; i += kBlock) part += load(i);
  const float mean = block_sum<kBlock>(part, red) / d;
  part = 0.f;
  for (int i = threadIdx.x; i < d; i += kBlock) {
    const float diff = load(i) - mean;
    part += diff * diff;
  }
  const float var = block_sum<kBlock>(part, red) / d;
  const float is = 1.0f / sqrtf(var + eps);
  if (threadIdx.x == 0 && inv_std != nullptr) inv_std[blockIdx.x] = is;
  for (int i = threadIdx.x; i < d; i += kBlock) {
    const float xh = (load(i) - mean) * is;
    // y may alias a or b: every element is read and written by one thread only.
    const float out = gamma[i] * xh + beta[i];
    if (xhat != nullptr) xhat[base + i] = S::from_float(xh);
    y[base + i] = S::from_float(out);
  }
}

// ----------------------------------------------------------------- backward
// Persistent CTAs: slot s of CTA c walks rows c*RPC+s, +grid*RPC, ... and keeps
// the dgamma/dbeta sums of its columns in registers.  At the end the CTA adds
// its slots in slot order and writes one partial row [2*d] (dgamma | dbeta).
template <typename T, int TPR, int VPT>
__global__ void __launch_bounds__(kBlock)
ln_bwd_kernel(const T *dy_a, const T *dy_b, const T *xhat,
              const float *inv_std, const float *gamma, T *dx,
              float *__restrict__ partial, int rows, int d) {
  pdl_prologue();
  using S = Store<T>;
  constexpr int E = S::kPerVec;
  constexpr int kRowsPerCta = kBlock / TPR;
  constexpr int kCols = TPR * VPT * E;  // padded row width covered by a slot
  __shared__ float scratch[2 * (kBlock / 32)];
  extern __shared__ float slot_acc[];  // [kRowsPerCta][kCols]

  const int slot = threadIdx.x / TPR;
  const int tir = threadIdx.x % TPR;
  const int nvec = d / E;

  float accg[VPT][E], accb[VPT][E];
#pragma unroll
  for (int j = 0; j < VPT; j++)
#pragma unroll
    for (int e = 0; e < E; e++) accg[j][e] = accb[j][e] = 0.f;

  // The loop bound is CTA-uniform so that the barriers inside row_sum match.
  for (int row0 = blockIdx.x * kRowsPerCta; row0 < rows; row0 += gridDim.x * kRowsPerCta) {
    const int row = row0 + slot;
    const bool live = row < rows;
    const size_t base = static_cast<size_t>(row) * d;
    float dyv[VPT][E], xh[VPT][E];
#pragma unroll
    for (int j = 0; j < VPT; j++) {
      const int vi = j * TPR + tir;
      if (live && vi < nvec) {
        const size_t off = base + static_cast<size_t>(vi) * E;
        S::unpack(ld_stream(dy_a + off), dyv[j]);
        S::unpack(ld_stream(xhat + off), xh[j]);
      } else {
#pragma unroll
        for (int e = 0; e < E; e++) dyv[j][e] = xh[j][e] = 0.f;
      }
    }
    if (dy_b != nullptr) {
#pragma unroll
      for (int j = 0; j < VPT; j++) {
        const int vi = j * TPR + tir;
        if (live && vi < nvec) {
          float t[E];
          S::unpack(ld_stream(dy_b + base + static_cast<size_t>(vi) * E), t);
#pragma unroll
          for (int e = 0; e < E; e++) dyv[j][e] += t[e];
        }
      }
    }
    const float is = live ? ld_co(inv_std + row) : 0.f;

    float c[2] = {0.f, 0.f};
    float gdy[VPT][E];
#pragma unroll
    for (int j = 0; j < VPT; j++) {
      const int vi = j * TPR + tir;
      float g[E];
      if (vi < nvec) {
#pragma unroll
        for (int q = 0; q < E / 4; q++) {
          const float4 g4 = ld_keep_f4(gamma + vi * E + 4 * q);
          g[4 * q] = g4.x; g[4 * q + 1] = g4.y; g[4 * q + 2] = g4.z; g[4 * q + 3] = g4.w;
        }
      } else {
#pragma unroll
        for (int e = 0; e < E; e++) g[e] = 0.f;
      }
#pragma unroll
      for (int e = 0; e < E; e++) {
        const float dxh = dyv[j][e] * g[e];
        gdy[j][e] = dxh;
        c[0] += dxh;
        c[1] += dxh * xh[j][e];
        accg[j][e] += dyv[j][e] * xh[j][e];
        accb[j][e] += dyv[j][e];
      }
    }
    row_sum<TPR>(c, scratch, slot);
    const float c1 = c[0] / d;
    const float c2 = c[1] / d;
#pragma unroll
    for (int j = 0; j < VPT; j++) {
      const int vi = j * TPR + tir;
      if (live && vi < nvec) {
        float o[E];
#pragma unroll
        for (int e = 0; e < E; e++) o[e] = (gdy[j][e] - c1 - xh[j][e] * c2) * is;
        st_stream(dx + base + static_cast<size_t>(vi) * E, S::pack(o));
      }
    }
  }

  // Slot-order reduction of the column sums, dgamma first, then dbeta.
#pragma unroll
  for (int which = 0; which < 2; which++) {
    __syncthreads();
#pragma unroll
    for (int j = 0; j < VPT; j++) {
      const int vi = j * TPR + tir;
#pragma unroll
      for (int e = 0; e < E; e++)
        slot_acc[slot * kCols + vi * E + e] = which == 0 ? accg[j][e] : accb[j][e];
    }
    __syncthreads();
    for (int col = threadIdx.x; col < d; col += kBlock) {
      float t = 0.f;
#pragma unroll
      for (int s2 = 0; s2 < kRowsPerCta; s2++) t += slot_acc[s2 * kCols + col];
      partial[(static_cast<size_t>(blockIdx.x) * 2 + which) * d + col] = t;
    }
  }
}

// Any d: one CTA per row computes dx; dgamma/dbeta come from ln_colsum_generic.
template <typename T>
__global__ void __launch_bounds__(kBlock)
ln_bwd_dx_generic_kernel(const T *dy_a, const T *dy_b, const T *xhat,
                         const float *inv_std,
                         const float *gamma, T *dx, int rows, int d) {
  pdl_prologue();
  using S = Store<T>;
  __shared__ float red[kBlock / 32];
  const size_t base = static_cast<size_t>(blockIdx.x) * d;
  auto load_dy = [&](int i) {
    float v = S::to_float(dy_a[base + i]);
    if (dy_b != nullptr) v += S::to_float(dy_b[base + i]);
    return v;
  };
  float p1 = 0.f, p2 = 0.f;
  for (int i = threadIdx.x; i < d; i += kBlock) {
    const float dxh = load_dy(i) * gamma[i];
    p1 += dxh;
    p2 += dxh * S::to_float(xhat[base + i]);
  }
  const float c1 = block_sum<kBlock>(p1, red) / d;
  const float c2 = block_sum<kBlock>(p2, red) / d;
  const float is = inv_std[blockIdx.x];
  for (int i = threadIdx.x; i < d; i += kBlock) {
    const float dxh = load_dy(i) * gamma[i];
    dx[base + i] = S::from_float((dxh - c1 - S::to_float(xhat[base + i]) * c2) * is);
  }
}

// Generic dgamma/dbeta partials: CTA (x = column block of kBlock, y = row
// chunk) sums its rows top to bottom.  Must run BEFORE the dx kernel when dx
// aliases dy_a.
template <typename T>
__global__ void __launch_bounds__(kBlock)
ln_colsum_generic_kernel(const T *dy_a, const T *dy_b,
                         const T *xhat, float *__restrict__ partial,
                         int rows, int d, int rows_per_chunk) {
  pdl_prologue();
  using S = Store<T>;
  const int col = blockIdx.x * kBlock + threadIdx.x;
  if (col >= d) return;
  const int r0 = blockIdx.y * rows_per_chunk;
  const int r1 = min(rows, r0 + rows_per_chunk);
  float dg = 0.f, db = 0.f;
  for (int r = r0; r < r1; r++) {
    const size_t off = static_cast<size_t>(r) * d + col;
    float v = S::to_float(dy_a[off]);
    if (dy_b != nullptr) v += S::to_float(dy_b[off]);
    dg += v * S::to_float(xhat[off]);
    db += v;
  }
  partial[(static_cast<size_t>(blockIdx.y) * 2) * d + col] = dg;
  partial[(static_cast<size_t>(blockIdx.y) * 2 + 1) * d + col] = db;
}

// --------------------------------------------------------------- dispatch
struct Shape {
  int tpr = 0, vpt = 0;  // 0 => generic path
};

// Smallest thread group that covers the row with at most 32 fp32 values held
// per thread; rows wider than 256 threads x 32 values take the generic path.
template <typename T>
Shape pick_shape(int d, bool all_aligned) {
  constexpr int E = Store<T>::kPerVec;
  constexpr int kMaxVpt = 32 / E;
  Shape s;
  if (!all_aligned || d % E != 0) return s;
  const int nvec = d / E;
  for (int tpr = 8; tpr <= kBlock; tpr *= 2) {
    const int need = ceil_div(nvec, tpr);
    if (need <= kMaxVpt) {
      int vpt = 1;
      while (vpt < need) vpt *= 2;
      // Only TPR=8 is built with every VPT; wider groups are built with the
      // largest VPT (the row did not fit the next smaller group, so need is
      // more than half of it).
      if (tpr > 8) vpt = kMaxVpt;
      s.tpr = tpr;
      s.vpt = vpt;
      return s;
    }
  }
  return s;
}

constexpr int kMaxPartialRows = 1024;  // upper bound on CTAs of the backward grid

int bwd_grid(int rows, int rows_per_cta, int ctas_per_sm) {
  const int want = ceil_div(rows, rows_per_cta);
  const int cap = min(kMaxPartialRows, sm_count() * ctas_per_sm);
  return want < cap ? want : cap;
}

template <typename T, int TPR, int VPT>
int launch_fwd(const void *a, const void *b, const float *gamma, const float *beta, void *y,
               void *xhat, float *inv_std, int rows, int d, float eps, cudaStream_t st) {
  const int grid = ceil_div(rows, kBlock / TPR);
  launch_pdl(ln_fwd_kernel<T, TPR, VPT>, grid, kBlock, 0, st, 
      static_cast<const T *>(a), static_cast<const T *>(b), gamma, beta, static_cast<T *>(y),
      static_cast<T *>(xhat), inv_std, rows, d, eps);
  DLB_LAUNCH_CHECK("ln_fwd");
  return DLB_OK;
}

template <typename T, int TPR, int VPT>
int launch_bwd(const void *dy_a, const void *dy_b, const void *xhat, const float *inv_std,
               const float *gamma, void *dx, float *partial, int *n_partial, int rows, int d,
               cudaStream_t st) {
  constexpr int E = Store<T>::kPerVec;
  constexpr int kRowsPerCta = kBlock / TPR;
  constexpr size_t kSmem = sizeof(float) * kRowsPerCta * TPR * VPT * E;
  static_assert(kSmem <= 48 * 1024, "slot accumulators must fit default dynamic smem");
  auto kern = ln_bwd_kernel<T, TPR, VPT>;
  // One occupancy query per instantiation; racing first calls compute the same value.
  static std::atomic<int> cached_ctas_per_sm{0};
  int ctas_per_sm = cached_ctas_per_sm.load(std::memory_order_relaxed);
  if (ctas_per_sm == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, kBlock, kSmem) != cudaSuccess || n < 1)
      n = 1;
    ctas_per_sm = n;
    cached_ctas_per_sm.store(n, std::memory_order_relaxed);
  }
  const int grid = bwd_grid(rows, kRowsPerCta, ctas_per_sm);
  launch_pdl(kern, grid, kBlock, kSmem, st, static_cast<const T *>(dy_a), static_cast<const T *>(dy_b),
                                    static_cast<const T *>(xhat), inv_std, gamma,
                                    static_cast<T *>(dx), partial, rows, d);
  DLB_LAUNCH_CHECK("ln_bwd");
  *n_partial = grid;
  return DLB_OK;
}

#define DLB_LN_CASES_F32(M)                                                   \
  M(8, 1) M(8, 2) M(8, 4) M(8, 8) M(16, 8) M(32, 8) M(64, 8) M(128, 8) M(256, 8)
#define DLB_LN_CASES_BF16(M) \
  M(8, 1) M(8, 2) M(8, 4) M(16, 4) M(32, 4) M(64, 4) M(128, 4) M(256, 4)

template <typename T>
int ln_fwd_typed(const void *a, const void *b, const float *gamma, const float *beta, void *y,
                 void *xhat, float *inv_std, int rows, int d, float eps, cudaStream_t st) {
  const bool al = aligned16(a) && (b == nullptr || aligned16(b)) && aligned16(y) &&
                  (xhat == nullptr || aligned16(xhat)) && aligned16(gamma) && aligned16(beta);
  const Shape s = pick_shape<T>(d, al);
#define M(TPR, VPT)                     \
  if (s.tpr == TPR && s.vpt == VPT)     \
    return launch_fwd<T, TPR, VPT>(a, b, gamma, beta, y, xhat, inv_std, rows, d, eps, st);
  if constexpr (sizeof(T) == 4) {
    DLB_LN_CASES_F32(M)
  } else {
    DLB_LN_CASES_BF16(M)
  }
#undef M
  launch_pdl(ln_fwd_generic_kernel<T>, rows, kBlock, 0, st, 
      static_cast<const T *>(a), static_cast<const T *>(b), gamma, beta, static_cast<T *>(y),
      static_cast<T *>(xhat), inv_std, rows, d, eps);
  DLB_LAUNCH_CHECK("ln_fwd_generic");
  return DLB_OK;
}

constexpr int kGenericRowsPerChunk = 256;

template <typename T>
int ln_bwd_typed(const void *dy_a, const void *dy_b, const void *xhat, const float *inv_std,
                 const float *gamma, void *dx, float *dgamma, float *dbeta, float *partial,
                 int rows, int d, cudaStream_t st) {
  const bool al = aligned16(dy_a) && (dy_b == nullptr || aligned16(dy_b)) && aligned16(xhat) &&
                  aligned16(dx) && aligned16(gamma);
  int n_partial = 0;
  int rc = -1;
  // Wide rows and enough of them: the bulk-copy pipeline; otherwise rows in registers.
  const PipeShape ps = pick_pipe_shape<T>(rows, d, dy_b != nullptr, al && aligned16(partial));
#define M(CT, KV, RT)                                  \
  if (ps.ct == CT && ps.kv == KV && ps.rt == RT)       \
    rc = launch_ln_bwd_pipe<T, CT, KV, RT>(ps, dy_a, dy_b, xhat, inv_std, gamma, dx, partial, &n_partial, rows, d, st);
  DLB_PIPE_CASES(M)
#undef M
  const Shape s = rc == -1 ? pick_shape<T>(d, al) : Shape{};
#define M(TPR, VPT)                 \
  if (rc == -1 && s.tpr == TPR && s.vpt == VPT) \
    rc = launch_bwd<T, TPR, VPT>(dy_a, dy_b, xhat, inv_std, gamma, dx, partial, &n_partial, rows, d, st);
  if constexpr (sizeof(T) == 4) {
    DLB_LN_CASES_F32(M)
  } else {
    DLB_LN_CASES_BF16(M)
  }
#undef M
  if (rc == -1) {
    n_partial = ceil_div(rows, kGenericRowsPerChunk);
    dim3 grid(ceil_div(d, kBlock), n_partial);
    launch_pdl(ln_colsum_generic_kernel<T>, grid, kBlock, 0, st, 
        static_cast<const T *>(dy_a), static_cast<const T *>(dy_b), static_cast<const T *>(xhat),
        partial, rows, d, kGenericRowsPerChunk);
    DLB_LAUNCH_CHECK("ln_colsum_generic");
    launch_pdl(ln_bwd_dx_generic_kernel<T>, rows, kBlock, 0, st, 
        static_cast<const T *>(dy_a), static_cast<const T *>(dy_b), static_cast<const T *>(xhat),
        inv_std, gamma, static_cast<T *>(dx), rows, d);
    DLB_LAUNCH_CHECK("ln_bwd_dx_generic");
    rc = DLB_OK;
  }
  if (rc != DLB_OK) return rc;
  // partial is [n_partial][2*d]: columns 0..d-1 -> dgamma, d..2d-1 -> dbeta.
  return colsum_finalize(partial, n_partial, 2 * d, dgamma, d, dbeta, st);
}

size_t partial_rows_bound(int rows) {
  const int generic = ceil_div(rows, kGenericRowsPerChunk);
  return static_cast<size_t>(generic > kMaxPartialRows ? generic : kMaxPartialRows);
}

}  // namespace
}  // namespace dlb

using namespace dlb;

extern "C" int dlb_ln_residual_fwd(const void *a, const void *b, const float *gamma,
                                   const float *beta, void *y, void *xhat, float *inv_std,
                                   int rows, int d, float eps, int dtype, void *stream) {
  DLB_REQUIRE(rows >= 0 && d > 0, DLB_ERR_INVALID_ARG, "ln_residual_fwd: rows=%d d=%d", rows, d);
  if (rows == 0) return DLB_OK;
  DLB_REQUIRE(a && gamma && beta && y, DLB_ERR_INVALID_ARG, "ln_residual_fwd: null pointer");
  DLB_REQUIRE((xhat == nullptr) == (inv_std == nullptr), DLB_ERR_INVALID_ARG,
              "ln_residual_fwd: xhat and inv_std must both be given or both be NULL");
  if (dtype == DLB_F32)
    return ln_fwd_typed<float>(a, b, gamma, beta, y, xhat, inv_std, rows, d, eps, as_stream(stream));
  if (dtype == DLB_BF16)
    return ln_fwd_typed<__nv_bfloat16>(a, b, gamma, beta, y, xhat, inv_std, rows, d, eps,
                                       as_stream(stream));
  set_error("ln_residual_fwd: unknown dtype %d", dtype);
  return DLB_ERR_INVALID_ARG;
}

extern "C" size_t dlb_ln_bwd_workspace_bytes(int rows, int d) {
  if (rows <= 0 || d <= 0) return 0;
  return partial_rows_bound(rows) * 2 * static_cast<size_t>(d) * sizeof(float);
}

extern "C" int dlb_ln_bwd(const void *dy_a, const void *dy_b, const void *xhat,
                          const float *inv_std, const float *gamma, void *dx, float *dgamma,
                          float *dbeta, void *workspace, size_t workspace_bytes, int rows, int d,
                          int dtype, void *stream) {
  DLB_REQUIRE(rows >= 0 && d > 0, DLB_ERR_INVALID_ARG, "ln_bwd: rows=%d d=%d", rows, d);
  DLB_REQUIRE(dgamma && dbeta, DLB_ERR_INVALID_ARG, "ln_bwd: null dgamma/dbeta");
  if (rows == 0) {
    cudaError_t e = cudaMemsetAsync(dgamma, 0, sizeof(float) * d, as_stream(stream));
    if (e == cudaSuccess) e = cudaMemsetAsync(dbeta, 0, sizeof(float) * d, as_stream(stream));
    DLB_REQUIRE(e == cudaSuccess, DLB_ERR_CUDA, "ln_bwd: memset: %s", cudaGetErrorString(e));
    return DLB_OK;
  }
  DLB_REQUIRE(dy_a && xhat && inv_std && gamma && dx, DLB_ERR_INVALID_ARG, "ln_bwd: null pointer");
  DLB_REQUIRE(workspace && workspace_bytes >= dlb_ln_bwd_workspace_bytes(rows, d) &&
                  aligned16(workspace),
              DLB_ERR_WORKSPACE, "ln_bwd: workspace of %zu bytes (16-byte aligned) required",
              dlb_ln_bwd_workspace_bytes(rows, d));
  float *partial = static_cast<float *>(workspace);
  if (dtype == DLB_F32)
    return ln_bwd_typed<float>(dy_a, dy_b, xhat, inv_std, gamma, dx, dgamma, dbeta, partial, rows,
                               d, as_stream(stream));
  if (dtype == DLB_BF16)
    return ln_bwd_typed<__nv_bfloat16>(dy_a, dy_b, xhat, inv_std, gamma, dx, dgamma, dbeta,
                                       partial, rows, d, as_stream(stream));
  set_error("ln_bwd: unknown dtype %d", dtype);
  return DLB_ERR_INVALID_ARG;
}

// ---------------------------------------------------------------------------
// Layer-norm backward for callers that cannot allocate device memory.
//
// Some hosts of this library are handed buffers by someone else and must not
// call cudaMalloc themselves: a plugin that runs inside another framework's
// memory pool, code on a latency-critical path where an allocation may stall or
// fail, a process whose memory budget is fixed at start-up.  dlb_ln_bwd() needs
// a workspace from its caller; this variant brings its own.  The workspace is a
// fixed array in the library's device image, so every GPU that loads the
// library holds kNoAllocScratchBytes for the life of the process.
constexpr size_t kNoAllocScratchBytes = 16u << 20;  // 16 MiB
static __device__ __align__(256) unsigned char g_ln_bwd_scratch[kNoAllocScratchBytes];

namespace {
// g_ln_bwd_scratch is a host-side stand-in for the array, not an address a
// kernel can use: the device address is asked for once per device, with that
// device current, and cached.
void *noalloc_scratch_address() {
  constexpr int kMaxDev = 64;
  static std::atomic<void *> cached[kMaxDev];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
  void *p = cached[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    if (cudaGetSymbolAddress(&p, g_ln_bwd_scratch) != cudaSuccess || p == nullptr) return nullptr;
    cached[dev].store(p, std::memory_order_release);
  }
  return p;
}
}  // namespace

extern "C" size_t dlb_ln_bwd_noalloc_max_bytes(void) { return kNoAllocScratchBytes; }

extern "C" int dlb_ln_bwd_noalloc(const void *dy_a, const void *dy_b, const void *xhat,
                                  const float *inv_std, const float *gamma, void *dx, float *dgamma,
                                  float *dbeta, int rows, int d, int dtype, void *stream) {
  DLB_REQUIRE(rows >= 0 && d > 0, DLB_ERR_INVALID_ARG, "ln_bwd_noalloc: rows=%d d=%d", rows, d);
  const size_t need = dlb_ln_bwd_workspace_bytes(rows, d);
  DLB_REQUIRE(need <= kNoAllocScratchBytes, DLB_ERR_UNSUPPORTED,
              "ln_bwd_noalloc: rows=%d d=%d needs %zu bytes of scratch, the built-in array holds %zu "
              "(use dlb_ln_bwd with a caller-provided workspace)",
              rows, d, need, kNoAllocScratchBytes);
  void *scratch = noalloc_scratch_address();
  DLB_REQUIRE(scratch != nullptr, DLB_ERR_CUDA, "ln_bwd_noalloc: cudaGetSymbolAddress failed: %s",
              cudaGetErrorString(cudaGetLastError()));
  return dlb_ln_bwd(dy_a, dy_b, xhat, inv_std, gamma, dx, dgamma, dbeta, scratch, kNoAllocScratchBytes,
                    rows, d, dtype, stream);
}
