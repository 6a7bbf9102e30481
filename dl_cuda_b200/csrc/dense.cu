// Pass-through dense ops: the fp32 matrix products, row softmax and loss kernels
// that sit between the bandwidth-bound layer kernels of this library inside
// dl-cuda's TransformerLayer, LinearLayer, SoftmaxActivation and loss helpers
// (src/transformer.cuh:8-134, src/layers.cuh:23-82, src/activation.cuh:121-165,
// src/loss.cuh:18-144).  They exist so that a model written against the
// reference's layer API runs end to end on this library; they are correctness
// implementations on the fp32 pipes (shared-memory tiled, no tensor cores) and
// are not tuned against a roofline.
//
// Every product keeps the reference's arithmetic per output element: one fused
// multiply-add per k in ascending k, starting from 0, then the scale, the bias
// and the optional add into the destination.  Only the work decomposition
// differs (64x64 tiles through shared memory, all (batch, head) pairs in one
// launch, heads addressed by stride instead of reshaped copies).
#include "common.cuh"

namespace dlb {
namespace {

constexpr int kTileM = 64, kTileN = 64, kTileK = 16, kGemmThreads = 256;

struct GemmArgs {
  const float *a, *b, *bias;
  float *c;
  int m, n, k;
  long long a_row, a_col;  // A(i,kk) = a[i*a_row + kk*a_col]
  long long b_row, b_col;  // B(kk,j) = b[kk*b_row + j*b_col]
  long long ldc;
  int batch_inner;  // batch z -> (z / batch_inner, z % batch_inner)
  long long a_outer, a_inner, b_outer, b_inner, c_outer, c_inner;
  float alpha;
  int accumulate;
};

// Loads a [tile_rows x kTileK] slab of an operand into smem[kk][row]; `row_stride`
// / `k_stride` are the element strides along the tile row and along k.
template <int ROWS>
__device__ __forceinline__ void load_slab(float (*smem)[ROWS + 4], const float *base, long long row_stride,
                                          long long k_stride, int row0, int k0, int rows, int k) {
  constexpr int kPerThread = ROWS * kTileK / kGemmThreads;
  const bool k_contiguous = (k_stride == 1);
#pragma unroll
  for (int e = 0; e < kPerThread; e++) {
    const int flat = threadIdx.x + e * kGemmThreads;
    const int r = k_contiguous ? flat / kTileK : flat % ROWS;
    const int kk = k_contiguous ? flat % kTileK : flat / ROWS;
    float v = 0.f;
    if (row0 + r < rows && k0 + kk < k) v = base[(row0 + r) * row_stride + (k0 + kk) * k_stride];
    smem[kk][r] = v;
  }
}

__global__ void __launch_bounds__(kGemmThreads) gemm_f32_kernel(const GemmArgs g) {
  pdl_prologue();
  __shared__ __align__(16) float sa[kTileK][kTileM + 4];
  __shared__ __align__(16) float sb[kTileK][kTileN + 4];

  const int zo = blockIdx.z / g.batch_inner, zi = blockIdx.z % g.batch_inner;
  const float *a = g.a + zo * g.a_outer + zi * g.a_inner;
  const float *b = g.b + zo * g.b_outer + zi * g.b_inner;
  float *c = g.c + zo * g.c_outer + zi * g.c_inner;

  const int m0 = blockIdx.y * kTileM, n0 = blockIdx.x * kTileN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < g.k; k0 += kTileK) {
    load_slab<kTileM>(sa, a, g.a_row, g.a_col, m0, k0, g.m, g.k);
    load_slab<kTileN>(sb, b, g.b_col, g.b_row, n0, k0, g.n, g.k);
    __syncthreads();
    // Columns past k hold zeros in both slabs: fma(0, 0, acc) leaves acc unchanged,
    // so the ragged last slab needs no separate loop bound.
#pragma unroll
    for (int kk = 0; kk < kTileK; kk++) {
      const float4 av = *reinterpret_cast<const float4 *>(&sa[kk][ty * 4]);
      const float4 bv = *reinterpret_cast<const float4 *>(&sb[kk][tx * 4]);
      const float ar[4] = {av.x, av.y, av.z, av.w};
      const float br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int row = m0 + ty * 4 + i;
    if (row >= g.m) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int col = n0 + tx * 4 + j;
      if (col >= g.n) continue;
      float v = acc[i][j] * g.alpha;
      if (g.bias) v = v + g.bias[col];
      float *dst = c + row * g.ldc + col;
      if (g.accumulate) v = *dst + v;
      *dst = v;
    }
  }
}

// One warp per row.  `causal_period` > 0 masks row r to its first (r % period) + 1
// entries, the rest come out as exact zeros (the reference overwrites them with
// -1e9 before the softmax, whose expf then underflows to 0).
__global__ void __launch_bounds__(256) softmax_fwd_kernel(const float *in, float *out, long long rows,
                                                          int width, int causal_period) {
  pdl_prologue();
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) / 32;
  if (row >= rows) return;
  const int lane = threadIdx.x % 32;
  const int valid = causal_period > 0 ? static_cast<int>(row % causal_period) + 1 : width;
  const float *src = in + row * width;
  float *dst = out + row * width;

  float mx = -INFINITY;
  for (int j = lane; j < valid; j += 32) mx = fmaxf(mx, src[j]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));

  float sum = 0.f;
  for (int j = lane; j < valid; j += 32) {
    const float e = expf(src[j] - mx);
    dst[j] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  const float inv = 1.0f / sum;
  for (int j = lane; j < valid; j += 32) dst[j] *= inv;
  for (int j = valid + lane; j < width; j += 32) dst[j] = 0.f;
}

// dx = (s * (dy - sum_j dy_j s_j)) * scale, one warp per row; dx may alias dy.
__global__ void __launch_bounds__(256) softmax_bwd_kernel(const float *dy, const float *s, float *dx,
                                                          long long rows, int width, float scale) {
  pdl_prologue();
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) / 32;
  if (row >= rows) return;
  const int lane = threadIdx.x % 32;
  const float *g = dy + row * width;
  const float *p = s + row * width;
  float *d = dx + row * width;
  float dot = 0.f;
  for (int j = lane; j < width; j += 32) dot = fmaf(g[j], p[j], dot);
  dot = warp_sum(dot);
  for (int j = lane; j < width; j += 32) d[j] = (p[j] * (g[j] - dot)) * scale;
}

// --- losses (src/loss.cuh) ------------------------------------------------------
constexpr float kLossEps = 1e-10f;

__device__ __forceinline__ float clamp_prob(float p) {
  if (p < kLossEps) return kLossEps;
  if (p > 1.0f - kLossEps) return 1.0f - kLossEps;
  return p;
}

__global__ void loss_fwd_kernel(int kind, const float *y, const float *yp, float *err, long long n,
                                int classes) {
  pdl_prologue();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (kind == DLB_LOSS_SQUARED) {
    const float diff = y[i] - yp[i];
    err[i] = diff * diff;
  } else if (kind == DLB_LOSS_ABSOLUTE) {
    err[i] = fabsf(y[i] - yp[i]);
  } else if (kind == DLB_LOSS_BCE) {
    const float p = clamp_prob(yp[i]);
    err[i] = -y[i] * logf(p) - (1.0f - y[i]) * logf(1.0f - p);
  } else {
    float loss = 0.f;
    for (int c = 0; c < classes; c++) loss -= y[i * classes + c] * logf(yp[i * classes + c] + kLossEps);
    err[i] = loss;
  }
}

__global__ void loss_bwd_kernel(int kind, const float *y, const float *yp, float *grad, long long n,
                                int classes) {
  pdl_prologue();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long total = kind == DLB_LOSS_CCE ? n * classes : n;
  if (i >= total) return;
  if (kind == DLB_LOSS_SQUARED) {
    grad[i] = 2.0f * (yp[i] - y[i]) / n;
  } else if (kind == DLB_LOSS_ABSOLUTE) {
    const float diff = yp[i] - y[i];
    grad[i] = ((diff > 0.0f) ? 1.0f : ((diff < 0.0f) ? -1.0f : 0.0f)) / n;
  } else if (kind == DLB_LOSS_BCE) {
    const float p = clamp_prob(yp[i]);
    grad[i] = (-y[i] / p + (1.0f - y[i]) / (1.0f - p)) / n;
  } else {
    grad[i] = -y[i] / (yp[i] + kLossEps) / n;
  }
}

__global__ void ce_ids_fwd_kernel(const int *target, const float *yp, float *err, int n, int classes,
                                  float eps) {
  pdl_prologue();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float p = yp[static_cast<long long>(i) * classes + target[i]];
  if (p < eps) p = eps;
  err[i] = -logf(p);
}

__global__ void ce_ids_bwd_kernel(const int *target, const float *yp, float *grad, int n, int classes,
                                  float eps) {
  pdl_prologue();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(n) * classes) return;
  const int row = static_cast<int>(i / classes), col = static_cast<int>(i % classes);
  float g = 0.f;
  if (col == target[row]) {
    float p = yp[i];
    if (p < eps) p = eps;
    g = -1.0f / (p * n);
  }
  grad[i] = g;
}

inline unsigned blocks_for(long long n, int block) { return static_cast<unsigned>((n + block - 1) / block); }

}  // namespace
}  // namespace dlb

using namespace dlb;

extern "C" int dlb_gemm_f32(const float *a, const float *b, const float *bias, float *c, int m, int n,
                            int k, int64_t a_row, int64_t a_col, int64_t b_row, int64_t b_col,
                            int64_t ldc, int batch, int batch_inner, int64_t a_outer, int64_t a_inner,
                            int64_t b_outer, int64_t b_inner, int64_t c_outer, int64_t c_inner,
                            float alpha, int accumulate, void *stream) {
  DLB_REQUIRE(m >= 0 && n >= 0 && k >= 0 && batch >= 0, DLB_ERR_INVALID_ARG, "gemm_f32: m=%d n=%d k=%d batch=%d",
              m, n, k, batch);
  if (m == 0 || n == 0 || batch == 0) return DLB_OK;
  DLB_REQUIRE(a && b && c, DLB_ERR_INVALID_ARG, "gemm_f32: null pointer");
  DLB_REQUIRE(batch_inner >= 1 && batch % batch_inner == 0, DLB_ERR_INVALID_ARG,
              "gemm_f32: batch=%d is not a multiple of batch_inner=%d", batch, batch_inner);
  DLB_REQUIRE(ldc >= n, DLB_ERR_INVALID_ARG, "gemm_f32: ldc=%lld < n=%d", static_cast<long long>(ldc), n);
  const int tiles_m = ceil_div(m, kTileM), tiles_n = ceil_div(n, kTileN);
  DLB_REQUIRE(tiles_m <= 65535 && batch <= 65535, DLB_ERR_UNSUPPORTED,
              "gemm_f32: m=%d or batch=%d beyond the launch grid", m, batch);
  GemmArgs g{a, b, bias, c, m, n, k, a_row, a_col, b_row, b_col, ldc, batch_inner,
             a_outer, a_inner, b_outer, b_inner, c_outer, c_inner, alpha, accumulate};
  launch_pdl(gemm_f32_kernel, dim3(tiles_n, tiles_m, batch), dim3(kGemmThreads), 0, as_stream(stream), g);
  DLB_LAUNCH_CHECK("gemm_f32");
  return DLB_OK;
}

extern "C" int dlb_softmax_fwd(const float *in, float *out, int64_t rows, int width, int causal_period,
                               void *stream) {
  DLB_REQUIRE(rows >= 0 && width > 0 && causal_period >= 0, DLB_ERR_INVALID_ARG,
              "softmax_fwd: rows=%lld width=%d causal_period=%d", static_cast<long long>(rows), width,
              causal_period);
  DLB_REQUIRE(causal_period <= width, DLB_ERR_INVALID_ARG, "softmax_fwd: causal_period=%d > width=%d",
              causal_period, width);
  if (rows == 0) return DLB_OK;
  DLB_REQUIRE(in && out, DLB_ERR_INVALID_ARG, "softmax_fwd: null pointer");
  launch_pdl(softmax_fwd_kernel, blocks_for(rows * 32, 256), 256, 0, as_stream(stream), in, out,
             static_cast<long long>(rows), width, causal_period);
  DLB_LAUNCH_CHECK("softmax_fwd");
  return DLB_OK;
}

extern "C" int dlb_softmax_bwd(const float *dy, const float *s, float *dx, int64_t rows, int width,
                               float scale, void *stream) {
  DLB_REQUIRE(rows >= 0 && width > 0, DLB_ERR_INVALID_ARG, "softmax_bwd: rows=%lld width=%d",
              static_cast<long long>(rows), width);
  if (rows == 0) return DLB_OK;
  DLB_REQUIRE(dy && s && dx, DLB_ERR_INVALID_ARG, "softmax_bwd: null pointer");
  launch_pdl(softmax_bwd_kernel, blocks_for(rows * 32, 256), 256, 0, as_stream(stream), dy, s, dx,
             static_cast<long long>(rows), width, scale);
  DLB_LAUNCH_CHECK("softmax_bwd");
  return DLB_OK;
}

static int loss_args_ok(const char *what, int kind, const float *y, const float *yp, float *out, int64_t n,
                        int classes) {
  DLB_REQUIRE(kind >= DLB_LOSS_SQUARED && kind <= DLB_LOSS_CCE, DLB_ERR_INVALID_ARG, "%s: unknown loss %d", what,
              kind);
  DLB_REQUIRE(n >= 0 && (kind != DLB_LOSS_CCE || classes > 0), DLB_ERR_INVALID_ARG, "%s: n=%lld classes=%d",
              what, static_cast<long long>(n), classes);
  DLB_REQUIRE(n == 0 || (y && yp && out), DLB_ERR_INVALID_ARG, "%s: null pointer", what);
  return DLB_OK;
}

extern "C" int dlb_loss_fwd(int kind, const float *y, const float *y_pred, float *error, int64_t n,
                            int classes, void *stream) {
  if (int st = loss_args_ok("loss_fwd", kind, y, y_pred, error, n, classes)) return st;
  if (n == 0) return DLB_OK;
  launch_pdl(loss_fwd_kernel, blocks_for(n, 256), 256, 0, as_stream(stream), kind, y, y_pred, error,
             static_cast<long long>(n), classes);
  DLB_LAUNCH_CHECK("loss_fwd");
  return DLB_OK;
}

extern "C" int dlb_loss_bwd(int kind, const float *y, const float *y_pred, float *grad, int64_t n,
                            int classes, void *stream) {
  if (int st = loss_args_ok("loss_bwd", kind, y, y_pred, grad, n, classes)) return st;
  if (n == 0) return DLB_OK;
  const long long total = kind == DLB_LOSS_CCE ? static_cast<long long>(n) * classes : n;
  launch_pdl(loss_bwd_kernel, blocks_for(total, 256), 256, 0, as_stream(stream), kind, y, y_pred, grad,
             static_cast<long long>(n), classes);
  DLB_LAUNCH_CHECK("loss_bwd");
  return DLB_OK;
}

extern "C" int dlb_ce_from_ids_fwd(const int32_t *target_ids, const float *y_pred, float *error, int n,
                                   int classes, float epsilon, void *stream) {
  DLB_REQUIRE(n >= 0 && classes > 0, DLB_ERR_INVALID_ARG, "ce_from_ids_fwd: n=%d classes=%d", n, classes);
  if (n == 0) return DLB_OK;
  DLB_REQUIRE(target_ids && y_pred && error, DLB_ERR_INVALID_ARG, "ce_from_ids_fwd: null pointer");
  launch_pdl(ce_ids_fwd_kernel, blocks_for(n, 256), 256, 0, as_stream(stream), target_ids, y_pred, error, n,
             classes, epsilon);
  DLB_LAUNCH_CHECK("ce_from_ids_fwd");
  return DLB_OK;
}

extern "C" int dlb_ce_from_ids_bwd(const int32_t *target_ids, const float *y_pred, float *grad, int n,
                                   int classes, float epsilon, void *stream) {
  DLB_REQUIRE(n >= 0 && classes > 0, DLB_ERR_INVALID_ARG, "ce_from_ids_bwd: n=%d classes=%d", n, classes);
  if (n == 0) return DLB_OK;
  DLB_REQUIRE(target_ids && y_pred && grad, DLB_ERR_INVALID_ARG, "ce_from_ids_bwd: null pointer");
  launch_pdl(ce_ids_bwd_kernel, blocks_for(static_cast<long long>(n) * classes, 256), 256, 0,
             as_stream(stream), target_ids, y_pred, grad, n, classes, epsilon);
  DLB_LAUNCH_CHECK("ce_from_ids_bwd");
  return DLB_OK;
}
