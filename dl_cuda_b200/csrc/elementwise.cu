// The small streaming kernels of the path: residual add, positional-encoding
// add on its own (for callers that do not use the fused gather), its identity
// backward, the SGD step EmbeddingLayer::update_weights uses, and the host-side
// builder of the sinusoidal table.
#include "common.cuh"

#include <cmath>

namespace dlb {
namespace {

constexpr int kBlock = 256;
constexpr int kUnroll = 4;

// out = a + b over n elements (n a multiple of the vector width).  A warp reads
// kUnroll consecutive 512-byte pieces per operand before it adds and stores.
template <typename T, bool kCopy>
__global__ void __launch_bounds__(kBlock)
add_kernel(const T *a, const T *b, T *out, int64_t nvec) {
  pdl_prologue();
  using S = Store<T>;
  constexpr int E = S::kPerVec;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kBlock;
  for (int64_t v0 = static_cast<int64_t>(blockIdx.x) * kBlock + threadIdx.x; v0 < nvec;
       v0 += stride * kUnroll) {
    uint4 va[kUnroll], vb[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; u++) {
      const int64_t v = v0 + u * stride;
      if (v < nvec) {
        va[u] = ld_stream(a + v * E);
        if (!kCopy) vb[u] = ld_stream(b + v * E);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; u++) {
      const int64_t v = v0 + u * stride;
      if (v < nvec) {
        if (kCopy) {
          st_stream(out + v * E, va[u]);
        } else {
          float fa[E], fb[E];
          S::unpack(va[u], fa);
          S::unpack(vb[u], fb);
#pragma unroll
          for (int e = 0; e < E; e++) fa[e] = fa[e] + fb[e];
          st_stream(out + v * E, S::pack(fa));
        }
      }
    }
  }
}

template <typename T, bool kCopy>
__global__ void __launch_bounds__(kBlock)
add_scalar_kernel(const T *a, const T *b, T *out, int64_t n) {
  pdl_prologue();
  using S = Store<T>;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kBlock + threadIdx.x;
  if (i >= n) return;
  out[i] = kCopy ? a[i] : S::from_float(S::to_float(a[i]) + S::to_float(b[i]));
}

// out[b,s,:] = in[b,s,:] + pe[s,:]; blockDim = (tx, ty) as in the gather: a
// thread keeps its PE vector and walks the batch.
template <typename T>
__global__ void __launch_bounds__(kBlock)
pe_add_kernel(const T *in, const float *__restrict__ pe, T *out, int batch, int seq_len, int d) {
  pdl_prologue();
  using S = Store<T>;
  constexpr int E = S::kPerVec;
  const int ncv = d / E;
  const int cv = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.y * blockDim.y + threadIdx.y;
  if (cv >= ncv || s >= seq_len) return;
  float pv[E];
#pragma unroll
  for (int q = 0; q < E / 4; q++) {
    const float4 p4 = ld_const_f4(pe + static_cast<size_t>(s) * d + cv * E + 4 * q);
    pv[4 * q] = p4.x; pv[4 * q + 1] = p4.y; pv[4 * q + 2] = p4.z; pv[4 * q + 3] = p4.w;
  }
  for (int b0 = 0; b0 < batch; b0 += kUnroll) {
    uint4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; u++)
      if (b0 + u < batch)
        v[u] = ld_stream(in + (static_cast<size_t>(b0 + u) * seq_len + s) * d + cv * E);
#pragma unroll
    for (int u = 0; u < kUnroll; u++) {
      if (b0 + u < batch) {
        float f[E];
        S::unpack(v[u], f);
#pragma unroll
        for (int e = 0; e < E; e++) f[e] = f[e] + pv[e];
        st_stream(out + (static_cast<size_t>(b0 + u) * seq_len + s) * d + cv * E, S::pack(f));
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kBlock)
pe_add_scalar_kernel(const T *in, const float *__restrict__ pe, T *out, int64_t total,
                     int64_t period) {
  pdl_prologue();
  using S = Store<T>;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kBlock + threadIdx.x;
  if (i >= total) return;
  out[i] = S::from_float(S::to_float(in[i]) + pe[i % period]);
}

__global__ void __launch_bounds__(kBlock)
sgd_kernel(float *__restrict__ p, const float *g, float lr, int64_t n) {
  pdl_prologue();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kBlock;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kBlock + threadIdx.x; i < n; i += stride)
    p[i] -= lr * g[i];
}

unsigned stream_grid(int64_t work_items) {
  const int64_t want = ceil_div<int64_t>(work_items, static_cast<int64_t>(kBlock) * kUnroll);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
  return static_cast<unsigned>(want < 1 ? 1 : (want < cap ? want : cap));
}

template <typename T, bool kCopy>
int add_typed(const void *a, const void *b, void *out, int64_t n, cudaStream_t st) {
  constexpr int E = Store<T>::kPerVec;
  if (n % E == 0 && aligned16(a) && (kCopy || aligned16(b)) && aligned16(out)) {
    const int64_t nvec = n / E;
    launch_pdl(add_kernel<T, kCopy>, stream_grid(nvec), kBlock, 0, st, 
        static_cast<const T *>(a), static_cast<const T *>(b), static_cast<T *>(out), nvec);
    DLB_LAUNCH_CHECK("add");
    return DLB_OK;
  }
  launch_pdl(add_scalar_kernel<T, kCopy>, static_cast<unsigned>(ceil_div<int64_t>(n, kBlock)), kBlock, 0, st, 
      static_cast<const T *>(a), static_cast<const T *>(b), static_cast<T *>(out), n);
  DLB_LAUNCH_CHECK("add_scalar");
  return DLB_OK;
}

template <typename T>
int pe_add_typed(const void *in, const float *pe, void *out, int batch, int seq_len, int d,
                 cudaStream_t st) {
  constexpr int E = Store<T>::kPerVec;
  int tx = 1;
  while (tx < kBlock && tx < d / E) tx *= 2;
  const int ty = kBlock / tx;
  if (d % E == 0 && aligned16(in) && aligned16(out) && aligned16(pe) &&
      ceil_div(seq_len, ty) <= 65535) {
    dim3 grid(ceil_div(d / E, tx), ceil_div(seq_len, ty));
    launch_pdl(pe_add_kernel<T>, grid, dim3(tx, ty), 0, st, static_cast<const T *>(in), pe,
                                                    static_cast<T *>(out), batch, seq_len, d);
    DLB_LAUNCH_CHECK("pe_add");
    return DLB_OK;
  }
  const int64_t period = static_cast<int64_t>(seq_len) * d, total = period * batch;
  launch_pdl(pe_add_scalar_kernel<T>, static_cast<unsigned>(ceil_div<int64_t>(total, kBlock)), kBlock, 0, st, 
      static_cast<const T *>(in), pe, static_cast<T *>(out), total, period);
  DLB_LAUNCH_CHECK("pe_add_scalar");
  return DLB_OK;
}

}  // namespace
}  // namespace dlb

using namespace dlb;

extern "C" int dlb_residual_add(const void *a, const void *b, void *out, int64_t n, int dtype,
                                void *stream) {
  DLB_REQUIRE(n >= 0, DLB_ERR_INVALID_ARG, "residual_add: n=%lld", static_cast<long long>(n));
  if (n == 0) return DLB_OK;
  DLB_REQUIRE(a && b && out, DLB_ERR_INVALID_ARG, "residual_add: null pointer");
  if (dtype == DLB_F32) return add_typed<float, false>(a, b, out, n, as_stream(stream));
  if (dtype == DLB_BF16) return add_typed<__nv_bfloat16, false>(a, b, out, n, as_stream(stream));
  set_error("residual_add: unknown dtype %d", dtype);
  return DLB_ERR_INVALID_ARG;
}

extern "C" int dlb_pe_build_table_host(float *h_table, int seq_len, int d) {
  DLB_REQUIRE(h_table && seq_len >= 0 && d > 0, DLB_ERR_INVALID_ARG, "pe_build_table_host: bad arguments");
  for (int pos = 0; pos < seq_len; pos++) {
    float *row = h_table + static_cast<size_t>(pos) * d;
    for (int i = 0; i < d; i++) {
      const float exponent = static_cast<float>(2 * (i / 2)) / d;
      const float angle = static_cast<float>(pos) / powf(10000.0f, exponent);
      row[i] = (i % 2 == 0) ? sinf(angle) : cosf(angle);
    }
  }
  return DLB_OK;
}

extern "C" int dlb_pe_add_fwd(const void *in, const float *pe, void *out, int batch, int seq_len,
                              int d, int dtype, void *stream) {
  DLB_REQUIRE(batch >= 0 && seq_len >= 0 && d > 0, DLB_ERR_INVALID_ARG, "pe_add_fwd: bad shape");
  if (batch == 0 || seq_len == 0) return DLB_OK;
  DLB_REQUIRE(in && pe && out, DLB_ERR_INVALID_ARG, "pe_add_fwd: null pointer");
  if (dtype == DLB_F32) return pe_add_typed<float>(in, pe, out, batch, seq_len, d, as_stream(stream));
  if (dtype == DLB_BF16)
    return pe_add_typed<__nv_bfloat16>(in, pe, out, batch, seq_len, d, as_stream(stream));
  set_error("pe_add_fwd: unknown dtype %d", dtype);
  return DLB_ERR_INVALID_ARG;
}

extern "C" int dlb_pe_add_bwd(const void *dy, void *dx, int64_t n, int dtype, void *stream) {
  DLB_REQUIRE(n >= 0, DLB_ERR_INVALID_ARG, "pe_add_bwd: n=%lld", static_cast<long long>(n));
  if (n == 0 || dy == dx) return DLB_OK;
  DLB_REQUIRE(dy && dx, DLB_ERR_INVALID_ARG, "pe_add_bwd: null pointer");
  if (dtype == DLB_F32) return add_typed<float, true>(dy, nullptr, dx, n, as_stream(stream));
  if (dtype == DLB_BF16) return add_typed<__nv_bfloat16, true>(dy, nullptr, dx, n, as_stream(stream));
  set_error("pe_add_bwd: unknown dtype %d", dtype);
  return DLB_ERR_INVALID_ARG;
}

extern "C" int dlb_sgd_update(float *params, const float *grads, float lr, int64_t n, void *stream) {
  DLB_REQUIRE(n >= 0, DLB_ERR_INVALID_ARG, "sgd_update: n=%lld", static_cast<long long>(n));
  if (n == 0) return DLB_OK;
  DLB_REQUIRE(params && grads, DLB_ERR_INVALID_ARG, "sgd_update: null pointer");
  launch_pdl(sgd_kernel, stream_grid(n), kBlock, 0, as_stream(stream), params, grads, lr, n);
  DLB_LAUNCH_CHECK("sgd");
  return DLB_OK;
}
