// Fixed-order reductions shared by the kernels: a CTA-wide sum, and the second
// stage that adds per-CTA column partials [n_partial][ncols] into the final
// parameter gradients.  No atomics anywhere, so results are reproducible.
#pragma once

#include "common.cuh"

namespace dlb {

// Sum of v over the CTA; every thread gets the result.  red holds kBlock/32 floats.
template <int kBlock>
__device__ __forceinline__ float block_sum(float v, float *red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < kBlock / 32; w++) t += red[w];
  return t;
}

constexpr int kFinalizeWarps = 32;

// out[c] = sum_p partial[p][c].  A CTA owns 32*VEC adjacent columns (VEC per
// lane); warp w adds the rows of its contiguous slice top to bottom, then the
// slices are added in warp order.  Columns [0,n0) go to out0, the rest to out1.
template <int VEC>
static __global__ void __launch_bounds__(kFinalizeWarps * 32)
colsum_finalize_kernel(const float *partial, int n_partial, int ncols,
                       float *__restrict__ out0, int n0, float *__restrict__ out1) {
  pdl_prologue();
  __shared__ float slice[kFinalizeWarps][32 * VEC];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = (blockIdx.x * 32 + lane) * VEC;
  const int per = (n_partial + kFinalizeWarps - 1) / kFinalizeWarps;
  const int p0 = min(n_partial, warp * per);
  const int p1 = min(n_partial, p0 + per);
  float t[VEC];
#pragma unroll
  for (int i = 0; i < VEC; i++) t[i] = 0.f;
  if (col < ncols) {
#pragma unroll 4
    for (int p = p0; p < p1; p++) {
      const float *src = partial + static_cast<size_t>(p) * ncols + col;
      if constexpr (VEC == 4) {
        const float4 v = __ldcg(reinterpret_cast<const float4 *>(src));
        t[0] += v.x; t[1] += v.y; t[2] += v.z; t[3] += v.w;
      } else {
        t[0] += __ldcg(src);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VEC; i++) slice[warp][lane * VEC + i] = t[i];
  __syncthreads();
  const int c = threadIdx.x;  // one column of the CTA's 32*VEC per thread
  if (c < 32 * VEC) {
    const int gcol = blockIdx.x * 32 * VEC + c;
    if (gcol < ncols) {
      float r = 0.f;
#pragma unroll
      for (int w = 0; w < kFinalizeWarps; w++) r += slice[w][c];
      if (gcol < n0)
        out0[gcol] = r;
      else
        out1[gcol - n0] = r;
    }
  }
}

static inline int colsum_finalize(const float *partial, int n_partial, int ncols, float *out0,
                                  int n0, float *out1, cudaStream_t st) {
  if (ncols % 4 == 0 && n0 % 4 == 0 && aligned16(partial)) {
    launch_pdl(colsum_finalize_kernel<4>, (ncols / 4 + 31) / 32, kFinalizeWarps * 32, 0, st, partial,
               n_partial, ncols, out0, n0, out1);
  } else {
    launch_pdl(colsum_finalize_kernel<1>, (ncols + 31) / 32, kFinalizeWarps * 32, 0, st, partial,
               n_partial, ncols, out0, n0, out1);
  }
  DLB_LAUNCH_CHECK("colsum_finalize");
  return DLB_OK;
}

}  // namespace dlb
