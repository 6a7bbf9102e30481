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

constexpr int kFinalizeWarps = 8;

// out[c] = sum_p partial[p][c].  A CTA owns 32 adjacent columns (one per lane);
// warp w adds the rows of its contiguous slice top to bottom, then the slices
// are added in warp order.  Columns [0,n0) go to out0, the rest to out1.
static __global__ void __launch_bounds__(kFinalizeWarps * 32)
colsum_finalize_kernel(const float *__restrict__ partial, int n_partial, int ncols,
                       float *__restrict__ out0, int n0, float *__restrict__ out1) {
  __shared__ float slice[kFinalizeWarps][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = blockIdx.x * 32 + lane;
  const int per = (n_partial + kFinalizeWarps - 1) / kFinalizeWarps;
  const int p0 = warp * per;
  const int p1 = min(n_partial, p0 + per);
  float t = 0.f;
  if (col < ncols) {
#pragma unroll 8
    for (int p = p0; p < p1; p++) t += partial[static_cast<size_t>(p) * ncols + col];
  }
  slice[warp][lane] = t;
  __syncthreads();
  if (warp == 0 && col < ncols) {
    float r = 0.f;
#pragma unroll
    for (int w = 0; w < kFinalizeWarps; w++) r += slice[w][lane];
    if (col < n0)
      out0[col] = r;
    else
      out1[col - n0] = r;
  }
}

static inline int colsum_finalize(const float *partial, int n_partial, int ncols, float *out0,
                                  int n0, float *out1, cudaStream_t st) {
  const int grid = (ncols + 31) / 32;
  colsum_finalize_kernel<<<grid, kFinalizeWarps * 32, 0, st>>>(partial, n_partial, ncols, out0, n0,
                                                               out1);
  DLB_LAUNCH_CHECK("colsum_finalize");
  return DLB_OK;
}

}  // namespace dlb
