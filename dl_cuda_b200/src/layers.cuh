// The pieces of dl-cuda's src/layers.cuh that the embedding / positional-
// encoding / activation layers depend on: the thread-count constant, the
// process-wide initialisation seed (:8-21) and the cuRAND weight initialiser
// (:92-99).  The dense layers of that file (Linear, LSTM, RNN, Conv) are GEMM
// work outside this library.
#pragma once

#include <curand_kernel.h>

#include <cmath>
#include <cstdint>

#include "sequential.cuh"

static const short NUM_THREADS = 256;

// Seed that the next layer's weights derive from; layers consume it in
// construction order (seed + 9973 * n for the n-th layer built).
inline uint64_t &global_init_seed() {
  static uint64_t value = 42ULL;
  return value;
}

inline uint64_t next_init_seed() {
  static uint64_t layers_built = 0ULL;
  layers_built += 1ULL;
  return global_init_seed() + 9973ULL * layers_built;
}

inline void set_global_init_seed(uint64_t seed) { global_init_seed() = seed; }

// data[i] = N(0,1) * scale from the Philox/XORWOW stream curand_init(seed, i, 0)
// gives: the same values as the reference's initWeightsKernel, but the generator
// state lives in registers instead of a 48-byte-per-weight device array.
static __global__ void dlb_init_normal_kernel(float *data, int n, float scale, uint64_t seed) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  curandState_t state;
  curand_init(seed, i, 0, &state);
  data[i] = curand_normal(&state) * scale;
}

inline void dlb_init_normal(float *d_data, int n, float scale, uint64_t seed) {
  if (n <= 0) return;
  dlb_init_normal_kernel<<<(n + NUM_THREADS - 1) / NUM_THREADS, NUM_THREADS>>>(d_data, n, scale, seed);
  CUDA_CHECK(cudaGetLastError());
}
