// The pieces of dl-cuda's src/layers.cuh that the embedding / positional-
// encoding / activation layers depend on: the thread-count constant, the
// process-wide initialisation seed (:8-21) and the cuRAND weight initialiser
// (:92-99), and LinearLayer (:101-200).  The recurrent and convolution layers
// of that file are outside this library.
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

// Row-major product helper over the library's pass-through fp32 GEMM:
//   C[m,n] (+)= op(A) * op(B) + bias, with op chosen by the strides given.
inline void dlb_dense(const float *a, long long a_row, long long a_col, const float *b, long long b_row,
                      long long b_col, const float *bias, float *c, int m, int n, int k,
                      bool accumulate = false) {
  DLB_CHECK(dlb_gemm_f32(a, b, bias, c, m, n, k, a_row, a_col, b_row, b_col, n, 1, 1, 0, 0, 0, 0, 0, 0, 1.0f,
                         accumulate ? 1 : 0, nullptr));
}

// y = x W + b over n rows; W is [in_features, out_features] row-major, drawn
// from N(0, 2/in_features) with the layer's init seed, b starts at zero.
class LinearLayer : public Operation {
public:
  LinearLayer(int n, int in_features, int out_features)
      : rows_(n), in_(in_features), out_(out_features),
        weight_(static_cast<size_t>(in_features) * out_features),
        bias_(static_cast<size_t>(out_features)),
        weight_grad_(static_cast<size_t>(in_features) * out_features),
        bias_grad_(static_cast<size_t>(out_features)),
        input_(static_cast<size_t>(n) * in_features),
        bias_ws_(dlb_bias_grad_workspace_bytes(n, out_features) + 16) {
    dlb_init_normal(weight_.get(), in_ * out_, sqrtf(2.0f / in_features), next_init_seed());
    CUDA_CHECK(cudaMemset(bias_.get(), 0, sizeof(float) * out_));
  }

  int input_size() const override { return rows_ * in_; }
  int output_size() const override { return rows_ * out_; }

  float *get_weights() { return weight_.get(); }
  float *get_bias() { return bias_.get(); }
  float *get_weight_grad() { return weight_grad_.get(); }
  float *get_bias_grad() { return bias_grad_.get(); }
  int get_in_features() const { return in_; }
  int get_out_features() const { return out_; }
  int get_n() const { return rows_; }

  void forward(float *d_input, float *d_output) override {
    // backward needs x for the weight gradient and the caller may reuse its buffer
    CUDA_CHECK(cudaMemcpyAsync(input_.get(), d_input, sizeof(float) * rows_ * in_, cudaMemcpyDeviceToDevice, 0));
    dlb_dense(d_input, in_, 1, weight_.get(), out_, 1, bias_.get(), d_output, rows_, out_, in_);
  }

  void backward(float *d_output_grad, float *d_input_grad) override {
    // dx = dy W^T ; dW = x^T dy ; db = column sums of dy
    dlb_dense(d_output_grad, out_, 1, weight_.get(), 1, out_, nullptr, d_input_grad, rows_, in_, out_);
    dlb_dense(input_.get(), 1, in_, d_output_grad, out_, 1, nullptr, weight_grad_.get(), in_, out_, rows_);
    DLB_CHECK(dlb_bias_grad(d_output_grad, bias_grad_.get(), bias_ws_.get(), bias_ws_.count(), rows_, out_,
                            DLB_F32, nullptr));
  }

  void update_weights(float lr) override {
    DLB_CHECK(dlb_sgd_update(weight_.get(), weight_grad_.get(), lr, static_cast<int64_t>(in_) * out_, nullptr));
    DLB_CHECK(dlb_sgd_update(bias_.get(), bias_grad_.get(), lr, out_, nullptr));
  }

  std::vector<ParamGroup> get_param_groups() override {
    return {{weight_.get(), weight_grad_.get(), in_ * out_}, {bias_.get(), bias_grad_.get(), out_}};
  }

private:
  int rows_, in_, out_;
  DeviceBuffer<float> weight_, bias_, weight_grad_, bias_grad_, input_;
  DeviceBuffer<unsigned char> bias_ws_;
};
