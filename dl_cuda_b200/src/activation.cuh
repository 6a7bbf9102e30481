// ReLU / Sigmoid / Tanh / GELU activation layers with the interface of dl-cuda's
// src/activation.cuh (:57-119, :228-290): constructed from an element count,
// forward caches what backward needs.  Here the cache is written by the forward
// kernel itself (ReLU: one bit per element; Sigmoid/Tanh: the output; GELU: the
// input) instead of by a device-to-device copy around it.
#pragma once

#include "sequential.cuh"

template <int KIND>
class DlbActivation : public Operation {
public:
  explicit DlbActivation(int size)
      : size_(size), cache_(dlb_act_cache_bytes(KIND, size, DLB_F32)) {}

  int input_size() const override { return size_; }
  int output_size() const override { return size_; }

  void forward(float *d_input, float *d_output) override {
    DLB_CHECK(dlb_act_fwd(KIND, d_input, nullptr, d_output, cache_.get(), 1, size_, DLB_F32, nullptr));
  }

  void backward(float *d_output_grad, float *d_input_grad) override {
    DLB_CHECK(dlb_act_bwd(KIND, d_output_grad, cache_.get(), d_input_grad, nullptr, nullptr, 0, 1, size_,
                          DLB_F32, nullptr));
  }

private:
  int size_;
  DeviceBuffer<unsigned char> cache_;
};

class ReLUActivation : public DlbActivation<DLB_ACT_RELU> {
public:
  explicit ReLUActivation(int size) : DlbActivation(size) {}
};
class SigmoidActivation : public DlbActivation<DLB_ACT_SIGMOID> {
public:
  explicit SigmoidActivation(int size) : DlbActivation(size) {}
};
class TanhActivation : public DlbActivation<DLB_ACT_TANH> {
public:
  explicit TanhActivation(int size) : DlbActivation(size) {}
};
class GELUActivation : public DlbActivation<DLB_ACT_GELU> {
public:
  explicit GELUActivation(int size) : DlbActivation(size) {}
};

// Row softmax over [num_rows, row_width] (src/activation.cuh:167-201 of dl-cuda);
// the layer keeps its own copy of the probabilities for backward.
class SoftmaxActivation : public Operation {
public:
  SoftmaxActivation(int num_rows, int row_width)
      : rows_(num_rows), width_(row_width), probs_(static_cast<size_t>(num_rows) * row_width) {}

  int input_size() const override { return rows_ * width_; }
  int output_size() const override { return rows_ * width_; }

  void forward(float *d_input, float *d_output) override {
    // softmax into the layer's cache, then hand the caller a copy: backward must
    // not depend on what the caller does with d_output afterwards
    DLB_CHECK(dlb_softmax_fwd(d_input, probs_.get(), rows_, width_, 0, nullptr));
    CUDA_CHECK(cudaMemcpyAsync(d_output, probs_.get(), sizeof(float) * rows_ * width_, cudaMemcpyDeviceToDevice, 0));
  }

  void backward(float *d_output_grad, float *d_input_grad) override {
    DLB_CHECK(dlb_softmax_bwd(d_output_grad, probs_.get(), d_input_grad, rows_, width_, 1.0f, nullptr));
  }

private:
  int rows_, width_;
  DeviceBuffer<float> probs_;
};
