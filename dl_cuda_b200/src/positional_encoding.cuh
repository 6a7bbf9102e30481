// PositionalEncoding with the interface of dl-cuda's
// src/positional_encoding.cuh (:19-71): the sinusoidal table is built on the host
// with float powf/sinf/cosf exactly as there; forward adds it to every batch
// element, backward passes the gradient through.
#pragma once

#include <vector>

#include "sequential.cuh"

class PositionalEncoding : public Operation {
public:
  PositionalEncoding(int batch_size, int max_seq_len, int d_model)
      : batch_(batch_size), seq_(max_seq_len), dim_(d_model),
        table_(static_cast<size_t>(max_seq_len) * d_model) {
    std::vector<float> host(table_.count());
    DLB_CHECK(dlb_pe_build_table_host(host.data(), seq_, dim_));
    CUDA_CHECK(cudaMemcpy(table_.get(), host.data(), sizeof(float) * host.size(), cudaMemcpyHostToDevice));
  }

  int input_size() const override { return batch_ * seq_ * dim_; }
  int output_size() const override { return batch_ * seq_ * dim_; }

  void forward(float *d_input, float *d_output) override {
    DLB_CHECK(dlb_pe_add_fwd(d_input, table_.get(), d_output, batch_, seq_, dim_, DLB_F32, nullptr));
  }

  void backward(float *d_output_grad, float *d_input_grad) override {
    DLB_CHECK(dlb_pe_add_bwd(d_output_grad, d_input_grad, static_cast<int64_t>(batch_) * seq_ * dim_, DLB_F32,
                             nullptr));
  }

  // Device table [max_seq_len, d_model]: lets a caller fuse the add into the
  // embedding gather (dlb_embed_gather_fwd takes it directly).
  const float *table() const { return table_.get(); }

private:
  int batch_, seq_, dim_;
  DeviceBuffer<float> table_;
};
