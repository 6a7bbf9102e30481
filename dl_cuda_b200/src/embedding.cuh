// EmbeddingLayer with the interface of dl-cuda's src/embedding.cuh (:32-104):
// same constructor, set_token_ids, forward/backward/update_weights, sizes and
// the single {table, grad} parameter group.  The kernels are the library's:
// a vectorised gather forward and, backward, a deterministic sorted-segment sum
// that writes every row of the gradient once (no memset, no atomics).
#pragma once

#include "layers.cuh"
#include "sequential.cuh"

class EmbeddingLayer : public Operation {
public:
  EmbeddingLayer(int vocab_size, int embedding_dim, int num_tokens)
      : vocab_(vocab_size), dim_(embedding_dim), tokens_(num_tokens),
        table_(static_cast<size_t>(vocab_size) * embedding_dim),
        grad_(static_cast<size_t>(vocab_size) * embedding_dim),
        ids_(static_cast<size_t>(num_tokens)),
        plan_(dlb_embed_workspace_bytes(num_tokens, vocab_size, embedding_dim)) {
    dlb_init_normal(table_.get(), vocab_ * dim_, sqrtf(2.0f / embedding_dim), next_init_seed());
  }

  int input_size() const override { return tokens_; }
  int output_size() const override { return tokens_ * dim_; }

  // h_token_ids: host array of num_tokens ids.  The sorted-segment plan that
  // backward needs depends on the ids alone, so it is built here, once per batch.
  void set_token_ids(const int *h_token_ids) {
    CUDA_CHECK(cudaMemcpy(ids_.get(), h_token_ids, sizeof(int) * tokens_, cudaMemcpyHostToDevice));
    DLB_CHECK(dlb_embed_sort_tokens(ids_.get(), plan_.get(), plan_.count(), tokens_, vocab_, dim_, nullptr));
    plan_valid_ = true;
  }

  void forward(float * /*d_input*/, float *d_output) override {
    DLB_CHECK(dlb_embed_gather_fwd(table_.get(), ids_.get(), nullptr, 0, d_output, tokens_, vocab_, dim_,
                                   DLB_F32, nullptr));
  }

  void backward(float *d_output_grad, float * /*d_input_grad*/) override {
    if (!plan_valid_) {  // ids were never set: whatever the id buffer holds, as in the reference
      DLB_CHECK(dlb_embed_sort_tokens(ids_.get(), plan_.get(), plan_.count(), tokens_, vocab_, dim_, nullptr));
      plan_valid_ = true;
    }
    DLB_CHECK(dlb_embed_scatter_bwd(d_output_grad, ids_.get(), grad_.get(), plan_.get(), plan_.count(),
                                    tokens_, vocab_, dim_, DLB_F32, nullptr));
  }

  void update_weights(float lr) override {
    DLB_CHECK(dlb_sgd_update(table_.get(), grad_.get(), lr, static_cast<int64_t>(vocab_) * dim_, nullptr));
  }

  std::vector<ParamGroup> get_param_groups() override {
    return {{table_.get(), grad_.get(), vocab_ * dim_}};
  }

private:
  int vocab_, dim_, tokens_;
  DeviceBuffer<float> table_, grad_;
  DeviceBuffer<int> ids_;
  DeviceBuffer<unsigned char> plan_;
  bool plan_valid_ = false;
};
