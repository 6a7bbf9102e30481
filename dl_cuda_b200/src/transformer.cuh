// TransformerLayer / TransformerStack with the interface of dl-cuda's
// src/transformer.cuh (:224-734, :736-824): post-norm encoder block
//   a   = MultiHeadAttention(x)            (no projection biases, optional causal mask)
//   h   = LayerNorm1(x + a)
//   f   = W2 * GELU(W1 * h + b1) + b2
//   out = LayerNorm2(h + f)
// with the same constructor, set_causal, parameter initialisation
// (std::mt19937(42), one normal_distribution per tensor, in the order q, k, v,
// wo, ff1, ff2) and the same twelve parameter groups, so checkpoints written by
// either implementation load into the other.
//
// What differs is where the time goes.  The residual adds are folded into the
// layer-norm kernels (forward reads both addends, backward reads both gradient
// streams), the FFN bias add and bias gradient ride in the GELU kernels, the
// layer-norm parameter gradients come out of the same pass as dx, and attention
// runs over all (batch, head) pairs in one launch per product, addressing heads
// by stride inside [tokens, d_model] instead of through reshaped copies.
#pragma once

#include <algorithm>
#include <cmath>
#include <random>
#include <vector>

#include "layers.cuh"
#include "sequential.cuh"

class TransformerLayer : public Operation {
public:
  TransformerLayer(int batch_size, int sequence_length, int d_model, int num_heads, float dropout_prob,
                   int d_ff = 0)
      : batch_(batch_size), seq_(sequence_length), dim_(d_model), ff_(d_ff > 0 ? d_ff : 4 * d_model),
        heads_(num_heads), head_dim_(d_model / num_heads), dropout_prob_(dropout_prob) {
    const size_t tokens = static_cast<size_t>(batch_) * seq_;
    const size_t act = tokens * dim_, wide = tokens * ff_;
    const size_t scores = static_cast<size_t>(batch_) * heads_ * seq_ * seq_;
    const size_t sq = static_cast<size_t>(dim_) * dim_, w1 = static_cast<size_t>(dim_) * ff_;

    for (Param *p : {&wq_, &wk_, &wv_, &wo_}) p->alloc(sq);
    w1_.alloc(w1);
    b1_.alloc(ff_);
    w2_.alloc(w1);
    b2_.alloc(dim_);
    for (Param *p : {&gamma1_, &beta1_, &gamma2_, &beta2_}) p->alloc(dim_);

    for (DeviceBuffer<float> *b : {&x_, &q_, &k_, &v_, &ctx_, &attn_out_, &xhat1_, &h_, &ff_out_, &xhat2_,
                                   &g_, &dres_, &dq_, &dk_, &dv_, &dctx_})
      b->reset(act);
    for (DeviceBuffer<float> *b : {&ff_pre_, &ff_act_, &ff_grad_}) b->reset(wide);
    probs_.reset(scores);
    dprobs_.reset(scores);
    inv_std1_.reset(tokens);
    inv_std2_.reset(tokens);

    const int rows = static_cast<int>(tokens);
    size_t ws = dlb_ln_bwd_workspace_bytes(rows, dim_);
    ws = std::max(ws, dlb_act_bwd_workspace_bytes(DLB_ACT_GELU, rows, ff_));
    ws = std::max(ws, dlb_bias_grad_workspace_bytes(rows, dim_));
    workspace_.reset(ws + 16);

    // Host-side initialisation: one generator for the whole layer, a fresh
    // distribution object per tensor (its cached second variate is dropped
    // between tensors).
    std::mt19937 rng(42);
    auto fill_normal = [&rng](Param &p, float stddev) {
      std::normal_distribution<float> draw(0.0f, stddev);
      std::vector<float> host(p.size);
      for (float &w : host) w = draw(rng);
      CUDA_CHECK(cudaMemcpy(p.value.get(), host.data(), sizeof(float) * p.size, cudaMemcpyHostToDevice));
    };
    const float attn_std = sqrtf(2.0f / dim_);
    for (Param *p : {&wq_, &wk_, &wv_, &wo_}) fill_normal(*p, attn_std);
    fill_normal(w1_, sqrtf(2.0f / dim_));
    fill_normal(w2_, sqrtf(2.0f / ff_));

    const std::vector<float> ones(dim_, 1.0f);
    for (Param *p : {&gamma1_, &gamma2_})
      CUDA_CHECK(cudaMemcpy(p->value.get(), ones.data(), sizeof(float) * dim_, cudaMemcpyHostToDevice));
    for (Param *p : {&beta1_, &beta2_, &b1_, &b2_}) CUDA_CHECK(cudaMemset(p->value.get(), 0, sizeof(float) * p->size));
  }

  void set_causal(bool causal) { causal_ = causal; }

  int input_size() const override { return batch_ * seq_ * dim_; }
  int output_size() const override { return batch_ * seq_ * dim_; }

  void forward(float *input, float *output) override {
    const int T = batch_ * seq_, D = dim_, F = ff_;
    const float inv_scale = 1.0f / sqrtf(static_cast<float>(head_dim_));

    // the weight gradients need x after the caller has moved on
    CUDA_CHECK(cudaMemcpyAsync(x_.get(), input, sizeof(float) * T * D, cudaMemcpyDeviceToDevice, 0));

    dlb_dense(input, D, 1, wq_.value.get(), D, 1, nullptr, q_.get(), T, D, D);
    dlb_dense(input, D, 1, wk_.value.get(), D, 1, nullptr, k_.get(), T, D, D);
    dlb_dense(input, D, 1, wv_.value.get(), D, 1, nullptr, v_.get(), T, D, D);

    // P[b,h] = softmax(Q_h K_h^T / sqrt(hd)) ; ctx[b, :, h] = P V_h
    per_head(q_.get(), D, 1, k_.get(), 1, D, probs_.get(), /*c_is_scores=*/true, seq_, seq_, head_dim_, inv_scale);
    DLB_CHECK(dlb_softmax_fwd(probs_.get(), probs_.get(), static_cast<int64_t>(batch_) * heads_ * seq_, seq_,
                              causal_ ? seq_ : 0, nullptr));
    per_head(probs_.get(), seq_, 1, v_.get(), D, 1, ctx_.get(), /*c_is_scores=*/false, seq_, head_dim_, seq_, 1.0f,
             /*a_is_scores=*/true);

    dlb_dense(ctx_.get(), D, 1, wo_.value.get(), D, 1, nullptr, attn_out_.get(), T, D, D);

    DLB_CHECK(dlb_ln_residual_fwd(input, attn_out_.get(), gamma1_.value.get(), beta1_.value.get(), h_.get(),
                                  xhat1_.get(), inv_std1_.get(), T, D, kEps, DLB_F32, nullptr));

    // W1 h, then bias + GELU in one pass that also keeps the pre-activation for backward
    dlb_dense(h_.get(), D, 1, w1_.value.get(), F, 1, nullptr, ff_act_.get(), T, F, D);
    DLB_CHECK(dlb_act_fwd(DLB_ACT_GELU, ff_act_.get(), b1_.value.get(), ff_act_.get(), ff_pre_.get(), T, F,
                          DLB_F32, nullptr));
    dlb_dense(ff_act_.get(), F, 1, w2_.value.get(), D, 1, b2_.value.get(), ff_out_.get(), T, D, F);

    DLB_CHECK(dlb_ln_residual_fwd(h_.get(), ff_out_.get(), gamma2_.value.get(), beta2_.value.get(), output,
                                  xhat2_.get(), inv_std2_.get(), T, D, kEps, DLB_F32, nullptr));
  }

  void backward(float *d_output_grad, float *d_input_grad) override {
    const int T = batch_ * seq_, D = dim_, F = ff_;
    const float inv_scale = 1.0f / sqrtf(static_cast<float>(head_dim_));
    void *ws = workspace_.get();
    const size_t ws_bytes = workspace_.count();

    // LayerNorm2: g = d(h + f), with d(gamma2), d(beta2) from the same pass
    DLB_CHECK(dlb_ln_bwd(d_output_grad, nullptr, xhat2_.get(), inv_std2_.get(), gamma2_.value.get(), g_.get(),
                         gamma2_.grad.get(), beta2_.grad.get(), ws, ws_bytes, T, D, DLB_F32, nullptr));

    // FFN: second linear, GELU (+ d(b1)), first linear
    dlb_dense(g_.get(), D, 1, w2_.value.get(), 1, D, nullptr, ff_grad_.get(), T, F, D);
    dlb_dense(ff_act_.get(), 1, F, g_.get(), D, 1, nullptr, w2_.grad.get(), F, D, T);
    DLB_CHECK(dlb_bias_grad(g_.get(), b2_.grad.get(), ws, ws_bytes, T, D, DLB_F32, nullptr));
    DLB_CHECK(dlb_act_bwd(DLB_ACT_GELU, ff_grad_.get(), ff_pre_.get(), ff_grad_.get(), b1_.grad.get(), ws,
                          ws_bytes, T, F, DLB_F32, nullptr));
    dlb_dense(ff_grad_.get(), F, 1, w1_.value.get(), 1, F, nullptr, ff_out_.get(), T, D, F);
    dlb_dense(h_.get(), 1, D, ff_grad_.get(), F, 1, nullptr, w1_.grad.get(), D, F, T);

    // LayerNorm1 over the sum of the skip gradient g and the FFN input gradient
    DLB_CHECK(dlb_ln_bwd(g_.get(), ff_out_.get(), xhat1_.get(), inv_std1_.get(), gamma1_.value.get(), dres_.get(),
                         gamma1_.grad.get(), beta1_.grad.get(), ws, ws_bytes, T, D, DLB_F32, nullptr));

    // skip path of the attention block
    CUDA_CHECK(cudaMemcpyAsync(d_input_grad, dres_.get(), sizeof(float) * T * D, cudaMemcpyDeviceToDevice, 0));

    // output projection
    dlb_dense(dres_.get(), D, 1, wo_.value.get(), 1, D, nullptr, dctx_.get(), T, D, D);
    dlb_dense(ctx_.get(), 1, D, dres_.get(), D, 1, nullptr, wo_.grad.get(), D, D, T);

    // attention core, all (batch, head) pairs per launch
    //   dP = dctx_h V_h^T ; dV_h = P^T dctx_h ; dS = P*(dP - <dP,P>)/sqrt(hd) ; dQ_h = dS K_h ; dK_h = dS^T Q_h
    per_head(dctx_.get(), D, 1, v_.get(), 1, D, dprobs_.get(), true, seq_, seq_, head_dim_, 1.0f);
    per_head(probs_.get(), 1, seq_, dctx_.get(), D, 1, dv_.get(), false, seq_, head_dim_, seq_, 1.0f, true);
    DLB_CHECK(dlb_softmax_bwd(dprobs_.get(), probs_.get(), dprobs_.get(),
                              static_cast<int64_t>(batch_) * heads_ * seq_, seq_, inv_scale, nullptr));
    per_head(dprobs_.get(), seq_, 1, k_.get(), D, 1, dq_.get(), false, seq_, head_dim_, seq_, 1.0f, true);
    per_head(dprobs_.get(), 1, seq_, q_.get(), D, 1, dk_.get(), false, seq_, head_dim_, seq_, 1.0f, true);

    // input projections: dx += dQ Wq^T + dK Wk^T + dV Wv^T, in that order
    dlb_dense(dq_.get(), D, 1, wq_.value.get(), 1, D, nullptr, d_input_grad, T, D, D, /*accumulate=*/true);
    dlb_dense(dk_.get(), D, 1, wk_.value.get(), 1, D, nullptr, d_input_grad, T, D, D, true);
    dlb_dense(dv_.get(), D, 1, wv_.value.get(), 1, D, nullptr, d_input_grad, T, D, D, true);
    dlb_dense(x_.get(), 1, D, dq_.get(), D, 1, nullptr, wq_.grad.get(), D, D, T);
    dlb_dense(x_.get(), 1, D, dk_.get(), D, 1, nullptr, wk_.grad.get(), D, D, T);
    dlb_dense(x_.get(), 1, D, dv_.get(), D, 1, nullptr, wv_.grad.get(), D, D, T);
  }

  void update_weights(float lr) override {
    for (Param *p : ordered()) DLB_CHECK(dlb_sgd_update(p->value.get(), p->grad.get(), lr, p->size, nullptr));
  }

  std::vector<ParamGroup> get_param_groups() override {
    std::vector<ParamGroup> groups;
    for (Param *p : ordered()) groups.push_back({p->value.get(), p->grad.get(), static_cast<int>(p->size)});
    return groups;
  }

private:
  static constexpr float kEps = 1e-5f;

  struct Param {
    DeviceBuffer<float> value, grad;
    size_t size = 0;
    void alloc(size_t n) {
      size = n;
      value.reset(n);
      grad.reset(n);
    }
  };

  // Checkpoint order of the reference: attention weights, FFN, then the two layer norms.
  std::vector<Param *> ordered() {
    return {&wq_, &wk_, &wv_, &wo_, &w1_, &b1_, &w2_, &b2_, &gamma1_, &beta1_, &gamma2_, &beta2_};
  }

  // One batched product over the batch*heads (batch, head) pairs.  An operand
  // that is a score matrix is a dense [seq, seq] block per pair; any other
  // operand is the head's column slice of a [tokens, d_model] activation.
  void per_head(const float *a, long long a_row, long long a_col, const float *b, long long b_row, long long b_col,
                float *c, bool c_is_scores, int m, int n, int k, float alpha, bool a_is_scores = false) {
    const long long block = static_cast<long long>(seq_) * seq_;
    const long long act_outer = static_cast<long long>(seq_) * dim_, act_inner = head_dim_;
    const long long sc_outer = block * heads_, sc_inner = block;
    DLB_CHECK(dlb_gemm_f32(a, b, nullptr, c, m, n, k, a_row, a_col, b_row, b_col, c_is_scores ? seq_ : dim_,
                           batch_ * heads_, heads_, a_is_scores ? sc_outer : act_outer,
                           a_is_scores ? sc_inner : act_inner, act_outer, act_inner,
                           c_is_scores ? sc_outer : act_outer, c_is_scores ? sc_inner : act_inner, alpha, 0,
                           nullptr));
  }

  int batch_, seq_, dim_, ff_, heads_, head_dim_;
  float dropout_prob_;  // accepted and stored; the block applies no dropout, as in the reference
  bool causal_ = false;

  Param wq_, wk_, wv_, wo_, w1_, b1_, w2_, b2_, gamma1_, beta1_, gamma2_, beta2_;

  // forward state kept for backward
  DeviceBuffer<float> x_, q_, k_, v_, probs_, ctx_, attn_out_, xhat1_, inv_std1_, h_, ff_pre_, ff_act_, ff_out_,
      xhat2_, inv_std2_;
  // backward scratch
  DeviceBuffer<float> g_, ff_grad_, dres_, dprobs_, dq_, dk_, dv_, dctx_;
  DeviceBuffer<unsigned char> workspace_;
};

// num_layers blocks chained through buffers owned by the stack (src/transformer.cuh:736-824).
class TransformerStack : public Operation {
public:
  TransformerStack(int num_layers, int batch_size, int sequence_length, int d_model, int num_heads,
                   float dropout_prob, int d_ff = 0, bool causal = false)
      : size_(batch_size * sequence_length * d_model) {
    for (int i = 0; i < num_layers; i++) {
      blocks_.push_back(new TransformerLayer(batch_size, sequence_length, d_model, num_heads, dropout_prob, d_ff));
      if (causal) blocks_.back()->set_causal(true);
    }
    // ping-pong buffers: block i reads one and writes the other
    if (num_layers > 1) {
      for (DeviceBuffer<float> &b : hop_) b.reset(static_cast<size_t>(size_));
    }
  }

  TransformerStack(const TransformerStack &) = delete;
  TransformerStack &operator=(const TransformerStack &) = delete;

  ~TransformerStack() override {
    for (TransformerLayer *block : blocks_) delete block;
  }

  int input_size() const override { return size_; }
  int output_size() const override { return size_; }

  void forward(float *input, float *output) override {
    const int n = static_cast<int>(blocks_.size());
    float *src = input;
    for (int i = 0; i < n; i++) {
      float *dst = (i + 1 == n) ? output : hop_[i % 2].get();
      blocks_[i]->forward(src, dst);
      src = dst;
    }
  }

  void backward(float *d_output_grad, float *d_input_grad) override {
    const int n = static_cast<int>(blocks_.size());
    float *src = d_output_grad;
    for (int i = n - 1; i >= 0; i--) {
      float *dst = (i == 0) ? d_input_grad : hop_[i % 2].get();
      blocks_[i]->backward(src, dst);
      src = dst;
    }
  }

  void update_weights(float lr) override {
    for (TransformerLayer *block : blocks_) block->update_weights(lr);
  }

  std::vector<ParamGroup> get_param_groups() override {
    std::vector<ParamGroup> groups;
    for (TransformerLayer *block : blocks_) {
      const std::vector<ParamGroup> own = block->get_param_groups();
      groups.insert(groups.end(), own.begin(), own.end());
    }
    return groups;
  }

private:
  int size_;
  std::vector<TransformerLayer *> blocks_;
  DeviceBuffer<float> hop_[2];
};
