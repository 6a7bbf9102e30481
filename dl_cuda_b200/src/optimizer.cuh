// Optimizer classes with the interface of dl-cuda's src/optimizer.cuh (:14-196) and the
// Sequential members it defines (:198-243).  A step is one kernel launch over all parameter
// groups instead of one per group, and clip_grad_norm reduces and scales every gradient on the
// device, reading the norm back once (the reference synchronises once per group).
#pragma once

#include <cmath>
#include <vector>

#include "layers.cuh"
#include "sequential.cuh"

class Optimizer {
public:
  virtual void step(float lr) = 0;
  virtual void register_params(const std::vector<ParamGroup> &groups) = 0;
  virtual ~Optimizer() = default;
};

// Holds the group list as the pointer/size arrays the C ABI takes, plus optional state buffers.
class DlbOptimizerBase : public Optimizer {
public:
  void register_params(const std::vector<ParamGroup> &groups) override {
    params_.clear(); grads_.clear(); sizes_.clear(); m_ptrs_.clear(); v_ptrs_.clear();
    m_.clear(); v_.clear();
    for (const ParamGroup &g : groups) {
      params_.push_back(g.params);
      grads_.push_back(g.grads);
      sizes_.push_back(g.size);
    }
    if (states_ >= 1) alloc_state(m_, m_ptrs_);
    if (states_ >= 2) alloc_state(v_, v_ptrs_);
    t_ = 0;
  }

protected:
  explicit DlbOptimizerBase(int states) : states_(states) {}

  void run(int kind, float lr, float beta1, float beta2, float eps, float weight_decay, float inv1, float inv2) {
    DLB_CHECK(dlb_optim_step(kind, static_cast<int>(params_.size()), params_.data(), grads_.data(),
                             m_ptrs_.empty() ? nullptr : m_ptrs_.data(), v_ptrs_.empty() ? nullptr : v_ptrs_.data(),
                             sizes_.data(), lr, beta1, beta2, eps, weight_decay, inv1, inv2, nullptr));
  }

  int t_ = 0;

private:
  void alloc_state(std::vector<DeviceBuffer<float>> &bufs, std::vector<float *> &ptrs) {
    bufs = std::vector<DeviceBuffer<float>>(sizes_.size());
    for (size_t i = 0; i < sizes_.size(); ++i) {
      bufs[i].reset(static_cast<size_t>(sizes_[i]));
      if (sizes_[i] > 0) CUDA_CHECK(cudaMemset(bufs[i].get(), 0, sizeof(float) * sizes_[i]));
      ptrs.push_back(bufs[i].get());
    }
  }

  int states_;
  std::vector<float *> params_, grads_, m_ptrs_, v_ptrs_;
  std::vector<int> sizes_;
  std::vector<DeviceBuffer<float>> m_, v_;
};

class SGDOptimizer : public DlbOptimizerBase {
public:
  SGDOptimizer() : DlbOptimizerBase(0) {}
  void step(float lr) override { run(DLB_OPT_SGD, lr, 0.f, 0.f, 0.f, 0.f, 1.f, 1.f); }
};

class AdamOptimizer : public DlbOptimizerBase {
public:
  AdamOptimizer(float beta1 = 0.9f, float beta2 = 0.999f, float epsilon = 1e-8f)
      : DlbOptimizerBase(2), beta1_(beta1), beta2_(beta2), epsilon_(epsilon) {}
  void step(float lr) override {
    t_++;
    const float inv1 = 1.0f / (1.0f - powf(beta1_, static_cast<float>(t_)));
    const float inv2 = 1.0f / (1.0f - powf(beta2_, static_cast<float>(t_)));
    run(DLB_OPT_ADAM, lr, beta1_, beta2_, epsilon_, 0.f, inv1, inv2);
  }

private:
  float beta1_, beta2_, epsilon_;
};

class AdamWOptimizer : public DlbOptimizerBase {
public:
  AdamWOptimizer(float beta1 = 0.9f, float beta2 = 0.999f, float epsilon = 1e-8f, float weight_decay = 0.01f)
      : DlbOptimizerBase(2), beta1_(beta1), beta2_(beta2), epsilon_(epsilon), weight_decay_(weight_decay) {}
  void step(float lr) override {
    t_++;
    const float inv1 = 1.0f / (1.0f - powf(beta1_, static_cast<float>(t_)));
    const float inv2 = 1.0f / (1.0f - powf(beta2_, static_cast<float>(t_)));
    run(DLB_OPT_ADAMW, lr, beta1_, beta2_, epsilon_, weight_decay_, inv1, inv2);
  }

private:
  float beta1_, beta2_, epsilon_, weight_decay_;
};

class RMSpropOptimizer : public DlbOptimizerBase {
public:
  RMSpropOptimizer(float decay_rate = 0.9f, float epsilon = 1e-8f)
      : DlbOptimizerBase(1), decay_rate_(decay_rate), epsilon_(epsilon) {}
  void step(float lr) override { run(DLB_OPT_RMSPROP, lr, decay_rate_, 0.f, epsilon_, 0.f, 1.f, 1.f); }

private:
  float decay_rate_, epsilon_;
};

inline void Sequential::set_optimizer(Optimizer *opt) {
  optimizer_ = opt;
  optimizer_->register_params(all_groups());
}

inline void Sequential::update_weights(float lr) {
  if (optimizer_) {
    optimizer_->step(lr);
    return;
  }
  for (Operation *op : ops_) op->update_weights(lr);
}

// Returns the global gradient norm; gradients are scaled in place when it exceeds max_norm.
inline float Sequential::clip_grad_norm(float max_norm) {
  std::vector<ParamGroup> groups = all_groups();
  if (groups.empty()) return 0.0f;
  std::vector<float *> grads;
  std::vector<int> sizes;
  for (const ParamGroup &g : groups) {
    grads.push_back(g.grads);
    sizes.push_back(g.size);
  }
  DeviceBuffer<unsigned char> ws(dlb_grad_norm_workspace_bytes());
  DeviceBuffer<float> result(3);
  DLB_CHECK(dlb_grad_norm_clip(static_cast<int>(grads.size()), grads.data(), sizes.data(), max_norm, ws.get(),
                               ws.count(), result.get(), nullptr));
  float norm = 0.0f;
  CUDA_CHECK(cudaMemcpy(&norm, result.get() + 1, sizeof(float), cudaMemcpyDeviceToHost));
  dlb_require_no_pipeline_timeouts("clip_grad_norm");
  return norm;
}
