// Learning-rate schedules with the interface of dl-cuda's src/scheduler.cuh:
// host-only float arithmetic, evaluated once per step.  The expressions keep
// the reference's operation order so that the rates agree to the last bit.
#pragma once

#include <cmath>

class LRScheduler {
public:
  virtual ~LRScheduler() = default;
  virtual float get_lr(int step) = 0;
};

// lr_min + (lr_max - lr_min) * (1 + cos(pi * step / t_max)) / 2, lr_min from t_max on.
class CosineAnnealingScheduler : public LRScheduler {
public:
  CosineAnnealingScheduler(float lr_max, float lr_min, int t_max)
      : hi_(lr_max), lo_(lr_min), period_(t_max) {}

  float get_lr(int step) override {
    if (step >= period_) return lo_;
    const float phase = static_cast<float>(M_PI) * step / period_;
    return lo_ + 0.5f * (hi_ - lo_) * (1.0f + cosf(phase));
  }

private:
  float hi_, lo_;
  int period_;
};

// initial_lr * gamma^(step / step_size), integer division.
class StepDecayScheduler : public LRScheduler {
public:
  StepDecayScheduler(float initial_lr, float gamma, int step_size)
      : base_(initial_lr), factor_(gamma), every_(step_size) {}

  float get_lr(int step) override {
    return base_ * powf(factor_, static_cast<float>(step / every_));
  }

private:
  float base_, factor_;
  int every_;
};

// Linear ramp to target_lr over warmup_steps, then the wrapped schedule (with
// its step counted from the end of the ramp) or the constant target.
class WarmupScheduler : public LRScheduler {
public:
  WarmupScheduler(float target_lr, int warmup_steps, LRScheduler *after_warmup = nullptr)
      : target_(target_lr), ramp_(warmup_steps), next_(after_warmup) {}

  float get_lr(int step) override {
    if (step < ramp_) return target_ * (static_cast<float>(step + 1) / ramp_);
    return next_ ? next_->get_lr(step - ramp_) : target_;
  }

private:
  float target_;
  int ramp_;
  LRScheduler *next_;
};
