// TEST INFRASTRUCTURE.  Small models written against dl-cuda's layer API only
// (Operation, Sequential, EmbeddingLayer, PositionalEncoding, TransformerStack,
// LinearLayer, SoftmaxActivation, the loss helpers, AdamWOptimizer, the
// schedulers), exported as plain C functions over HOST arrays.
//
// This one source is compiled twice, unchanged:
//   * against the headers of this repository (dl_cuda_b200/src)  -> the code under test;
//   * against the reference's own headers                          -> the checker.
// That it compiles against both is the API drop-in claim; that both give the
// same numbers is what the tests around it assert.
#include <cstdint>
#include <cstring>
#include <vector>

#include "activation.cuh"
#include "embedding.cuh"
#include "layers.cuh"
#include "loss.cuh"
#include "optimizer.cuh"
#include "positional_encoding.cuh"
#include "sampling.cuh"
#include "scheduler.cuh"
#include "sequential.cuh"
#include "transformer.cuh"

#define LM_API extern "C" __attribute__((visibility("default")))

namespace {

struct DeviceArray {
  float *ptr = nullptr;
  explicit DeviceArray(size_t n) { CUDA_CHECK(cudaMalloc(&ptr, (n ? n : 1) * sizeof(float))); }
  ~DeviceArray() { cudaFree(ptr); }
  void put(const float *h, size_t n) { CUDA_CHECK(cudaMemcpy(ptr, h, n * sizeof(float), cudaMemcpyHostToDevice)); }
  void get(float *h, size_t n) const { CUDA_CHECK(cudaMemcpy(h, ptr, n * sizeof(float), cudaMemcpyDeviceToHost)); }
};

int total_size(const std::vector<ParamGroup> &groups) {
  int n = 0;
  for (const ParamGroup &g : groups) n += g.size;
  return n;
}

void download_groups(const std::vector<ParamGroup> &groups, float *h_params, float *h_grads) {
  size_t at = 0;
  for (const ParamGroup &g : groups) {
    if (h_params) CUDA_CHECK(cudaMemcpy(h_params + at, g.params, g.size * sizeof(float), cudaMemcpyDeviceToHost));
    if (h_grads) CUDA_CHECK(cudaMemcpy(h_grads + at, g.grads, g.size * sizeof(float), cudaMemcpyDeviceToHost));
    at += g.size;
  }
}

void upload_params(const std::vector<ParamGroup> &groups, const float *h_params) {
  size_t at = 0;
  for (const ParamGroup &g : groups) {
    CUDA_CHECK(cudaMemcpy(g.params, h_params + at, g.size * sizeof(float), cudaMemcpyHostToDevice));
    at += g.size;
  }
}

}  // namespace

// Forward + backward of a TransformerStack on x, dy [B*S*D].  Returns the number
// of parameter floats over all groups (in get_param_groups() order); fills
// h_params / h_grads when capacity allows.
LM_API int lm_transformer_run(int layers, int B, int S, int D, int H, int F, int causal, const float *h_x,
                              const float *h_dy, float *h_y, float *h_dx, float *h_params, float *h_grads,
                              int capacity) {
  TransformerStack stack(layers, B, S, D, H, 0.0f, F, causal != 0);
  const size_t n = static_cast<size_t>(B) * S * D;
  DeviceArray x(n), y(n), dy(n), dx(n);
  x.put(h_x, n);
  dy.put(h_dy, n);
  stack.forward(x.ptr, y.ptr);
  y.get(h_y, n);
  stack.backward(dy.ptr, dx.ptr);
  dx.get(h_dx, n);
  const std::vector<ParamGroup> groups = stack.get_param_groups();
  const int total = total_size(groups);
  if (total <= capacity) download_groups(groups, h_params, h_grads);
  return total;
}

// LinearLayer with given weights [in*out] and bias [out]: y, dx, dW, db.
LM_API int lm_linear_run(int n, int in, int out, const float *h_w, const float *h_b, const float *h_x,
                         const float *h_dy, float *h_y, float *h_dx, float *h_dw, float *h_db) {
  LinearLayer layer(n, in, out);
  CUDA_CHECK(cudaMemcpy(layer.get_weights(), h_w, sizeof(float) * in * out, cudaMemcpyHostToDevice));
  CUDA_CHECK(cudaMemcpy(layer.get_bias(), h_b, sizeof(float) * out, cudaMemcpyHostToDevice));
  DeviceArray x(static_cast<size_t>(n) * in), y(static_cast<size_t>(n) * out), dy(static_cast<size_t>(n) * out),
      dx(static_cast<size_t>(n) * in);
  x.put(h_x, static_cast<size_t>(n) * in);
  dy.put(h_dy, static_cast<size_t>(n) * out);
  layer.forward(x.ptr, y.ptr);
  y.get(h_y, static_cast<size_t>(n) * out);
  layer.backward(dy.ptr, dx.ptr);
  dx.get(h_dx, static_cast<size_t>(n) * in);
  CUDA_CHECK(cudaMemcpy(h_dw, layer.get_weight_grad(), sizeof(float) * in * out, cudaMemcpyDeviceToHost));
  CUDA_CHECK(cudaMemcpy(h_db, layer.get_bias_grad(), sizeof(float) * out, cudaMemcpyDeviceToHost));
  return 0;
}

// SoftmaxActivation forward + backward over [rows, width].
LM_API int lm_softmax_run(int rows, int width, const float *h_x, const float *h_dy, float *h_y, float *h_dx) {
  SoftmaxActivation layer(rows, width);
  const size_t n = static_cast<size_t>(rows) * width;
  DeviceArray x(n), y(n), dy(n), dx(n);
  x.put(h_x, n);
  dy.put(h_dy, n);
  layer.forward(x.ptr, y.ptr);
  y.get(h_y, n);
  layer.backward(dy.ptr, dx.ptr);
  dx.get(h_dx, n);
  return 0;
}

// computeLoss / computeLossBackward for one LossType (0..3 in the enum's order).
LM_API int lm_loss_run(int loss_type, int n, int classes, const float *h_y, const float *h_pred, float *h_error,
                       float *h_grad) {
  const size_t width = loss_type == CATEGORICAL_CROSS_ENTROPY ? classes : 1;
  DeviceArray y(n * width), pred(n * width), err(n), grad(n * width);
  y.put(h_y, n * width);
  pred.put(h_pred, n * width);
  computeLoss(y.ptr, pred.ptr, err.ptr, n, classes, static_cast<LossType>(loss_type), dim3((n + 255) / 256),
              dim3(256));
  computeLossBackward(y.ptr, pred.ptr, grad.ptr, n, classes, static_cast<LossType>(loss_type));
  err.get(h_error, n);
  grad.get(h_grad, n * width);
  return 0;
}

// Cross entropy against integer targets, forward and backward.
LM_API int lm_ce_ids_run(int n, int classes, const int *h_target, const float *h_pred, float *h_error,
                         float *h_grad) {
  const size_t total = static_cast<size_t>(n) * classes;
  DeviceArray pred(total), err(n), grad(total);
  int *d_target = nullptr;
  CUDA_CHECK(cudaMalloc(&d_target, sizeof(int) * (n ? n : 1)));
  CUDA_CHECK(cudaMemcpy(d_target, h_target, sizeof(int) * n, cudaMemcpyHostToDevice));
  pred.put(h_pred, total);
  computeCategoricalCrossEntropyFromIds(d_target, pred.ptr, err.ptr, n, classes);
  computeCategoricalCrossEntropyBackwardFromIds(d_target, pred.ptr, grad.ptr, n, classes);
  err.get(h_error, n);
  grad.get(h_grad, total);
  cudaFree(d_target);
  return 0;
}

// Learning-rate schedule of the char-LM example: warm-up into cosine annealing.
LM_API void lm_schedule(float lr_max, float lr_min, int warmup, int epochs, float *h_lr) {
  CosineAnnealingScheduler cosine(lr_max, lr_min, epochs);
  WarmupScheduler schedule(lr_max, warmup, &cosine);
  for (int e = 0; e < epochs; e++) h_lr[e] = schedule.get_lr(e);
}

// Token sampling (host only): `draws` tokens from one probability row with the given temperature,
// top-k (0 = off) and top-p (1 = off), from std::mt19937(seed).  h_filtered receives the row after
// temperature, top-k and top-p (what the draw is made from).
LM_API void lm_sample(const float *h_probs, int n, float temperature, int top_k, float top_p, unsigned seed,
                      int draws, int *h_tokens, float *h_filtered) {
  const std::vector<float> probs(h_probs, h_probs + n);
  std::mt19937 rng(seed);
  for (int i = 0; i < draws; i++) h_tokens[i] = sampleWithStrategy(probs, temperature, top_k, top_p, rng);
  std::vector<float> filtered(probs);
  if (temperature != 1.0f)
    for (float &p : filtered) p = powf(p, 1.0f / temperature);
  if (top_k > 0) applyTopK(filtered, top_k);
  if (top_p < 1.0f) applyTopP(filtered, top_p);
  std::memcpy(h_filtered, filtered.data(), sizeof(float) * n);
}

// The training loop of the reference's character language model
// (embedding -> positional encoding -> causal transformer stack -> linear ->
// softmax, cross entropy from ids, gradient clipping, AdamW, warm-up + cosine
// schedule) on caller-provided token windows: h_ids / h_targets hold `epochs`
// windows of S ids.  If load != 0 the parameters start from h_params_init,
// else h_params_init receives what the constructors drew.  Outputs the mean loss
// of every epoch and the final parameters.  Returns the parameter count.
LM_API int lm_char_lm_train(uint64_t seed, int vocab, int S, int D, int F, int H, int layers, int epochs,
                            const int *h_ids, const int *h_targets, float lr_max, float lr_min, int warmup,
                            float clip, int load, float *h_params_init, float *h_losses, float *h_params_final,
                            int capacity, const char *checkpoint_path) {
  set_global_init_seed(seed);
  EmbeddingLayer embedding(vocab, D, S);
  PositionalEncoding positions(1, S, D);
  TransformerStack blocks(layers, 1, S, D, H, 0.0f, F, true);
  LinearLayer head(S, D, vocab);
  SoftmaxActivation softmax(S, vocab);

  Sequential model;
  model.add(&embedding);
  model.add(&positions);
  model.add(&blocks);
  model.add(&head);
  model.add(&softmax);
  AdamWOptimizer adamw(0.9f, 0.999f, 1e-8f, 0.01f);
  model.set_optimizer(&adamw);

  std::vector<ParamGroup> groups = embedding.get_param_groups();
  for (Operation *op : {static_cast<Operation *>(&blocks), static_cast<Operation *>(&head)}) {
    const std::vector<ParamGroup> own = op->get_param_groups();
    groups.insert(groups.end(), own.begin(), own.end());
  }
  const int total = total_size(groups);
  if (total > capacity) return total;
  if (load) upload_params(groups, h_params_init);
  else download_groups(groups, h_params_init, nullptr);

  CosineAnnealingScheduler cosine(lr_max, lr_min, epochs);
  WarmupScheduler schedule(lr_max, warmup, &cosine);

  const size_t out_total = static_cast<size_t>(S) * vocab;
  DeviceArray pred(out_total), loss_grad(out_total), error(S), input_grad(S), dummy(S);
  int *d_targets = nullptr;
  CUDA_CHECK(cudaMalloc(&d_targets, sizeof(int) * S));
  std::vector<float> h_error(S);

  for (int epoch = 0; epoch < epochs; epoch++) {
    embedding.set_token_ids(h_ids + static_cast<size_t>(epoch) * S);
    CUDA_CHECK(cudaMemcpy(d_targets, h_targets + static_cast<size_t>(epoch) * S, sizeof(int) * S,
                          cudaMemcpyHostToDevice));
    model.forward(dummy.ptr, pred.ptr);
    computeCategoricalCrossEntropyFromIds(d_targets, pred.ptr, error.ptr, S, vocab);
    error.get(h_error.data(), S);
    float mean = 0.0f;
    for (float e : h_error) mean += e;
    h_losses[epoch] = mean / S;

    computeCategoricalCrossEntropyBackwardFromIds(d_targets, pred.ptr, loss_grad.ptr, S, vocab);
    model.backward(loss_grad.ptr, input_grad.ptr);
    model.clip_grad_norm(clip);
    model.update_weights(schedule.get_lr(epoch));
  }
  CUDA_CHECK(cudaDeviceSynchronize());
  download_groups(groups, h_params_final, nullptr);
  cudaFree(d_targets);
  if (checkpoint_path && checkpoint_path[0] && !model.save_weights(checkpoint_path)) return -1;
  return total;
}
