// Token sampling helpers with the interface of dl-cuda's src/sampling.cuh: all
// host-side work on one probability row (a few dozen to a few thousand floats
// that the caller has already copied back), so there is nothing here for the
// GPU.  The random draws consume the generator exactly as the reference does
// (one uniform_real_distribution<float>(0, sum) draw per sample), which keeps
// generated text identical for identical probabilities.
#pragma once

#include <algorithm>
#include <cmath>
#include <numeric>
#include <random>
#include <vector>

#include "sequential.cuh"

// Inverse-CDF draw over unnormalised weights.
inline int sampleFromProbs(const std::vector<float> &probs, std::mt19937 &rng) {
  float total = 0.0f;
  for (size_t i = 0; i < probs.size(); i++) total += probs[i];
  std::uniform_real_distribution<float> pick(0.0f, total);
  const float threshold = pick(rng);
  float running = 0.0f;
  const int n = static_cast<int>(probs.size());
  for (int i = 0; i < n; i++) {
    running += probs[i];
    if (threshold < running) return i;
  }
  return n - 1;
}

// Descending order of the entries of probs, as indices (first `head` sorted when head < n).
inline std::vector<int> dlb_rank_desc(const std::vector<float> &probs, int head) {
  std::vector<int> order(probs.size());
  std::iota(order.begin(), order.end(), 0);
  auto larger = [&probs](int a, int b) { return probs[a] > probs[b]; };
  if (head < static_cast<int>(order.size()))
    std::partial_sort(order.begin(), order.begin() + head, order.end(), larger);
  else
    std::sort(order.begin(), order.end(), larger);
  return order;
}

// Zeroes everything but the k largest entries.
inline void applyTopK(std::vector<float> &probs, int k) {
  const int n = static_cast<int>(probs.size());
  if (k >= n) return;
  const std::vector<int> order = dlb_rank_desc(probs, k);
  for (int i = k; i < n; i++) probs[order[i]] = 0.0f;
}

// Keeps the shortest prefix of the descending order whose mass reaches p.
inline void applyTopP(std::vector<float> &probs, float p) {
  const int n = static_cast<int>(probs.size());
  const std::vector<int> order = dlb_rank_desc(probs, n);
  float mass = 0.0f;
  int keep = n;
  for (int i = 0; i < n; i++) {
    mass += probs[order[i]];
    if (mass >= p) {
      keep = i + 1;
      break;
    }
  }
  for (int i = keep; i < n; i++) probs[order[i]] = 0.0f;
}

// probs^(1/temperature), then top-k (k > 0), then top-p (p < 1), then one draw.
inline int sampleWithStrategy(const std::vector<float> &raw_probs, float temperature, int top_k, float top_p,
                              std::mt19937 &rng) {
  std::vector<float> probs(raw_probs);
  if (temperature != 1.0f) {
    const float exponent = 1.0f / temperature;
    for (size_t i = 0; i < probs.size(); i++) probs[i] = powf(probs[i], exponent);
  }
  if (top_k > 0) applyTopK(probs, top_k);
  if (top_p < 1.0f) applyTopP(probs, top_p);
  return sampleFromProbs(probs, rng);
}
