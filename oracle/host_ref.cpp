// TEST INFRASTRUCTURE -- NOT PART OF THE PRODUCT.
//
// CPU restatement of the arithmetic of dl-cuda's layer kernels, one row (or one
// element) at a time on a single host thread, in the reference's own summation
// order.  It exists to check the CUDA kernels in tests/, in
// __graft_entry__.smoke() and as the timed host baseline of bench.py; nothing
// in the shipped library may call it.
//
// The reference has no CPU implementation: every function below follows a CUDA
// kernel of the reference, cited as path:lines inside that project.  nvcc
// compiles those kernels with its default -fmad=true, i.e. `a*b + c` becomes
// one fused multiply-add; the places where that happens are written with
// fmaf() here so that the host result carries the same rounding.  Division,
// sqrtf and the fp32 adds are IEEE on both sides.  expf/tanhf come from the
// host C library here and from CUDA's math library on the GPU: those two may
// differ by a few units in the last place, everything else is bit-for-bit.
//
// Parity pin: the embedding known-answer test of the reference
// (tests/gpu_correctness_tests.cu:196-252) and fixtures written by the
// reference's own kernels (tests/golden/) are checked against this file by
// tests/test_oracle_golden.py.
//
// Build: g++ -O2 -std=c++17 -shared -fPIC (no -ffast-math, no -march flags: the
// compiler must not contract or reassociate anything by itself).
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

extern "C" {

// transformerResidualAddKernel, src/transformer.cuh:216-222 (also
// addVectorsKernel, src/layers.cuh:256-262): out[i] = a[i] + b[i].
void orc_residual_add(const float *a, const float *b, float *out, int64_t n) {
  for (int64_t i = 0; i < n; i++) out[i] = a[i] + b[i];
}

// Residual add (src/transformer.cuh:499-502) followed by
// layerNormForwardCachingKernel (src/transformer.cuh:136-164): the sum is
// rounded to float first (the reference stores it in residual_buf), then mean,
// biased two-pass variance, inv_std, xhat and y, all accumulated left to right.
void orc_ln_residual_fwd(const float *a, const float *b, const float *gamma, const float *beta,
                         float *y, float *xhat, float *inv_std, int rows, int d, float eps) {
  std::vector<float> s(static_cast<size_t>(d));
  for (int r = 0; r < rows; r++) {
    const size_t base = static_cast<size_t>(r) * d;
    for (int j = 0; j < d; j++) s[j] = b ? a[base + j] + b[base + j] : a[base + j];
    float mean = 0.0f;
    for (int j = 0; j < d; j++) mean += s[j];
    mean /= d;
    float var = 0.0f;
    for (int j = 0; j < d; j++) {
      const float diff = s[j] - mean;
      var = fmaf(diff, diff, var);
    }
    var /= d;
    const float is = 1.0f / sqrtf(var + eps);
    if (inv_std) inv_std[r] = is;
    for (int j = 0; j < d; j++) {
      const float xh = (s[j] - mean) * is;
      if (xhat) xhat[base + j] = xh;
      y[base + j] = fmaf(gamma[j], xh, beta[j]);
    }
  }
}

// Gradient residual add (src/transformer.cuh:583-585) followed by
// layerNormBackwardKernel (src/transformer.cuh:166-190).
void orc_ln_bwd_dx(const float *dy_a, const float *dy_b, const float *xhat, const float *inv_std,
                   const float *gamma, float *dx, int rows, int d) {
  std::vector<float> g(static_cast<size_t>(d));
  for (int r = 0; r < rows; r++) {
    const size_t base = static_cast<size_t>(r) * d;
    const float is = inv_std[r];
    float c1 = 0.0f, c2 = 0.0f;
    for (int j = 0; j < d; j++) {
      const float dy = dy_b ? dy_a[base + j] + dy_b[base + j] : dy_a[base + j];
      const float dxh = dy * gamma[j];
      g[j] = dxh;
      c1 += dxh;
      c2 = fmaf(dxh, xhat[base + j], c2);
    }
    c1 /= d;
    c2 /= d;
    for (int j = 0; j < d; j++) dx[base + j] = fmaf(-xhat[base + j], c2, g[j] - c1) * is;
  }
}

// layerNormParamGradKernel (src/transformer.cuh:192-207): per column, rows
// added top to bottom in fp32.
void orc_ln_param_grad(const float *dy_a, const float *dy_b, const float *xhat, float *dgamma,
                       float *dbeta, int rows, int d) {
  for (int j = 0; j < d; j++) {
    float dg = 0.0f, db = 0.0f;
    for (int r = 0; r < rows; r++) {
      const size_t i = static_cast<size_t>(r) * d + j;
      const float dy = dy_b ? dy_a[i] + dy_b[i] : dy_a[i];
      dg = fmaf(dy, xhat[i], dg);
      db += dy;
    }
    dgamma[j] = dg;
    dbeta[j] = db;
  }
}

// The same sums carried in double: the value both fp32 summation orders (the
// reference's top-to-bottom loop and the GPU's tree) approximate.
void orc_ln_param_grad_f64(const float *dy_a, const float *dy_b, const float *xhat, double *dgamma,
                           double *dbeta, int rows, int d) {
  for (int j = 0; j < d; j++) {
    double dg = 0.0, db = 0.0;
    for (int r = 0; r < rows; r++) {
      const size_t i = static_cast<size_t>(r) * d + j;
      const float dy = dy_b ? dy_a[i] + dy_b[i] : dy_a[i];
      dg += static_cast<double>(dy) * static_cast<double>(xhat[i]);
      db += static_cast<double>(dy);
    }
    dgamma[j] = dg;
    dbeta[j] = db;
  }
}

// PositionalEncoding's constructor, src/positional_encoding.cuh:33-41.
void orc_pe_table(float *table, int seq_len, int d) {
  for (int pos = 0; pos < seq_len; pos++)
    for (int i = 0; i < d; i++) {
      const float angle =
          static_cast<float>(pos) / powf(10000.0f, static_cast<float>(2 * (i / 2)) / d);
      table[static_cast<size_t>(pos) * d + i] = (i % 2 == 0) ? sinf(angle) : cosf(angle);
    }
}

// addPositionalEncodingKernel, src/positional_encoding.cuh:7-17.
void orc_pe_add(const float *in, const float *pe, float *out, int batch, int seq_len, int d) {
  const int64_t period = static_cast<int64_t>(seq_len) * d;
  const int64_t total = period * batch;
  for (int64_t i = 0; i < total; i++) out[i] = in[i] + pe[i % period];
}

// embeddingForwardKernel (src/embedding.cuh:8-17), optionally followed by
// addPositionalEncodingKernel (src/positional_encoding.cuh:7-17).
void orc_embed_gather(const float *table, const int32_t *ids, const float *pe, int seq_len,
                      float *out, int num_tokens, int d) {
  for (int t = 0; t < num_tokens; t++) {
    const float *src = table + static_cast<size_t>(ids[t]) * d;
    float *dst = out + static_cast<size_t>(t) * d;
    if (pe) {
      const float *p = pe + static_cast<size_t>(t % seq_len) * d;
      for (int j = 0; j < d; j++) dst[j] = src[j] + p[j];
    } else {
      std::memcpy(dst, src, sizeof(float) * d);
    }
  }
}

// cudaMemset + embeddingBackwardKernel (src/embedding.cuh:19-30, 82-92).  The
// reference adds with atomicAdd in whatever order the hardware picks; here the
// tokens of a row are added in ascending token order.
void orc_embed_scatter(const float *dy, const int32_t *ids, float *grad, int num_tokens, int vocab,
                       int d) {
  std::memset(grad, 0, sizeof(float) * static_cast<size_t>(vocab) * d);
  for (int t = 0; t < num_tokens; t++) {
    float *dst = grad + static_cast<size_t>(ids[t]) * d;
    const float *src = dy + static_cast<size_t>(t) * d;
    for (int j = 0; j < d; j++) dst[j] += src[j];
  }
}

// The same sum in the association the CUDA kernel fixes: the tokens of a row in
// ascending order; a row with more than `sub_len` tokens is cut into pieces of
// sub_len tokens, each summed from 0.0f; the piece sums are added in order inside
// `slices` contiguous groups of pieces, and the group sums are added in order.
void orc_embed_scatter_segmented(const float *dy, const int32_t *ids, float *grad, int num_tokens,
                                 int vocab, int d, int sub_len, int slices) {
  std::vector<std::vector<int>> rows(static_cast<size_t>(vocab));
  for (int t = 0; t < num_tokens; t++) rows[ids[t]].push_back(t);
  std::vector<float> part(static_cast<size_t>(d)), group(static_cast<size_t>(d));
  for (int v = 0; v < vocab; v++) {
    float *dst = grad + static_cast<size_t>(v) * d;
    for (int j = 0; j < d; j++) dst[j] = 0.0f;
    const std::vector<int> &tok = rows[v];
    const int n = static_cast<int>(tok.size());
    if (n <= sub_len) {
      for (int k = 0; k < n; k++)
        for (int j = 0; j < d; j++) dst[j] += dy[static_cast<size_t>(tok[k]) * d + j];
      continue;
    }
    const int pieces = (n + sub_len - 1) / sub_len;
    const int per = (pieces + slices - 1) / slices;
    for (int q = 0; q < slices; q++) {
      for (int j = 0; j < d; j++) group[j] = 0.0f;
      for (int piece = q * per; piece < pieces && piece < (q + 1) * per; piece++) {
        for (int j = 0; j < d; j++) part[j] = 0.0f;
        for (int k = piece * sub_len; k < n && k < (piece + 1) * sub_len; k++)
          for (int j = 0; j < d; j++) part[j] += dy[static_cast<size_t>(tok[k]) * d + j];
        for (int j = 0; j < d; j++) group[j] += part[j];
      }
      if (q == 0)
        for (int j = 0; j < d; j++) dst[j] = group[j];
      else
        for (int j = 0; j < d; j++) dst[j] += group[j];
    }
  }
}

void orc_embed_scatter_f64(const float *dy, const int32_t *ids, double *grad, int num_tokens,
                           int vocab, int d) {
  for (size_t i = 0; i < static_cast<size_t>(vocab) * d; i++) grad[i] = 0.0;
  for (int t = 0; t < num_tokens; t++)
    for (int j = 0; j < d; j++)
      grad[static_cast<size_t>(ids[t]) * d + j] += static_cast<double>(dy[static_cast<size_t>(t) * d + j]);
}

// Bias add at the end of linearLayerKernel (src/layers.cuh:34) followed by
// reluKernel / sigmoidKernel / tanhActivationKernel / geluForwardKernel
// (src/activation.cuh:5-10, 22-27, 39-45, 203-210).  kind: 0 relu, 1 sigmoid,
// 2 tanh, 3 gelu.  `pre` (optional) receives x + bias.
void orc_act_fwd(int kind, const float *x, const float *bias, float *y, float *pre_out, int64_t rows,
                 int64_t cols) {
  for (int64_t r = 0; r < rows; r++)
    for (int64_t c = 0; c < cols; c++) {
      const int64_t i = r * cols + c;
      const float pre = bias ? x[i] + bias[c] : x[i];
      if (pre_out) pre_out[i] = pre;
      float out;
      switch (kind) {
        case 0: out = (pre > 0.0f) ? pre : 0.0f; break;
        case 1: out = 1.0f / (1.0f + expf(-pre)); break;
        case 2: out = tanhf(pre); break;
        default: {
          // 0.044715f * x * x * x is ((0.044715f*x)*x)*x; the outer add fuses with
          // the last product.
          const float inner = 0.7978845608f * fmaf(0.044715f * pre * pre, pre, pre);
          const float cdf = 0.5f * (1.0f + tanhf(inner));
          out = pre * cdf;
        }
      }
      y[i] = out;
    }
}

// reluBackwardKernel / sigmoidBackwardKernel / tanhBackwardKernel /
// geluBackwardKernel (src/activation.cuh:12-20, 29-37, 47-55, 212-226;
// tanhBackwardElementKernel, src/layers.cuh:247-254).  `cache` is what the
// reference layer cached: the forward INPUT for relu and gelu, the forward
// OUTPUT for sigmoid and tanh.
void orc_act_bwd(int kind, const float *dy, const float *cache, float *dx, int64_t n) {
  for (int64_t i = 0; i < n; i++) {
    const float c = cache[i];
    float out;
    switch (kind) {
      case 0: out = dy[i] * ((c > 0.0f) ? 1.0f : 0.0f); break;
      case 1: out = dy[i] * c * (1.0f - c); break;
      case 2: out = dy[i] * fmaf(-c, c, 1.0f); break;
      default: {
        const float x = c;
        const float x3 = x * x * x;
        const float inner = 0.7978845608f * fmaf(0.044715f, x3, x);
        const float tanh_val = tanhf(inner);
        const float sech2 = fmaf(-tanh_val, tanh_val, 1.0f);
        const float d_inner = 0.7978845608f * fmaf(0.134145f * x, x, 1.0f);
        const float cdf = 0.5f * (1.0f + tanh_val);
        out = dy[i] * fmaf(x * 0.5f * sech2, d_inner, cdf);
      }
    }
    dx[i] = out;
  }
}

// linearBackwardBiasKernel, src/layers.cuh:70-82: per column, rows top to bottom.
void orc_bias_grad(const float *dy, float *dbias, int64_t rows, int64_t cols) {
  for (int64_t c = 0; c < cols; c++) {
    float sum = 0.0f;
    for (int64_t r = 0; r < rows; r++) sum += dy[r * cols + c];
    dbias[c] = sum;
  }
}

void orc_bias_grad_f64(const float *dy, double *dbias, int64_t rows, int64_t cols) {
  for (int64_t c = 0; c < cols; c++) {
    double sum = 0.0;
    for (int64_t r = 0; r < rows; r++) sum += static_cast<double>(dy[r * cols + c]);
    dbias[c] = sum;
  }
}

// sgdUpdateKernel, src/layers.cuh:84-90: p -= lr*g (one fused multiply-add).
void orc_sgd_update(float *p, const float *g, float lr, int64_t n) {
  for (int64_t i = 0; i < n; i++) p[i] = fmaf(-lr, g[i], p[i]);
}

}  // extern "C"

extern "C" {

// updateAdam / updateAdamW (src/optimizers.cuh:16-48), updateRMSprop (:6-14): one element at a
// time, in place.  kind: 1 adam, 2 adamw, 3 rmsprop (state in m, decay in beta1).  The products
// that nvcc may or may not fuse are left to the compiler here; tests compare within 1e-6.
void orc_optim_step(int kind, float *p, const float *g, float *m, float *v, int64_t n, float lr, float beta1,
                    float beta2, float eps, float weight_decay, float inv_bc1, float inv_bc2) {
  for (int64_t i = 0; i < n; i++) {
    if (kind == 3) {
      m[i] = beta1 * m[i] + (1 - beta1) * g[i] * g[i];
      p[i] -= lr * g[i] / (sqrtf(m[i]) + eps);
      continue;
    }
    m[i] = beta1 * m[i] + (1.0f - beta1) * g[i];
    v[i] = beta2 * v[i] + (1.0f - beta2) * g[i] * g[i];
    const float m_hat = m[i] * inv_bc1;
    const float v_hat = v[i] * inv_bc2;
    if (kind == 1)
      p[i] -= lr * m_hat / (sqrtf(v_hat) + eps);
    else
      p[i] -= lr * (m_hat / (sqrtf(v_hat) + eps) + weight_decay * p[i]);
  }
}

// Sum of squares as Sequential::clip_grad_norm forms it (src/optimizer.cuh:213-221), in double.
double orc_sq_norm_f64(const float *g, int64_t n) {
  double s = 0.0;
  for (int64_t i = 0; i < n; i++) s += static_cast<double>(g[i]) * static_cast<double>(g[i]);
  return s;
}

}  // extern "C"

extern "C" {

// The reference's matrix products all have one shape per output element: a sum
// over k in ascending order that nvcc contracts into one fused multiply-add per
// step, starting from 0.0f (linearLayerKernel src/layers.cuh:23-36,
// linearBackwardInputKernel :38-52, linearBackwardWeightKernel :54-68,
// attnScoresKernel / attnApplyKernel / matMulBTKernel / matMulATKernel
// src/transformer.cuh:8-19, 47-58, 84-108).  Strides select the variant:
//   A(i,kk) = a[i*a_row + kk*a_col],  B(kk,j) = b[kk*b_row + j*b_col].
// Then sum*alpha (attnScoresKernel's inv_scale), + bias[j] (linearLayerKernel),
// and optionally c += (transformerResidualAddKernel after the Q/K/V input
// gradients, src/transformer.cuh:663-677).
void orc_gemm(const float *a, const float *b, const float *bias, float *c, int m, int n, int k, int64_t a_row,
              int64_t a_col, int64_t b_row, int64_t b_col, int64_t ldc, float alpha, int accumulate) {
  for (int i = 0; i < m; i++)
    for (int j = 0; j < n; j++) {
      float sum = 0.0f;
      for (int kk = 0; kk < k; kk++) sum = fmaf(a[i * a_row + kk * a_col], b[kk * b_row + j * b_col], sum);
      float v = sum * alpha;
      if (bias) v = v + bias[j];
      if (accumulate) v = c[i * ldc + j] + v;
      c[i * ldc + j] = v;
    }
}

// applyCausalMaskKernel + softmaxForwardKernel (src/transformer.cuh:21-45) and
// softmaxForwardGeneralKernel (src/activation.cuh:121-143): row max, expf, sequential sum,
// multiply by 1/sum.  causal_period > 0 overwrites entries past (row % period) with -1e9f first.
void orc_softmax_fwd(const float *in, float *out, int64_t rows, int width, int causal_period) {
  std::vector<float> row(width);
  for (int64_t r = 0; r < rows; r++) {
    for (int j = 0; j < width; j++) {
      row[j] = in[r * width + j];
      if (causal_period > 0 && j > r % causal_period) row[j] = -1e9f;
    }
    float mx = row[0];
    for (int j = 1; j < width; j++) mx = fmaxf(mx, row[j]);
    float sum = 0.0f;
    for (int j = 0; j < width; j++) {
      row[j] = expf(row[j] - mx);
      sum += row[j];
    }
    const float inv = 1.0f / sum;
    for (int j = 0; j < width; j++) out[r * width + j] = row[j] * inv;
  }
}

// softmaxBackwardKernel + scaleBufferKernel (src/transformer.cuh:60-82, 209-214),
// softmaxBackwardGeneralKernel (src/activation.cuh:145-165) with scale = 1.
void orc_softmax_bwd(const float *dy, const float *s, float *dx, int64_t rows, int width, float scale) {
  for (int64_t r = 0; r < rows; r++) {
    const float *g = dy + r * width, *p = s + r * width;
    float dot = 0.0f;
    for (int j = 0; j < width; j++) dot = fmaf(g[j], p[j], dot);
    for (int j = 0; j < width; j++) dx[r * width + j] = (p[j] * (g[j] - dot)) * scale;
  }
}

static float orc_clamp_prob(float p) {
  const float eps = 1e-10f;
  if (p < eps) return eps;
  if (p > 1.0f - eps) return 1.0f - eps;
  return p;
}

// src/loss.cuh:18-109.  kind 0 squared, 1 absolute, 2 binary CE, 3 categorical CE.
void orc_loss(int kind, const float *y, const float *yp, float *err, float *grad, int64_t n, int classes) {
  const float eps = 1e-10f;
  const float fn = static_cast<float>(n);
  for (int64_t i = 0; i < n; i++) {
    if (kind == 0) {
      const float diff = y[i] - yp[i];
      err[i] = diff * diff;
      grad[i] = 2.0f * (yp[i] - y[i]) / fn;
    } else if (kind == 1) {
      err[i] = fabsf(y[i] - yp[i]);
      const float diff = yp[i] - y[i];
      grad[i] = ((diff > 0.0f) ? 1.0f : ((diff < 0.0f) ? -1.0f : 0.0f)) / fn;
    } else if (kind == 2) {
      const float p = orc_clamp_prob(yp[i]);
      err[i] = -y[i] * logf(p) - (1.0f - y[i]) * logf(1.0f - p);
      grad[i] = (-y[i] / p + (1.0f - y[i]) / (1.0f - p)) / fn;
    } else {
      float loss = 0.0f;
      for (int c = 0; c < classes; c++) {
        const int64_t at = i * classes + c;
        loss -= y[at] * logf(yp[at] + eps);
        grad[at] = -y[at] / (yp[at] + eps) / fn;
      }
      err[i] = loss;
    }
  }
}

// categoricalCrossEntropyFromIdsKernel / ...BackwardFromIdsKernel, src/loss.cuh:111-144.
void orc_ce_from_ids(const int32_t *target, const float *yp, float *err, float *grad, int n, int classes,
                     float eps) {
  for (int i = 0; i < n; i++) {
    for (int c = 0; c < classes; c++) grad[static_cast<int64_t>(i) * classes + c] = 0.0f;
    float p = yp[static_cast<int64_t>(i) * classes + target[i]];
    if (p < eps) p = eps;
    err[i] = -logf(p);
    grad[static_cast<int64_t>(i) * classes + target[i]] = -1.0f / (p * static_cast<float>(n));
  }
}

}  // extern "C"
