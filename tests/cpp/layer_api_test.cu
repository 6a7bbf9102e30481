// Exercises the C++ layer classes (dl_cuda_b200/src/*.cuh) the way the reference's
// own tests/gpu_correctness_tests.cu drives its classes.  Usage:
//   layer_api_test known_answer | roundtrip | chain | optimizer
//   layer_api_test checkpoint <path> <seed> <vocab> <dim> <tokens> <layers built before>
// Exit code 0 = pass.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "activation.cuh"
#include "embedding.cuh"
#include "optimizer.cuh"
#include "positional_encoding.cuh"
#include "sequential.cuh"

namespace {

std::vector<float> download(const float *d, size_t n) {
  std::vector<float> h(n);
  CUDA_CHECK(cudaMemcpy(h.data(), d, n * sizeof(float), cudaMemcpyDeviceToHost));
  return h;
}

void upload(float *d, const std::vector<float> &h) {
  CUDA_CHECK(cudaMemcpy(d, h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice));
}

bool same(const std::vector<float> &a, const std::vector<float> &b) {
  return a.size() == b.size() && memcmp(a.data(), b.data(), a.size() * sizeof(float)) == 0;
}

// The embedding known answer of the reference (tests/gpu_correctness_tests.cu:196-252):
// a 5x3 table holding 0..14, ids {1,3,1,4}, upstream gradient rows of 1,2,3,4.
int known_answer() {
  set_global_init_seed(3);
  EmbeddingLayer layer(5, 3, 4);
  ParamGroup pg = layer.get_param_groups()[0];
  std::vector<float> table(15);
  for (int i = 0; i < 15; i++) table[i] = static_cast<float>(i);
  upload(pg.params, table);
  const int ids[4] = {1, 3, 1, 4};
  layer.set_token_ids(ids);
  DeviceBuffer<float> out(12), dummy(4);
  layer.forward(nullptr, out.get());
  const std::vector<float> got = download(out.get(), 12);
  const std::vector<float> want = {3, 4, 5, 9, 10, 11, 3, 4, 5, 12, 13, 14};
  std::vector<float> dout(12);
  for (int t = 0; t < 4; t++)
    for (int j = 0; j < 3; j++) dout[t * 3 + j] = static_cast<float>(t + 1);
  upload(out.get(), dout);
  layer.backward(out.get(), dummy.get());
  const std::vector<float> grad = download(pg.grads, 15);
  std::vector<float> grad_want(15, 0.f);
  for (int j = 0; j < 3; j++) {
    grad_want[3 + j] = 4.f;
    grad_want[9 + j] = 2.f;
    grad_want[12 + j] = 4.f;
  }
  if (layer.input_size() != 4 || layer.output_size() != 12 || pg.size != 15) return 1;
  // SGD step of the layer itself: table -= lr * grad
  layer.update_weights(0.5f);
  const std::vector<float> stepped = download(pg.params, 15);
  for (int i = 0; i < 15; i++)
    if (stepped[i] != table[i] - 0.5f * grad_want[i]) return 1;
  return same(got, want) && same(grad, grad_want) ? 0 : 1;
}

// The n-th layer built in a process draws its weights from seed + 9973*n, so a process that has
// already built `built_before` layers is imitated by consuming that many seeds first.
int checkpoint(const char *path, unsigned long long seed, int vocab, int dim, int tokens, int built_before) {
  set_global_init_seed(seed);
  for (int i = 0; i < built_before; i++) (void)next_init_seed();
  EmbeddingLayer layer(vocab, dim, tokens);
  Sequential model;
  model.add(&layer);
  return model.save_weights(path) ? 0 : 1;
}

int roundtrip() {
  const std::string path = "/tmp/dlcuda_b200_roundtrip.bin";
  set_global_init_seed(4);
  EmbeddingLayer a(7, 5, 3);
  Sequential m1;
  m1.add(&a);
  if (!m1.save_weights(path)) return 1;
  EmbeddingLayer b(7, 5, 3);
  Sequential m2;
  m2.add(&b);
  if (!m2.load_weights(path)) return 1;
  const bool eq = same(download(a.get_param_groups()[0].params, 35), download(b.get_param_groups()[0].params, 35));
  EmbeddingLayer c(7, 6, 3);  // different group size: must be refused
  Sequential m3;
  m3.add(&c);
  const bool refused = !m3.load_weights(path) && !m3.load_weights("/nonexistent/dir/file.bin");
  remove(path.c_str());
  return eq && refused ? 0 : 1;
}

// Embedding -> PositionalEncoding -> Tanh through Sequential, forward and backward, against
// the same math on the host (tanhf on the host may differ by ulps: tolerance 1e-6).
int chain() {
  const int B = 2, S = 3, D = 8, V = 6, T = B * S;
  set_global_init_seed(9);
  EmbeddingLayer emb(V, D, T);
  PositionalEncoding pe(B, S, D);
  TanhActivation act(T * D);
  ReLUActivation relu(T * D);
  Sequential model;
  model.add(&emb);
  model.add(&pe);
  model.add(&act);
  model.add(&relu);
  const int ids[T] = {0, 5, 2, 2, 1, 5};
  emb.set_token_ids(ids);
  DeviceBuffer<float> out(T * D), dummy_in(T), dummy_grad(T), dout(T * D);
  model.forward(dummy_in.get(), out.get());
  const std::vector<float> table = download(emb.get_param_groups()[0].params, V * D);
  std::vector<float> pe_host(S * D);
  DLB_CHECK(dlb_pe_build_table_host(pe_host.data(), S, D));
  const std::vector<float> got = download(out.get(), T * D);
  std::vector<float> tanh_out(T * D);
  for (int t = 0; t < T; t++)
    for (int j = 0; j < D; j++) {
      const float th = tanhf(table[ids[t] * D + j] + pe_host[(t % S) * D + j]);
      tanh_out[t * D + j] = th;
      const float want = th > 0.f ? th : 0.f;
      if (fabsf(got[t * D + j] - want) > 1e-6f) return 1;
    }
  std::vector<float> g(T * D);
  for (int i = 0; i < T * D; i++) g[i] = 0.25f * static_cast<float>((i % 7) - 3);
  upload(dout.get(), g);
  model.backward(dout.get(), dummy_grad.get());
  const std::vector<float> grad = download(emb.get_param_groups()[0].grads, V * D);
  std::vector<float> want(V * D, 0.f);
  for (int t = 0; t < T; t++)
    for (int j = 0; j < D; j++) {
      const float th = tanh_out[t * D + j];
      want[ids[t] * D + j] += g[t * D + j] * (th > 0.f ? 1.f : 0.f) * (1.f - th * th);
    }
  for (int i = 0; i < V * D; i++)
    if (fabsf(grad[i] - want[i]) > 1e-5f) return 1;
  return 0;
}

// Sequential::set_optimizer / clip_grad_norm / update_weights with AdamW over two embedding layers,
// against the same arithmetic on the host (src/optimizers.cuh:32-48, src/optimizer.cuh:205-233).
int optimizer() {
  set_global_init_seed(11);
  EmbeddingLayer e1(9, 8, 4), e2(5, 16, 4);
  Sequential model;
  model.add(&e1);
  model.add(&e2);
  AdamWOptimizer opt(0.9f, 0.999f, 1e-8f, 0.01f);
  model.set_optimizer(&opt);
  std::vector<ParamGroup> groups = {e1.get_param_groups()[0], e2.get_param_groups()[0]};
  std::vector<std::vector<float>> p, g;
  double sq = 0.0;
  for (size_t k = 0; k < groups.size(); k++) {
    p.push_back(download(groups[k].params, groups[k].size));
    std::vector<float> grad(groups[k].size);
    for (int i = 0; i < groups[k].size; i++) grad[i] = 0.5f * static_cast<float>((i * 7 + 3 * (int)k) % 11 - 5);
    for (float v : grad) sq += static_cast<double>(v) * v;
    upload(groups[k].grads, grad);
    g.push_back(grad);
  }
  const float max_norm = 1.0f;
  const float norm = model.clip_grad_norm(max_norm);
  if (fabs(norm - sqrt(sq)) > 1e-4 * sqrt(sq)) return 1;
  const float coeff = max_norm / (norm + 1e-6f);
  const float lr = 0.01f;
  model.update_weights(lr);
  const float inv1 = 1.0f / (1.0f - powf(0.9f, 1.0f)), inv2 = 1.0f / (1.0f - powf(0.999f, 1.0f));
  for (size_t k = 0; k < groups.size(); k++) {
    const std::vector<float> got = download(groups[k].params, groups[k].size);
    const std::vector<float> got_g = download(groups[k].grads, groups[k].size);
    for (int i = 0; i < groups[k].size; i++) {
      const float gi = g[k][i] * coeff;
      if (fabsf(got_g[i] - gi) > 1e-6f * fabsf(gi) + 1e-12f) return 1;
      const float m = 0.1f * gi, v = 0.001f * gi * gi;
      const float want = p[k][i] - lr * (m * inv1 / (sqrtf(v * inv2) + 1e-8f) + 0.01f * p[k][i]);
      if (fabsf(got[i] - want) > 1e-5f * fmaxf(1.0f, fabsf(want))) return 1;
    }
  }
  return 0;
}

}  // namespace

int main(int argc, char **argv) {
  int devices = 0;
  if (cudaGetDeviceCount(&devices) != cudaSuccess || devices == 0) {
    printf("SKIP: no CUDA device\n");
    return 77;
  }
  const std::string mode = argc > 1 ? argv[1] : "";
  int rc = 2;
  if (mode == "known_answer") rc = known_answer();
  else if (mode == "roundtrip") rc = roundtrip();
  else if (mode == "chain") rc = chain();
  else if (mode == "optimizer") rc = optimizer();
  else if (mode == "checkpoint" && argc == 8)
    rc = checkpoint(argv[2], strtoull(argv[3], nullptr, 10), atoi(argv[4]), atoi(argv[5]), atoi(argv[6]), atoi(argv[7]));
  CUDA_CHECK(cudaDeviceSynchronize());
  printf("%s: %s\n", mode.c_str(), rc == 0 ? "PASS" : "FAIL");
  return rc;
}
