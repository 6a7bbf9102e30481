// Operation / ParamGroup / Sequential with the interface of dl-cuda's
// src/sequential.cuh (:19-36, :111-267), so that code written against the
// reference's layer API compiles against these headers unchanged.  The layer
// classes beside this file run their forward/backward through the C ABI of
// libdlcuda_b200.so; this file owns only the plumbing between layers and the
// DLCU checkpoint file, whose bytes are those of the reference:
//   'D','L','C','U' | int32 version = 1 | int32 group count |
//   per parameter group: int32 size, float32[size]   (host byte order).
#pragma once

#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/dlcuda_b200.h"

#define CUDA_CHECK(call)                                                                      \
  do {                                                                                        \
    cudaError_t cuda_check_err = (call);                                                      \
    if (cuda_check_err != cudaSuccess) {                                                      \
      fprintf(stderr, "CUDA error at %s:%d: %s\n", __FILE__, __LINE__,                        \
              cudaGetErrorString(cuda_check_err));                                            \
      exit(EXIT_FAILURE);                                                                     \
    }                                                                                         \
  } while (0)

// Same convention for the kernel library: print and exit, as CUDA_CHECK does.
#define DLB_CHECK(call)                                                                       \
  do {                                                                                        \
    int dlb_check_status = (call);                                                            \
    if (dlb_check_status != DLB_OK) {                                                         \
      fprintf(stderr, "dlcuda_b200 error at %s:%d: %s\n", __FILE__, __LINE__, dlb_last_error()); \
      exit(EXIT_FAILURE);                                                                     \
    }                                                                                         \
  } while (0)

struct ParamGroup {
  float *params;
  float *grads;
  int size;
};

class Optimizer;

class Operation {
public:
  virtual void forward(float *d_input, float *d_output) = 0;
  virtual void backward(float *d_output_grad, float *d_input_grad) = 0;
  virtual void update_weights(float /*lr*/) {}
  virtual int input_size() const = 0;
  virtual int output_size() const = 0;
  virtual std::vector<ParamGroup> get_param_groups() { return {}; }
  virtual ~Operation() = default;
};

// A device allocation that frees itself; layers hold these instead of raw
// cudaMalloc/cudaFree pairs.
template <typename T>
class DeviceBuffer {
public:
  DeviceBuffer() = default;
  explicit DeviceBuffer(size_t count) { reset(count); }
  DeviceBuffer(const DeviceBuffer &) = delete;
  DeviceBuffer &operator=(const DeviceBuffer &) = delete;
  ~DeviceBuffer() { release(); }
  void reset(size_t count) {
    release();
    count_ = count;
    if (count > 0) CUDA_CHECK(cudaMalloc(&ptr_, count * sizeof(T)));
  }
  T *get() const { return ptr_; }
  size_t count() const { return count_; }

private:
  void release() {
    if (ptr_) cudaFree(ptr_);
    ptr_ = nullptr;
    count_ = 0;
  }
  T *ptr_ = nullptr;
  size_t count_ = 0;
};

class Sequential {
public:
  void add(Operation *op) {
    ops_.push_back(op);
    activations_.clear();
    gradients_.clear();
  }

  // Activations between layers live in buffers owned here, sized from each
  // layer's output_size(); the caller owns d_input and d_output.
  void forward(float *d_input, float *d_output) {
    if (ops_.empty()) return;
    size_links(activations_, /*forward=*/true);
    float *in = d_input;
    for (size_t i = 0; i < ops_.size(); ++i) {
      float *out = (i + 1 == ops_.size()) ? d_output : activations_[i].get();
      ops_[i]->forward(in, out);
      in = out;
    }
  }

  void backward(float *d_output_grad, float *d_input_grad) {
    if (ops_.empty()) return;
    size_links(gradients_, /*forward=*/false);
    float *grad = d_output_grad;
    for (size_t i = ops_.size(); i-- > 0;) {
      float *prev = (i == 0) ? d_input_grad : gradients_[i - 1].get();
      ops_[i]->backward(grad, prev);
      grad = prev;
    }
  }

  inline void set_optimizer(Optimizer *opt);
  inline void update_weights(float lr);
  inline float clip_grad_norm(float max_norm);

  std::vector<Operation *> &get_operations() { return ops_; }

  bool save_weights(const std::string &path) {
    std::vector<ParamGroup> groups = all_groups();
    // Stage the whole file in host memory, then write it in one go.
    std::vector<char> bytes;
    auto put = [&bytes](const void *p, size_t n) {
      const char *c = static_cast<const char *>(p);
      bytes.insert(bytes.end(), c, c + n);
    };
    put("DLCU", 4);
    const int version = kVersion, count = static_cast<int>(groups.size());
    put(&version, sizeof(int));
    put(&count, sizeof(int));
    std::vector<float> host;
    for (const ParamGroup &g : groups) {
      put(&g.size, sizeof(int));
      host.resize(static_cast<size_t>(g.size));
      CUDA_CHECK(cudaMemcpy(host.data(), g.params, sizeof(float) * host.size(), cudaMemcpyDeviceToHost));
      put(host.data(), sizeof(float) * host.size());
    }
    FILE *f = fopen(path.c_str(), "wb");
    if (!f) return false;
    const bool ok = fwrite(bytes.data(), 1, bytes.size(), f) == bytes.size();
    return (fclose(f) == 0) && ok;
  }

  // Any mismatch (magic, version, group count, a group's size, a short file)
  // returns false.  Groups read before the mismatch have already been uploaded,
  // as in the reference.
  bool load_weights(const std::string &path) {
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) return false;
    bool ok = false;
    do {
      char magic[4];
      int version = 0, count = 0;
      if (fread(magic, 1, 4, f) != 4 || memcmp(magic, "DLCU", 4) != 0) break;
      if (fread(&version, sizeof(int), 1, f) != 1 || version != kVersion) break;
      std::vector<ParamGroup> groups = all_groups();
      if (fread(&count, sizeof(int), 1, f) != 1 || count != static_cast<int>(groups.size())) break;
      std::vector<float> host;
      size_t done = 0;
      for (const ParamGroup &g : groups) {
        int size = 0;
        if (fread(&size, sizeof(int), 1, f) != 1 || size != g.size) break;
        host.resize(static_cast<size_t>(size));
        if (fread(host.data(), sizeof(float), host.size(), f) != host.size()) break;
        CUDA_CHECK(cudaMemcpy(g.params, host.data(), sizeof(float) * host.size(), cudaMemcpyHostToDevice));
        ++done;
      }
      ok = done == groups.size();
    } while (false);
    fclose(f);
    return ok;
  }

private:
  static constexpr int kVersion = 1;

  std::vector<ParamGroup> all_groups() {
    std::vector<ParamGroup> groups;
    for (Operation *op : ops_)
      for (const ParamGroup &g : op->get_param_groups()) groups.push_back(g);
    return groups;
  }

  // link i sits between op i and op i+1: op i's output going forward, op i+1's
  // input gradient going backward.
  void size_links(std::vector<DeviceBuffer<float>> &links, bool forward) {
    const size_t need = ops_.size() - 1;
    bool fits = links.size() == need;
    for (size_t i = 0; fits && i < need; ++i) {
      const int want = forward ? ops_[i]->output_size() : ops_[i + 1]->input_size();
      fits = links[i].count() == static_cast<size_t>(want);
    }
    if (fits) return;
    links = std::vector<DeviceBuffer<float>>(need);
    for (size_t i = 0; i < need; ++i)
      links[i].reset(static_cast<size_t>(forward ? ops_[i]->output_size() : ops_[i + 1]->input_size()));
  }

  std::vector<Operation *> ops_;
  Optimizer *optimizer_ = nullptr;
  std::vector<DeviceBuffer<float>> activations_, gradients_;
};
