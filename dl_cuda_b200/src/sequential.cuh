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

// A bounded wait inside a pipelined kernel that gave up leaves wrong results behind without a
// CUDA error.  Called where the host synchronises anyway (gradient clipping, checkpoint
// writing), so that such a step is neither trained on nor saved.
inline void dlb_require_no_pipeline_timeouts(const char *where) {
  unsigned int gave_up = 0;
  DLB_CHECK(dlb_pipeline_timeouts(&gave_up));
  if (gave_up != 0) {
    fprintf(stderr, "dlcuda_b200: %u pipeline wait(s) timed out before %s: results since then are invalid\n",
            gave_up, where);
    exit(EXIT_FAILURE);
  }
}

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

  // The file is assembled on the device (one launch writes every group's size word and values
  // into one buffer), copied to pinned host memory in one transfer and written with one fwrite.
  bool save_weights(const std::string &path) {
    dlb_require_no_pipeline_timeouts("save_weights");
    const GroupArrays g = group_arrays();
    const size_t body = dlb_checkpoint_body_bytes(static_cast<int>(g.sizes.size()), g.sizes.data());
    PinnedFile file(kHeaderBytes + body);
    memcpy(file.bytes, "DLCU", 4);
    const int version = kVersion, count = static_cast<int>(g.sizes.size());
    memcpy(file.bytes + 4, &version, sizeof(int));
    memcpy(file.bytes + 8, &count, sizeof(int));
    if (body > 0) {
      DeviceBuffer<unsigned char> staging(body);
      DLB_CHECK(dlb_checkpoint_pack(count, g.params.data(), g.sizes.data(), staging.get(), body, nullptr));
      CUDA_CHECK(cudaMemcpy(file.bytes + kHeaderBytes, staging.get(), body, cudaMemcpyDeviceToHost));
    }
    FILE *f = fopen(path.c_str(), "wb");
    if (!f) return false;
    const bool ok = fwrite(file.bytes, 1, file.size, f) == file.size;
    return (fclose(f) == 0) && ok;
  }

  // Any mismatch (magic, version, group count, a group's size, a short file) returns false and
  // leaves every parameter untouched: the file is validated on the host before its body goes to
  // the device in one transfer and one launch scatters it into the groups.
  bool load_weights(const std::string &path) {
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) return false;
    const GroupArrays g = group_arrays();
    const size_t body = dlb_checkpoint_body_bytes(static_cast<int>(g.sizes.size()), g.sizes.data());
    PinnedFile file(kHeaderBytes + body);
    const size_t got = fread(file.bytes, 1, file.size, f);
    fclose(f);
    if (got != file.size || memcmp(file.bytes, "DLCU", 4) != 0) return false;
    int version = 0, count = 0;
    memcpy(&version, file.bytes + 4, sizeof(int));
    memcpy(&count, file.bytes + 8, sizeof(int));
    if (version != kVersion || count != static_cast<int>(g.sizes.size())) return false;
    size_t at = kHeaderBytes;
    for (int size : g.sizes) {
      int stored = 0;
      memcpy(&stored, file.bytes + at, sizeof(int));
      if (stored != size) return false;
      at += sizeof(int) + sizeof(float) * static_cast<size_t>(size);
    }
    if (body > 0) {
      DeviceBuffer<unsigned char> staging(body);
      CUDA_CHECK(cudaMemcpy(staging.get(), file.bytes + kHeaderBytes, body, cudaMemcpyHostToDevice));
      DLB_CHECK(dlb_checkpoint_unpack(count, g.params.data(), g.sizes.data(), staging.get(), body, nullptr));
      CUDA_CHECK(cudaDeviceSynchronize());  // the staging buffer is freed on return
    }
    return true;
  }

private:
  static constexpr int kVersion = 1;
  static constexpr size_t kHeaderBytes = 12;  // magic, version, group count

  struct GroupArrays {
    std::vector<float *> params;
    std::vector<int> sizes;
  };
  GroupArrays group_arrays() {
    GroupArrays g;
    for (const ParamGroup &pg : all_groups()) {
      g.params.push_back(pg.params);
      g.sizes.push_back(pg.size);
    }
    return g;
  }

  // Page-locked host image of a weights file.
  struct PinnedFile {
    unsigned char *bytes = nullptr;
    size_t size;
    explicit PinnedFile(size_t n) : size(n) { CUDA_CHECK(cudaMallocHost(reinterpret_cast<void **>(&bytes), n ? n : 1)); }
    PinnedFile(const PinnedFile &) = delete;
    PinnedFile &operator=(const PinnedFile &) = delete;
    ~PinnedFile() { cudaFreeHost(bytes); }
  };

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
