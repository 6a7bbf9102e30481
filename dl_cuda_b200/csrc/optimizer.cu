// Optimizer steps and gradient clipping over a whole list of parameter groups
// in ONE launch each, for sm_100a.
//
// dl-cuda launches one kernel per parameter group (39 for its default char-LM)
// and, for gradient clipping, one Thrust reduction plus one host synchronisation
// per group.  Here the pointer table of up to kMaxGroups groups travels in the
// kernel arguments; the groups are cut into chunks of kChunk elements and the
// CTAs of one grid walk the chunks of all groups.  The squared gradient norm is
// reduced in a fixed order (per-CTA partials, then one CTA) into device memory,
// and the clip kernel reads it there, so clipping needs no host round trip.
//
// The update arithmetic is spelled exactly as in the reference's kernels
// (src/optimizers.cuh:6-55, src/layers.cuh:84-90) so that fp32 results carry the
// same bits.
#include "common.cuh"

namespace dlb {
namespace {

constexpr int kBlock = 256;
constexpr int kMaxGroups = 64;       // groups per launch (more are handled by further launches)
constexpr int kChunk = 4096;         // elements per work item
constexpr int kNormPartials = 1024;  // upper bound on the CTAs of the norm kernel

struct GroupTable {
  float *params[kMaxGroups];
  float *grads[kMaxGroups];
  float *m[kMaxGroups];
  float *v[kMaxGroups];
  int chunk_start[kMaxGroups + 1];  // first work item of each group
  int size[kMaxGroups];
  int count;
};

struct Hyper {
  float lr, beta1, beta2, eps, weight_decay, inv_bc1, inv_bc2;
};

enum Kind { kSgd = 0, kAdam = 1, kAdamW = 2, kRmsprop = 3 };

__device__ __forceinline__ int group_of(const GroupTable &t, int item) {
  int lo = 0, hi = t.count;  // last group whose first item is <= item
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (t.chunk_start[mid] <= item) lo = mid; else hi = mid;
  }
  return lo;
}

template <int KIND>
__device__ __forceinline__ void update_one(float g, float &m, float &v, float &theta, const Hyper &h) {
  if constexpr (KIND == kSgd) {
    theta -= h.lr * g;
  } else if constexpr (KIND == kRmsprop) {
    // m is the running mean of squares (the reference calls it s)
    m = h.beta1 * m + (1 - h.beta1) * g * g;
    theta -= h.lr * g / (sqrtf(m) + h.eps);
  } else {
    m = h.beta1 * m + (1.0f - h.beta1) * g;
    v = h.beta2 * v + (1.0f - h.beta2) * g * g;
    float m_hat = m * h.inv_bc1;
    float v_hat = v * h.inv_bc2;
    if constexpr (KIND == kAdam) {
      theta -= h.lr * m_hat / (sqrtf(v_hat) + h.eps);
    } else {
      theta -= h.lr * (m_hat / (sqrtf(v_hat) + h.eps) + h.weight_decay * theta);
    }
  }
}

// One work item = kChunk consecutive elements of one group; a thread handles
// float4 vectors of it (scalar tail and unaligned groups element by element).
template <int KIND>
__global__ void __launch_bounds__(kBlock)
optim_step_kernel(const __grid_constant__ GroupTable t, const Hyper h, int items) {
  pdl_prologue();
  for (int item = blockIdx.x; item < items; item += gridDim.x) {
    const int gi = group_of(t, item);
    const int begin = (item - t.chunk_start[gi]) * kChunk;
    const int end = min(t.size[gi], begin + kChunk);
    float *p = t.params[gi], *g = t.grads[gi], *m = t.m[gi], *v = t.v[gi];
    const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                       reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15u) == 0;
    const int vend = vec ? begin + ((end - begin) & ~3) : begin;
    for (int i = begin + threadIdx.x * 4; i < vend; i += kBlock * 4) {
      float4 gv = __ldcs(reinterpret_cast<const float4 *>(g + i));
      float4 pv = *reinterpret_cast<float4 *>(p + i);
      float4 mv = make_float4(0.f, 0.f, 0.f, 0.f), vv = mv;
      if (KIND != kSgd) mv = *reinterpret_cast<float4 *>(m + i);
      if (KIND == kAdam || KIND == kAdamW) vv = *reinterpret_cast<float4 *>(v + i);
      update_one<KIND>(gv.x, mv.x, vv.x, pv.x, h);
      update_one<KIND>(gv.y, mv.y, vv.y, pv.y, h);
      update_one<KIND>(gv.z, mv.z, vv.z, pv.z, h);
      update_one<KIND>(gv.w, mv.w, vv.w, pv.w, h);
      *reinterpret_cast<float4 *>(p + i) = pv;
      if (KIND != kSgd) *reinterpret_cast<float4 *>(m + i) = mv;
      if (KIND == kAdam || KIND == kAdamW) *reinterpret_cast<float4 *>(v + i) = vv;
    }
    for (int i = vend + threadIdx.x; i < end; i += kBlock) {
      float mv = KIND != kSgd ? m[i] : 0.f, vv = (KIND == kAdam || KIND == kAdamW) ? v[i] : 0.f, pv = p[i];
      update_one<KIND>(g[i], mv, vv, pv, h);
      p[i] = pv;
      if (KIND != kSgd) m[i] = mv;
      if (KIND == kAdam || KIND == kAdamW) v[i] = vv;
    }
  }
}

// Sum of squares of every gradient: CTA b adds the work items b, b+grid, ... in
// that order (threads keep their own running sums, combined by a fixed tree),
// writes partial[b]; accumulate != 0 adds to what is already in partial[b]
// (second and later launches of one call).
__global__ void __launch_bounds__(kBlock)
grad_sq_partial_kernel(const __grid_constant__ GroupTable t, int items, float *__restrict__ partial,
                       int accumulate) {
  pdl_prologue();
  __shared__ float red[kBlock / 32];
  float acc = 0.f;
  for (int item = blockIdx.x; item < items; item += gridDim.x) {
    const int gi = group_of(t, item);
    const int begin = (item - t.chunk_start[gi]) * kChunk;
    const int end = min(t.size[gi], begin + kChunk);
    const float *g = t.grads[gi];
    const bool vec = (reinterpret_cast<uintptr_t>(g) & 15u) == 0;
    const int vend = vec ? begin + ((end - begin) & ~3) : begin;
    for (int i = begin + threadIdx.x * 4; i < vend; i += kBlock * 4) {
      const float4 gv = __ldcs(reinterpret_cast<const float4 *>(g + i));
      acc += gv.x * gv.x;
      acc += gv.y * gv.y;
      acc += gv.z * gv.z;
      acc += gv.w * gv.w;
    }
    for (int i = vend + threadIdx.x; i < end; i += kBlock) acc += g[i] * g[i];
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < kBlock / 32; w++) total += red[w];
    partial[blockIdx.x] = accumulate ? partial[blockIdx.x] + total : total;
  }
}

// out[0] = sum of the partials (fixed order), out[1] = sqrt of it (the norm),
// out[2] = the factor gradients are scaled by: max_norm/(norm + 1e-6) when the
// norm exceeds max_norm, else 1 (src/optimizer.cuh:222-231 of the reference).
__global__ void __launch_bounds__(kBlock)
grad_norm_finish_kernel(const float *partial, int n, float max_norm, float *__restrict__ out) {
  pdl_prologue();
  __shared__ float red[kBlock];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += kBlock) acc += partial[i];
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int s = kBlock / 2; s > 0; s >>= 1) {
    if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float total = red[0];
    const float norm = sqrtf(total);
    out[0] = total;
    out[1] = norm;
    out[2] = (max_norm > 0.f && norm > max_norm) ? max_norm / (norm + 1e-6f) : 1.0f;
  }
}

__global__ void __launch_bounds__(kBlock)
scale_grads_kernel(const __grid_constant__ GroupTable t, int items, const float *coeff) {
  pdl_prologue();
  const float c = *coeff;
  if (c == 1.0f) return;  // not above the limit: gradients stay untouched, as in the reference
  for (int item = blockIdx.x; item < items; item += gridDim.x) {
    const int gi = group_of(t, item);
    const int begin = (item - t.chunk_start[gi]) * kChunk;
    const int end = min(t.size[gi], begin + kChunk);
    float *g = t.grads[gi];
    const bool vec = (reinterpret_cast<uintptr_t>(g) & 15u) == 0;
    const int vend = vec ? begin + ((end - begin) & ~3) : begin;
    for (int i = begin + threadIdx.x * 4; i < vend; i += kBlock * 4) {
      float4 gv = *reinterpret_cast<float4 *>(g + i);
      gv.x *= c; gv.y *= c; gv.z *= c; gv.w *= c;
      *reinterpret_cast<float4 *>(g + i) = gv;
    }
    for (int i = vend + threadIdx.x; i < end; i += kBlock) g[i] *= c;
  }
}

// Checkpoint body: per group one int32 size word followed by the group's floats, groups back to
// back (the DLCU file after its 12-byte header).  word_offset[i] is where group i's size word sits.
struct PackTable {
  float *group[kMaxGroups];
  long long word_offset[kMaxGroups];
  int chunk_start[kMaxGroups + 1];
  int size[kMaxGroups];
  int count;
};

__global__ void __launch_bounds__(kBlock)
checkpoint_copy_kernel(const __grid_constant__ PackTable t, int items, uint32_t *body, int to_body) {
  pdl_prologue();
  for (int item = blockIdx.x; item < items; item += gridDim.x) {
    int lo = 0, hi = t.count;  // last group whose first item is <= item
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (t.chunk_start[mid] <= item) lo = mid; else hi = mid;
    }
    const int begin = (item - t.chunk_start[lo]) * kChunk;
    const int end = min(t.size[lo], begin + kChunk);
    uint32_t *words = body + t.word_offset[lo];
    float *g = t.group[lo];
    if (to_body) {
      if (begin == 0 && threadIdx.x == 0) words[0] = static_cast<uint32_t>(t.size[lo]);
      for (int i = begin + threadIdx.x; i < end; i += kBlock) words[1 + i] = __float_as_uint(g[i]);
    } else {
      for (int i = begin + threadIdx.x; i < end; i += kBlock) g[i] = __uint_as_float(words[1 + i]);
    }
  }
}

// Fills a table with groups [first, first+count) of the caller's arrays; returns the work items.
int fill_table(GroupTable &t, int first, int count, float *const *params, float *const *grads,
               float *const *m, float *const *v, const int *sizes) {
  t.count = count;
  int items = 0;
  for (int i = 0; i < count; i++) {
    t.params[i] = params ? params[first + i] : nullptr;
    t.grads[i] = grads[first + i];
    t.m[i] = m ? m[first + i] : nullptr;
    t.v[i] = v ? v[first + i] : nullptr;
    t.size[i] = sizes[first + i];
    t.chunk_start[i] = items;
    items += ceil_div(sizes[first + i], kChunk);
  }
  t.chunk_start[count] = items;
  return items;
}

int grid_for(int items, int cap) {
  const int want = items < 1 ? 1 : items;
  return want < cap ? want : cap;
}

bool groups_ok(int n_groups, float *const *grads, const int *sizes) {
  if (n_groups < 0 || (n_groups > 0 && (!grads || !sizes))) return false;
  for (int i = 0; i < n_groups; i++)
    if (sizes[i] < 0 || (sizes[i] > 0 && !grads[i])) return false;
  return true;
}

}  // namespace
}  // namespace dlb

using namespace dlb;

extern "C" int dlb_optim_step(int kind, int n_groups, float *const *h_params, float *const *h_grads,
                              float *const *h_m, float *const *h_v, const int *h_sizes, float lr,
                              float beta1, float beta2, float eps, float weight_decay,
                              float inv_bias_correction1, float inv_bias_correction2, void *stream) {
  DLB_REQUIRE(kind >= kSgd && kind <= kRmsprop, DLB_ERR_INVALID_ARG, "optim_step: unknown optimizer %d", kind);
  DLB_REQUIRE(groups_ok(n_groups, h_grads, h_sizes) && (n_groups == 0 || h_params), DLB_ERR_INVALID_ARG,
              "optim_step: bad group arrays");
  DLB_REQUIRE(kind == kSgd || n_groups == 0 || h_m, DLB_ERR_INVALID_ARG, "optim_step: first-moment buffers required");
  DLB_REQUIRE((kind != kAdam && kind != kAdamW) || n_groups == 0 || h_v, DLB_ERR_INVALID_ARG,
              "optim_step: second-moment buffers required");
  const Hyper h{lr, beta1, beta2, eps, weight_decay, inv_bias_correction1, inv_bias_correction2};
  cudaStream_t st = as_stream(stream);
  for (int first = 0; first < n_groups; first += kMaxGroups) {
    GroupTable t;
    const int count = n_groups - first < kMaxGroups ? n_groups - first : kMaxGroups;
    const int items = fill_table(t, first, count, h_params, h_grads, h_m, h_v, h_sizes);
    if (items == 0) continue;
    const int grid = grid_for(items, sm_count() * 16);
    switch (kind) {
      case kSgd: launch_pdl(optim_step_kernel<kSgd>, grid, kBlock, 0, st, t, h, items); break;
      case kAdam: launch_pdl(optim_step_kernel<kAdam>, grid, kBlock, 0, st, t, h, items); break;
      case kAdamW: launch_pdl(optim_step_kernel<kAdamW>, grid, kBlock, 0, st, t, h, items); break;
      default: launch_pdl(optim_step_kernel<kRmsprop>, grid, kBlock, 0, st, t, h, items); break;
    }
    DLB_LAUNCH_CHECK("optim_step");
  }
  return DLB_OK;
}

extern "C" size_t dlb_grad_norm_workspace_bytes(void) { return sizeof(float) * (kNormPartials + 4); }

extern "C" int dlb_grad_norm_clip(int n_groups, float *const *h_grads, const int *h_sizes, float max_norm,
                                  void *workspace, size_t workspace_bytes, float *d_result, void *stream) {
  DLB_REQUIRE(groups_ok(n_groups, h_grads, h_sizes), DLB_ERR_INVALID_ARG, "grad_norm_clip: bad group arrays");
  DLB_REQUIRE(workspace && aligned16(workspace) && workspace_bytes >= dlb_grad_norm_workspace_bytes(),
              DLB_ERR_WORKSPACE, "grad_norm_clip: 16-byte aligned workspace of %zu bytes required",
              dlb_grad_norm_workspace_bytes());
  DLB_REQUIRE(d_result != nullptr, DLB_ERR_INVALID_ARG, "grad_norm_clip: null result");
  cudaStream_t st = as_stream(stream);
  float *partial = static_cast<float *>(workspace);
  // Every launch uses the same grid so that partial[b] accumulates across launches.
  const int grid = grid_for(INT32_MAX, min(kNormPartials, sm_count() * 6));
  bool any = false;
  for (int first = 0; first < n_groups; first += kMaxGroups) {
    GroupTable t;
    const int count = n_groups - first < kMaxGroups ? n_groups - first : kMaxGroups;
    const int items = fill_table(t, first, count, nullptr, h_grads, nullptr, nullptr, h_sizes);
    launch_pdl(grad_sq_partial_kernel, grid, kBlock, 0, st, t, items, partial, any ? 1 : 0);
    DLB_LAUNCH_CHECK("grad_sq_partial");
    any = true;
  }
  launch_pdl(grad_norm_finish_kernel, 1, kBlock, 0, st, partial, any ? grid : 0, max_norm, d_result);
  DLB_LAUNCH_CHECK("grad_norm_finish");
  if (max_norm > 0.f) {
    for (int first = 0; first < n_groups; first += kMaxGroups) {
      GroupTable t;
      const int count = n_groups - first < kMaxGroups ? n_groups - first : kMaxGroups;
      const int items = fill_table(t, first, count, nullptr, h_grads, nullptr, nullptr, h_sizes);
      if (items == 0) continue;
      launch_pdl(scale_grads_kernel, grid_for(items, sm_count() * 16), kBlock, 0, st, t, items, d_result + 2);
      DLB_LAUNCH_CHECK("scale_grads");
    }
  }
  return DLB_OK;
}

// ---- checkpoint staging ------------------------------------------------------------------------

extern "C" size_t dlb_checkpoint_body_bytes(int n_groups, const int *h_sizes) {
  if (n_groups < 0 || (n_groups > 0 && !h_sizes)) return 0;
  size_t words = 0;
  for (int i = 0; i < n_groups; i++) {
    if (h_sizes[i] < 0) return 0;
    words += 1 + static_cast<size_t>(h_sizes[i]);
  }
  return words * sizeof(uint32_t);
}

static int checkpoint_copy(const char *what, int n_groups, float *const *h_params, const int *h_sizes, void *d_body,
                           size_t body_bytes, int to_body, void *stream) {
  DLB_REQUIRE(groups_ok(n_groups, h_params, h_sizes), DLB_ERR_INVALID_ARG, "%s: bad group arrays", what);
  DLB_REQUIRE(n_groups == 0 || (d_body && (reinterpret_cast<uintptr_t>(d_body) & 3u) == 0 &&
                                body_bytes >= dlb_checkpoint_body_bytes(n_groups, h_sizes)),
              DLB_ERR_WORKSPACE, "%s: a body buffer of %zu bytes is required", what,
              dlb_checkpoint_body_bytes(n_groups, h_sizes));
  long long offset = 0;
  for (int first = 0; first < n_groups; first += kMaxGroups) {
    PackTable t;
    t.count = n_groups - first < kMaxGroups ? n_groups - first : kMaxGroups;
    int items = 0;
    for (int i = 0; i < t.count; i++) {
      t.group[i] = h_params[first + i];
      t.size[i] = h_sizes[first + i];
      t.word_offset[i] = offset;
      t.chunk_start[i] = items;
      // a group of size 0 still owns its size word: give it one (empty) work item
      items += h_sizes[first + i] > 0 ? ceil_div(h_sizes[first + i], kChunk) : 1;
      offset += 1 + static_cast<long long>(h_sizes[first + i]);
    }
    t.chunk_start[t.count] = items;
    launch_pdl(checkpoint_copy_kernel, grid_for(items, sm_count() * 16), kBlock, 0, as_stream(stream), t, items,
               static_cast<uint32_t *>(d_body), to_body);
    DLB_LAUNCH_CHECK(what);
  }
  return DLB_OK;
}

extern "C" int dlb_checkpoint_pack(int n_groups, float *const *h_params, const int *h_sizes, void *d_body,
                                   size_t body_bytes, void *stream) {
  return checkpoint_copy("checkpoint_pack", n_groups, h_params, h_sizes, d_body, body_bytes, 1, stream);
}

extern "C" int dlb_checkpoint_unpack(int n_groups, float *const *h_params, const int *h_sizes, const void *d_body,
                                     size_t body_bytes, void *stream) {
  return checkpoint_copy("checkpoint_unpack", n_groups, h_params, h_sizes, const_cast<void *>(d_body), body_bytes, 0,
                         stream);
}
