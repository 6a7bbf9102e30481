// The whole sorted-segment plan of the embedding scatter-add in ONE launch, for
// batches of up to kClusterPlanMaxTokens tokens: a thread-block cluster of 8
// CTAs (8192 threads) runs every phase back to back and meets at hardware
// cluster barriers instead of kernel boundaries:
//   per radix pass   digit histogram of the CTA's slice of the tokens (shared
//                    memory), cluster barrier, every CTA reads the other CTAs'
//                    histograms through distributed shared memory and derives
//                    its own scatter bases, stable scatter of its slice in token
//                    order (warp match-any ranks + per-warp digit counters),
//                    cluster barrier;
//   segment starts   seg_start[v] = lower_bound(sorted ids, v), v in [0, V];
//   long rows        ordered list of ids with more than kSubLen tokens and the
//                    running count of their sub-segments (per-CTA counts are
//                    exchanged through distributed shared memory).
// Everything a later phase reads was written by other CTAs of the same kernel,
// so those reads use ld.global.cg (L2), never the non-coherent path.
#pragma once

#include <cooperative_groups.h>

#include "common.cuh"

namespace dlb {

namespace cg = cooperative_groups;

constexpr int kClusterCtas = 8;
constexpr int kClusterThreads = 1024;
constexpr int kClusterPlanMaxTokens = 1 << 16;
constexpr size_t kClusterPlanSmem = sizeof(int) * (1024 + 2 * (kClusterThreads / 32) * 256);

struct ClusterPlanArgs {
  const uint32_t *ids;
  uint32_t *keys[2];
  int32_t *vals[2];
  int32_t *seg_start, *long_row, *long_first, *meta;
  int num_tokens, vocab, passes, sub_len;
};

// Exclusive scan of one int per thread over the first `n` threads (n a multiple
// of 32, n <= 1024); `tmp` holds 33 ints.  Returns the exclusive prefix; *total
// receives the sum.  All threads of the CTA must call it.
__device__ __forceinline__ int cta_exclusive_scan(int v, int n, int *tmp, int *total) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int incl = tid < n ? v : 0;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  __syncthreads();
  if (lane == 31) tmp[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const int w = tmp[lane];
    int wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    tmp[lane] = wi - w;
    if (lane == 31) tmp[32] = wi;
  }
  __syncthreads();
  *total = tmp[32];
  return tmp[warp] + incl - (tid < n ? v : 0);
}

__global__ void __cluster_dims__(kClusterCtas, 1, 1) __launch_bounds__(kClusterThreads)
embed_plan_cluster_kernel(ClusterPlanArgs a) {
  // Launched plainly and without an early trigger: this kernel neither overlaps its
  // predecessor nor lets its successor be scheduled before it has finished.  (With
  // programmatic dependent launch around this cluster kernel, the kernel after it
  // was seen reading the plan before it was complete.)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  cg::cluster_group cluster = cg::this_cluster();
  // Dynamic shared memory (68 KB, above the static limit), same layout in every CTA.
  extern __shared__ int smem_i[];
  int *hist = smem_i;            // [256] this CTA's digit counts (read by the other CTAs)
  int *running = smem_i + 256;   // [256] next free slot per digit for this CTA
  int *counts = smem_i + 512;    // [2]   {long rows, sub-segments} of this CTA's id slice
  int *tmp = smem_i + 520;       // [33]  scan scratch
  int (*wcnt)[256] = reinterpret_cast<int (*)[256]>(smem_i + 1024);  // per-warp digit counts of a tile
  int (*wbase)[256] = wcnt + kClusterThreads / 32;                   // per-warp digit bases of a tile

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rank = static_cast<int>(cluster.block_rank());
  const int T = a.num_tokens, V = a.vocab;
  const int chunk = ((T + kClusterCtas - 1) / kClusterCtas + kClusterThreads - 1) / kClusterThreads * kClusterThreads;
  const int begin = min(T, rank * chunk), end = min(T, begin + chunk);

  for (int i = tid; i < (kClusterThreads / 32) * 256; i += kClusterThreads) (&wcnt[0][0])[i] = 0;

  for (int pass = 0; pass < a.passes; pass++) {
    const int shift = 8 * pass;
    const uint32_t *kin = pass == 0 ? a.ids : a.keys[pass & 1];
    const int32_t *vin = pass == 0 ? nullptr : a.vals[pass & 1];
    uint32_t *kout = a.keys[(pass + 1) & 1];
    int32_t *vout = a.vals[(pass + 1) & 1];

    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    for (int i = begin + tid; i < end; i += kClusterThreads)
      atomicAdd(&hist[(__ldcg(kin + i) >> shift) & 255u], 1);  // integer counts: order-free
    cluster.sync();

    // Scatter base of digit d for this CTA: all smaller digits anywhere, plus
    // digit d in the CTAs that hold earlier tokens.
    int tot = 0, mine = 0;
    if (tid < 256) {
      for (int c = 0; c < kClusterCtas; c++) {
        const int h = *cluster.map_shared_rank(&hist[tid], c);
        if (c < rank) mine += h;
        tot += h;
      }
    }
    int all;
    const int excl = cta_exclusive_scan(tot, 256, tmp, &all);
    if (tid < 256) running[tid] = excl + mine;
    __syncthreads();

    for (int tile = begin; tile < end; tile += kClusterThreads) {
      const int i = tile + tid;
      const bool ok = i < end;
      const uint32_t key = ok ? __ldcg(kin + i) : 0u;
      const int32_t val = ok ? (vin ? __ldcg(vin + i) : i) : -1;
      const uint32_t digit = ok ? ((key >> shift) & 255u) : 256u;  // 256: padding lanes
      const uint32_t peers = __match_any_sync(0xffffffffu, digit);
      const int below = __popc(peers & ((1u << lane) - 1u));
      if (ok && below == 0) wcnt[warp][digit] = __popc(peers);
      __syncthreads();
      if (tid < 256) {
        int run = running[tid];
#pragma unroll 8
        for (int w = 0; w < kClusterThreads / 32; w++) {
          const int c = wcnt[w][tid];
          wcnt[w][tid] = 0;  // clean for the next tile
          wbase[w][tid] = run;
          run += c;
        }
        running[tid] = run;
      }
      __syncthreads();
      if (ok) {
        const int pos = wbase[warp][digit] + below;
        kout[pos] = key;
        vout[pos] = val;
      }
    }
    __threadfence();
    cluster.sync();  // the scatter of every CTA is visible; hist may be reused
  }

  // seg_start[v] = first position whose key is >= v.
  const uint32_t *sorted = a.passes == 0 ? a.ids : a.keys[a.passes & 1];
  for (int v = rank * kClusterThreads + tid; v <= V; v += kClusterCtas * kClusterThreads) {
    int lo = 0, hi = T;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (__ldcg(sorted + mid) < static_cast<uint32_t>(v)) lo = mid + 1; else hi = mid;
    }
    a.seg_start[v] = lo;
  }
  __threadfence();
  cluster.sync();

  // Long rows of this CTA's slice of the ids, in id order.
  const int vchunk = (V + kClusterCtas - 1) / kClusterCtas;
  const int v0 = min(V, rank * vchunk), v1 = min(V, v0 + vchunk);
  int nl = 0, ns = 0;
  for (int v = v0 + tid; v < v1; v += kClusterThreads) {
    const int c = __ldcg(a.seg_start + v + 1) - __ldcg(a.seg_start + v);
    if (c > a.sub_len) { nl++; ns += (c + a.sub_len - 1) / a.sub_len; }
  }
  int total_l, total_s;
  cta_exclusive_scan(nl, kClusterThreads, tmp, &total_l);
  cta_exclusive_scan(ns, kClusterThreads, tmp, &total_s);
  if (tid == 0) { counts[0] = total_l; counts[1] = total_s; }
  cluster.sync();
  int base_l = 0, base_s = 0, all_l = 0, all_s = 0;
  for (int c = 0; c < kClusterCtas; c++) {
    const int *pc = cluster.map_shared_rank(&counts[0], c);
    const int l = pc[0], s = pc[1];
    if (c < rank) { base_l += l; base_s += s; }
    all_l += l; all_s += s;
  }
  for (int vb = v0; vb < v1; vb += kClusterThreads) {
    const int v = vb + tid;
    int f = 0, m = 0;
    if (v < v1) {
      const int c = __ldcg(a.seg_start + v + 1) - __ldcg(a.seg_start + v);
      if (c > a.sub_len) { f = 1; m = (c + a.sub_len - 1) / a.sub_len; }
    }
    int tl, ts;
    const int ol = cta_exclusive_scan(f, kClusterThreads, tmp, &tl);
    const int os = cta_exclusive_scan(m, kClusterThreads, tmp, &ts);
    if (f) {
      a.long_row[base_l + ol] = v;
      a.long_first[base_l + ol] = base_s + os;
    }
    base_l += tl;
    base_s += ts;
  }
  if (rank == kClusterCtas - 1 && tid == 0) {
    a.meta[0] = all_l;
    a.meta[1] = all_s;
    a.long_first[all_l] = all_s;
  }
  // No CTA may retire while another can still read its shared memory.
  cluster.sync();
}

}  // namespace dlb
