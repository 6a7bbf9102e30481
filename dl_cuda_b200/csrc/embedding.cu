// Token embedding for sm_100a: the gather with the sinusoidal positional-
// encoding add folded in, and the gradient of the table as a deterministic
// sorted-segment sum (no atomics, no memset).
//
// Backward in three steps.
//  1. dlb_embed_sort_tokens: a stable LSD radix sort of (id, token index) pairs
//     (8-bit digits, 2048-token tiles, warp match-any ranking), then per id the
//     start of its run in the sorted list (binary search), then the list of
//     "long" ids (more than kSubLen tokens) with their sub-segment offsets.
//  2. scatter_rows_kernel (embed_scatter.cuh): one thread group per table row.
//     A row with at most kSubLen tokens is summed in ascending token order and
//     written once (zero if no token refers to it).  Long rows are cut into
//     sub-segments of kSubLen tokens, each summed by its own thread group into a
//     scratch row.
//  3. combine_long_kernel: adds a long row's scratch rows: 8 contiguous slices of
//     the sub-segments are summed in order, then the 8 slice sums in order.
// The order of every addition is a function of ids alone, so two runs give the
// same bits whatever the scheduling.
#include "common.cuh"
#include "embed_plan_cluster.cuh"
#include "embed_scatter.cuh"
#include "tma.cuh"

namespace dlb {
namespace {

constexpr int kBlock = kEmbBlock;

// ------------------------------------------------------------------ gather
// blockDim = (tx, ty): tx threads cover tx column vectors, ty positions per
// CTA.  A thread keeps the PE vector of its (position, column) and walks the
// tokens that share the position (t = s, s+S, s+2S, ...), U gathers in flight.
// U = 4 keeps the kernel at 40 registers (six CTAs per SM) and is the default; U = 8 with the ids
// fetched one group ahead (three CTAs per SM) was measured slower on B200: bf16, 32768 tokens of
// 4096: 88.6 against 74.4 us; fp32: 148.8 against 119.9 us (dlb_set_option "gather_rows_in_flight").
template <typename T, int U>
__global__ void __launch_bounds__(kBlock, U >= 8 ? 3 : 6)
embed_gather_kernel(const T *table, const int32_t *ids,
                    const float *__restrict__ pe, T *__restrict__ out, int num_tokens, int vocab,
                    int d, int stride_s) {
  pdl_prologue();
  using S = Store<T>;
  constexpr int E = S::kPerVec;
  const int ncv = d / E;
  const int cv = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.y * blockDim.y + threadIdx.y;
  if (cv >= ncv || s >= stride_s) return;

  float pv[E];
#pragma unroll
  for (int e = 0; e < E; e++) pv[e] = 0.f;
  if (pe != nullptr) {
#pragma unroll
    for (int q = 0; q < E / 4; q++) {
      const float4 p4 = ld_const_f4(pe + static_cast<size_t>(s) * d + cv * E + 4 * q);
      pv[4 * q] = p4.x; pv[4 * q + 1] = p4.y; pv[4 * q + 2] = p4.z; pv[4 * q + 3] = p4.w;
    }
  }
  // (token indices fit an int: num_tokens + U * stride_s stays below 2^31, checked on the host)
  int next_id[U];
  if constexpr (U >= 8) {
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int t = s + u * stride_s;
      next_id[u] = t < num_tokens ? ld_co(ids + t) : 0;
    }
  }
  for (int t0 = s; t0 < num_tokens; t0 += U * stride_s) {
    uint4 row[U];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int t = t0 + u * stride_s;
      ok[u] = t < num_tokens;
      if (ok[u]) {
        int id = U >= 8 ? next_id[u] : ld_co(ids + t);
        id = max(0, min(id, vocab - 1));  // out-of-range ids cannot leave the table
        row[u] = ld_keep(table + static_cast<size_t>(id) * d + cv * E);
      }
    }
    if constexpr (U >= 8) {
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int t = t0 + (U + u) * stride_s;
        next_id[u] = t < num_tokens ? ld_co(ids + t) : 0;
      }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      if (ok[u]) {
        float v[E];
        S::unpack(row[u], v);
#pragma unroll
        for (int e = 0; e < E; e++) v[e] = v[e] + pv[e];
        const size_t t = static_cast<size_t>(t0) + static_cast<size_t>(u) * stride_s;
        st_stream(out + t * d + cv * E, S::pack(v));
      }
    }
  }
}

// The gather as a bulk-copy (TMA) pipeline, the alternative form of embed_gather_kernel
// (dlb_set_option "gather_variant" = 2).  A CTA takes positions s = cta, cta + grid, ...; the launch code
// sizes the grid so that a CTA moves about 450 KB of table rows.
//   producer warp   lane l fetches the id of the l-th token that shares the position, lane 0 then
//                   streams the positional-encoding row and the table rows of those tokens into a
//                   ring of shared-memory stages with cp.async.bulk (completion on mbarriers);
//   consumer warps  keep the position's PE values of their columns in registers, and per row read
//                   their vectors from the stage, add, and store to the output (coalesced 16-byte
//                   stores); a stage is handed back once every consumer warp has read it.
// No thread holds a table row in registers while it is in flight, and the id -> row dependency is the
// producer's alone, so the bytes in flight are set by the ring depth.
constexpr int kGatherConsumers = 256;
constexpr int kGatherThreads = kGatherConsumers + 32;

struct GatherBulkLayout {
  int stages;
  unsigned row_bytes, pe_bytes, pe_off, bar_off, total;
};

template <typename T>
__global__ void __launch_bounds__(kGatherThreads)
embed_gather_bulk_kernel(const T *table, const int32_t *ids, const float *pe, T *__restrict__ out, int num_tokens,
                         int vocab, int d, int stride_s, GatherBulkLayout L, unsigned int *timeouts) {
  pdl_prologue();
  using S = Store<T>;
  constexpr int E = S::kPerVec;
  constexpr int kMaxVec = 4;  // column vectors per consumer thread (rows of up to 1024 vectors)
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char *ring = smem_raw;
  float *pe_buf = reinterpret_cast<float *>(smem_raw + L.pe_off);       // two rows
  uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw + L.bar_off);  // [stages]
  uint64_t *empty = full + 16;                                          // [stages]
  uint64_t *pe_full = empty + 16;                                       // [2]
  uint64_t *pe_empty = pe_full + 2;                                     // [2]
  volatile int *dead = reinterpret_cast<volatile int *>(pe_empty + 2);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int stages = L.stages;
  const int ncv = d / E;
  if (tid == 0) {
    for (int i = 0; i < stages; i++) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], kGatherConsumers / 32);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(&pe_full[i], 1);
      mbar_init(&pe_empty[i], kGatherConsumers / 32);
    }
    *dead = 0;
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == kGatherConsumers / 32) {
    // ---------------------------------------------------------------- producer
    int it = 0, pit = 0;
    for (int s = blockIdx.x; s < stride_s; s += gridDim.x, ++pit) {
      const int nb = (num_tokens - s + stride_s - 1) / stride_s;  // tokens that share position s
      if (lane == 0) {
        mbar_wait(&pe_empty[pit & 1], ((pit >> 1) & 1) ^ 1, dead, timeouts);
        mbar_expect_tx(&pe_full[pit & 1], L.pe_bytes);
        bulk_load(pe_buf + static_cast<size_t>(pit & 1) * d, pe + static_cast<size_t>(s) * d, L.pe_bytes, &pe_full[pit & 1]);
      }
      for (int b0 = 0; b0 < nb; b0 += 32) {
        int id = 0;
        if (b0 + lane < nb) {
          id = ld_co(ids + s + static_cast<size_t>(b0 + lane) * stride_s);
          id = max(0, min(id, vocab - 1));  // out-of-range ids cannot leave the table
        }
        const int here = min(32, nb - b0);
        for (int b = 0; b < here; b++, ++it) {
          const int row = __shfl_sync(0xffffffffu, id, b);
          if (lane == 0) {
            const int st = it % stages;
            mbar_wait(&empty[st], ((it / stages) & 1) ^ 1, dead, timeouts);
            mbar_expect_tx(&full[st], L.row_bytes);
            bulk_load(ring + static_cast<size_t>(st) * L.row_bytes, table + static_cast<size_t>(row) * d, L.row_bytes,
                      &full[st]);
          }
        }
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumers
  int it = 0, pit = 0;
  for (int s = blockIdx.x; s < stride_s; s += gridDim.x, ++pit) {
    const int nb = (num_tokens - s + stride_s - 1) / stride_s;
    float pv[kMaxVec][E];
    mbar_wait(&pe_full[pit & 1], (pit >> 1) & 1, dead, timeouts);
    {
      const float *prow = pe_buf + static_cast<size_t>(pit & 1) * d;
#pragma unroll
      for (int k = 0; k < kMaxVec; k++) {
        const int cv = tid + k * kGatherConsumers;
#pragma unroll
        for (int q = 0; q < E / 4; q++) {
          float4 p4 = make_float4(0.f, 0.f, 0.f, 0.f);
          if (cv < ncv) p4 = *reinterpret_cast<const float4 *>(prow + static_cast<size_t>(cv) * E + 4 * q);
          pv[k][4 * q] = p4.x; pv[k][4 * q + 1] = p4.y; pv[k][4 * q + 2] = p4.z; pv[k][4 * q + 3] = p4.w;
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&pe_empty[pit & 1]);  // the values are in registers now
    for (int b = 0; b < nb; b++, ++it) {
      const int st = it % stages;
      mbar_wait(&full[st], (it / stages) & 1, dead, timeouts);
      const unsigned char *row = ring + static_cast<size_t>(st) * L.row_bytes;
      const size_t t = static_cast<size_t>(s) + static_cast<size_t>(b) * stride_s;
      uint4 raw[kMaxVec];
#pragma unroll
      for (int k = 0; k < kMaxVec; k++) {
        const int cv = tid + k * kGatherConsumers;
        if (cv < ncv) raw[k] = lds128(row + static_cast<size_t>(cv) * 16);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[st]);  // this warp's reads of the stage have returned
#pragma unroll
      for (int k = 0; k < kMaxVec; k++) {
        const int cv = tid + k * kGatherConsumers;
        if (cv < ncv) {
          float v[E];
          S::unpack(raw[k], v);
#pragma unroll
          for (int e = 0; e < E; e++) v[e] = v[e] + pv[k][e];
          st_stream(out + t * d + static_cast<size_t>(cv) * E, S::pack(v));
        }
      }
    }
  }
  // After a wait gave up, copies may still be landing in this CTA's shared memory.
  if (*dead) {
    for (int i = 0; i < 1000; i++) __nanosleep(1000);
  }
}

// Ring depth and shared-memory layout, or stages == 0 when the shape does not fit this kernel.
template <typename T>
GatherBulkLayout gather_bulk_layout(int d, int ctas_per_sm) {
  constexpr int E = Store<T>::kPerVec;
  GatherBulkLayout L{};
  if (d % E != 0 || d / E > 4 * kGatherConsumers) return L;
  L.row_bytes = static_cast<unsigned>(d * sizeof(T));
  L.pe_bytes = static_cast<unsigned>(d * sizeof(float));
  const size_t budget = (216 * 1024) / ctas_per_sm - 1024;
  const size_t fixed = 2 * static_cast<size_t>(L.pe_bytes) + 512;
  if (fixed + 2 * static_cast<size_t>(L.row_bytes) > budget) return L;
  size_t stages = (budget - fixed) / L.row_bytes;
  L.stages = static_cast<int>(stages > 16 ? 16 : stages);
  L.pe_off = L.row_bytes * L.stages;
  L.bar_off = L.pe_off + 2 * L.pe_bytes;
  L.total = L.bar_off + 512;
  return L;
}

template <typename T>
__global__ void __launch_bounds__(kBlock)
embed_gather_scalar_kernel(const T *table, const int32_t *ids,
                           const float *__restrict__ pe, T *__restrict__ out, int num_tokens,
                           int vocab, int d, int seq_len) {
  pdl_prologue();
  using S = Store<T>;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kBlock + threadIdx.x;
  if (i >= static_cast<int64_t>(num_tokens) * d) return;
  const int t = static_cast<int>(i / d), c = static_cast<int>(i % d);
  int id = ids[t];
  id = max(0, min(id, vocab - 1));
  float v = S::to_float(table[static_cast<size_t>(id) * d + c]);
  if (pe != nullptr) v = v + pe[static_cast<size_t>(t % seq_len) * d + c];
  out[i] = S::from_float(v);
}

// -------------------------------------------------------------------- sort

__global__ void __launch_bounds__(kBlock)
sort_hist_kernel(const uint32_t *keys, int n, int shift, int nblocks,
                 int32_t *__restrict__ block_hist) {
  pdl_prologue();
  __shared__ int hist[kDigits];
  hist[threadIdx.x] = 0;
  __syncthreads();
  const int base = blockIdx.x * kSortTile;
#pragma unroll
  for (int j = 0; j < kSortItems; j++) {
    const int i = base + j * kBlock + threadIdx.x;
    if (i < n) atomicAdd(&hist[(keys[i] >> shift) & 255u], 1);  // integer counts: order-free
  }
  __syncthreads();
  block_hist[threadIdx.x * nblocks + blockIdx.x] = hist[threadIdx.x];
}

// Exclusive scan of `data[0..n)` in place by one CTA of 1024 threads: thread i
// owns a contiguous chunk.  Returns (to every thread) the total.
__device__ int cta_exclusive_scan_inplace(int32_t *data, int n, int *smem /*[33]*/) {
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int per = (n + nthreads - 1) / nthreads;
  const int b = min(n, tid * per), e = min(n, b + per);
  int sum = 0;
  for (int i = b; i < e; i++) sum += data[i];
  // exclusive scan of the per-thread sums
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if ((tid & 31) >= o) incl += t;
  }
  __syncthreads();
  if ((tid & 31) == 31) smem[tid >> 5] = incl;
  __syncthreads();
  if (tid < 32) {
    const int nw = nthreads >> 5;
    int w = tid < nw ? smem[tid] : 0;
    int wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, wi, o);
      if (tid >= o) wi += t;
    }
    smem[tid] = wi - w;  // exclusive warp offsets
    if (tid == 31) smem[32] = wi;
  }
  __syncthreads();
  int run = smem[tid >> 5] + incl - sum;
  const int total = smem[32];
  for (int i = b; i < e; i++) {
    const int v = data[i];
    data[i] = run;
    run += v;
  }
  return total;
}

__global__ void __launch_bounds__(1024) scan_inplace_kernel(int32_t *data, int n) {
  pdl_prologue();
  __shared__ int smem[33];
  cta_exclusive_scan_inplace(data, n, smem);
}

// Stable scatter of one radix pass.  Items are taken in index order: warp w,
// round j, lane l holds item tile + (w*8+j)*32 + l; its rank among equal digits
// is (digits in earlier warps) + (earlier rounds of this warp) + (lower lanes).
__global__ void __launch_bounds__(kBlock)
sort_scatter_kernel(const uint32_t *keys_in, const int32_t *vals_in,
                    uint32_t *__restrict__ keys_out, int32_t *__restrict__ vals_out, int n,
                    int shift, int nblocks, const int32_t *block_base) {
  pdl_prologue();
  constexpr int kWarps = kBlock / 32;
  __shared__ int cnt[kWarps][kDigits];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kWarps * kDigits; i += kBlock) (&cnt[0][0])[i] = 0;
  __syncthreads();

  uint32_t key[kSortItems];
  int32_t val[kSortItems];
  int rank[kSortItems];
  const int base = blockIdx.x * kSortTile + warp * (kSortItems * 32);
#pragma unroll
  for (int j = 0; j < kSortItems; j++) {
    const int i = base + j * 32 + lane;
    const bool ok = i < n;
    key[j] = ok ? keys_in[i] : 0u;
    val[j] = ok ? (vals_in ? vals_in[i] : i) : -1;
    const uint32_t digit = ok ? ((key[j] >> shift) & 255u) : 256u;  // 256: padding lanes
    const uint32_t peers = __match_any_sync(0xffffffffu, digit);
    const int below = __popc(peers & ((1u << lane) - 1u));
    int prev = 0;
    if (ok) prev = cnt[warp][digit];
    __syncwarp();
    if (ok && below == 0) cnt[warp][digit] = prev + __popc(peers);
    __syncwarp();
    rank[j] = prev + below;
  }
  __syncthreads();
  {
    const int dgt = threadIdx.x;  // kBlock == kDigits
    int run = block_base[dgt * nblocks + blockIdx.x];
#pragma unroll
    for (int w = 0; w < kWarps; w++) {
      const int c = cnt[w][dgt];
      cnt[w][dgt] = run;
      run += c;
    }
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < kSortItems; j++) {
    if (val[j] >= 0) {
      const int pos = cnt[warp][(key[j] >> shift) & 255u] + rank[j];
      keys_out[pos] = key[j];
      vals_out[pos] = val[j];
    }
  }
}

// seg_start[v] = first position in the sorted keys whose key is >= v, v in [0,V].
__global__ void __launch_bounds__(kBlock)
segment_start_kernel(const uint32_t *sorted_keys, int n, int vocab,
                     int32_t *__restrict__ seg_start) {
  pdl_prologue();
  const int v = blockIdx.x * kBlock + threadIdx.x;
  if (v > vocab) return;
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (sorted_keys[mid] < static_cast<uint32_t>(v)) lo = mid + 1; else hi = mid;
  }
  seg_start[v] = lo;
}

// One CTA: lists the long rows (more than kSubLen tokens) in ascending id with
// the exclusive prefix of their sub-segment counts.  meta = {n_long, n_sub}.
__global__ void __launch_bounds__(1024)
plan_long_rows_kernel(const int32_t *seg_start, int vocab,
                      int32_t *__restrict__ long_row, int32_t *__restrict__ long_first,
                      int32_t *__restrict__ meta) {
  pdl_prologue();
  __shared__ int wsum[2][33];
  const int tid = threadIdx.x;
  const int per = (vocab + 1023) / 1024;
  const int b = min(vocab, tid * per), e = min(vocab, b + per);
  int nl = 0, ns = 0;
  for (int v = b; v < e; v++) {
    const int c = seg_start[v + 1] - seg_start[v];
    if (c > kSubLen) { nl++; ns += (c + kSubLen - 1) / kSubLen; }
  }
  int il = nl, is = ns;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int tl = __shfl_up_sync(0xffffffffu, il, o);
    const int ts = __shfl_up_sync(0xffffffffu, is, o);
    if ((tid & 31) >= o) { il += tl; is += ts; }
  }
  if ((tid & 31) == 31) { wsum[0][tid >> 5] = il; wsum[1][tid >> 5] = is; }
  __syncthreads();
  if (tid < 32) {
    const int wl = wsum[0][tid], ws = wsum[1][tid];
    int xl = wl, xs = ws;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int tl = __shfl_up_sync(0xffffffffu, xl, o);
      const int ts = __shfl_up_sync(0xffffffffu, xs, o);
      if (tid >= o) { xl += tl; xs += ts; }
    }
    wsum[0][tid] = xl - wl; wsum[1][tid] = xs - ws;
    if (tid == 31) { wsum[0][32] = xl; wsum[1][32] = xs; }
  }
  __syncthreads();
  int li = wsum[0][tid >> 5] + il - nl;
  int si = wsum[1][tid >> 5] + is - ns;
  for (int v = b; v < e; v++) {
    const int c = seg_start[v + 1] - seg_start[v];
    if (c > kSubLen) {
      long_row[li] = v;
      long_first[li] = si;
      li++;
      si += (c + kSubLen - 1) / kSubLen;
    }
  }
  if (tid == 0) {
    meta[0] = wsum[0][32];
    meta[1] = wsum[1][32];
    long_first[wsum[0][32]] = wsum[1][32];
  }
}

// ---------------------------------------------------------------- scatter
// Any d / alignment: one thread per (row, column) walks the row's tokens.
template <typename T>
__global__ void __launch_bounds__(kBlock)
scatter_scalar_kernel(const T *dy, const int32_t *perm,
                      const int32_t *seg_start, float *__restrict__ grad, int vocab,
                      int d) {
  pdl_prologue();
  using S = Store<T>;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kBlock + threadIdx.x;
  if (i >= static_cast<int64_t>(vocab) * d) return;
  const int v = static_cast<int>(i / d), c = static_cast<int>(i % d);
  const int b = seg_start[v], e = seg_start[v + 1];
  float total = 0.f;
  // Same association as the vector path: sub-segments of kSubLen tokens, their sums
  // added inside kCombineSlices contiguous slices, then the slice sums in order.
  if (e - b <= kSubLen) {
    for (int j = b; j < e; j++) total += S::to_float(dy[static_cast<size_t>(perm[j]) * d + c]);
  } else {
    const int pieces = (e - b + kSubLen - 1) / kSubLen;
    const int per = (pieces + kCombineSlices - 1) / kCombineSlices;
    for (int q = 0; q < kCombineSlices; q++) {
      float quarter = 0.f;
      for (int piece = q * per; piece < pieces && piece < (q + 1) * per; piece++) {
        float part = 0.f;
        const int b2 = b + piece * kSubLen, e2 = min(e, b2 + kSubLen);
        for (int j = b2; j < e2; j++) part += S::to_float(dy[static_cast<size_t>(perm[j]) * d + c]);
        quarter += part;
      }
      total = q == 0 ? quarter : total + quarter;
    }
  }
  grad[i] = total;
}

template <typename T>
int gather_typed(const void *table, const int32_t *ids, const float *pe, int seq_len, void *out,
                 int num_tokens, int vocab, int d, cudaStream_t st) {
  constexpr int E = Store<T>::kPerVec;
  const bool vec = d % E == 0 && aligned16(table) && aligned16(out) && (pe == nullptr || aligned16(pe));
  if (vec) {
    const int ncv = d / E;
    const BlockShape bs = shape_for(ncv);
    // Without PE any grouping of tokens works: walk 8 (or, for very many
    // tokens, more) tokens per thread so that grid.y stays within its limit.
    int stride_s = min(seq_len, num_tokens);
    if (pe == nullptr) {
      int64_t per_thread = ceil_div<int64_t>(num_tokens, 65535LL * bs.ty);
      if (per_thread < 8) per_thread = 8;
      stride_s = static_cast<int>(ceil_div<int64_t>(num_tokens, per_thread));
    }
    dim3 grid(ceil_div(ncv, bs.tx), ceil_div(stride_s, bs.ty));
    DLB_REQUIRE(grid.y <= 65535u, DLB_ERR_UNSUPPORTED,
                "embed_gather_fwd: seq_len=%d exceeds %d positions", seq_len, 65535 * bs.ty);
    DLB_REQUIRE(static_cast<int64_t>(num_tokens) + 16LL * stride_s < INT32_MAX, DLB_ERR_UNSUPPORTED,
                "embed_gather_fwd: %d tokens at a stride of %d overflow the token index", num_tokens, stride_s);
    // Which form: the bulk-copy pipeline when a row keeps all of its consumer threads busy (V 32000 x D 4096,
    // each form alone: bf16, 8 x 4096 tokens, 71.7 against 80.1 us; fp32, 16 x 2048 tokens, 122.9 against
    // 129.0 us).  "gather_variant" 1 / 2 asks for one form.
    const int want_form = get_option("gather_variant");
    if (pe != nullptr && (want_form == 2 || (want_form == 0 && ncv >= kGatherConsumers))) {
      const int ctas_per_sm = get_option("gather_bulk_ctas_per_sm") == 1 ? 1 : 2;
      const GatherBulkLayout L = gather_bulk_layout<T>(d, ctas_per_sm);
      unsigned int *timeouts = wait_timeouts_counter();
      if (L.stages >= 2 && timeouts != nullptr) {
        auto kern = embed_gather_bulk_kernel<T>;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(L.total));
        DLB_REQUIRE(e == cudaSuccess, DLB_ERR_CUDA, "embed_gather_fwd: shared memory attribute: %s", cudaGetErrorString(e));
        // Grid: a CTA should move about 450 KB of table rows (measured best for both storage types: fewer,
        // longer-lived CTAs pay for their start-up once, more of them even out the end of the kernel), and
        // there should be at least as many CTAs as fit the GPU.  "gather_bulk_waves" sets the grid in units of
        // the CTAs that fit instead.
        const int resident = ctas_per_sm * sm_count();
        const int64_t per_position = static_cast<int64_t>(ceil_div(num_tokens, stride_s)) * L.row_bytes;
        const int positions_per_cta = static_cast<int>(std::max<int64_t>(1, (450 * 1024) / std::max<int64_t>(per_position, 1)));
        int bgrid = std::max(ceil_div(stride_s, positions_per_cta), std::min(stride_s, resident));
        const int waves = get_option("gather_bulk_waves");
        if (waves >= 1 && waves <= 16) bgrid = waves * resident;
        bgrid = std::min(bgrid, stride_s);
        launch_pdl(kern, bgrid, kGatherThreads, L.total, st, static_cast<const T *>(table), ids, pe, static_cast<T *>(out),
                   num_tokens, vocab, d, stride_s, L, timeouts);
        DLB_LAUNCH_CHECK("embed_gather_bulk");
        return DLB_OK;
      }
    }
    // Rows in flight per thread: four (six CTAs fit an SM) unless asked otherwise.
    if (get_option("gather_rows_in_flight") == 8 && ceil_div(num_tokens, stride_s) > 4)
      launch_pdl(embed_gather_kernel<T, 8>, grid, dim3(bs.tx, bs.ty), 0, st, static_cast<const T *>(table), ids, pe,
                 static_cast<T *>(out), num_tokens, vocab, d, stride_s);
    else
      launch_pdl(embed_gather_kernel<T, 4>, grid, dim3(bs.tx, bs.ty), 0, st, static_cast<const T *>(table), ids, pe,
                 static_cast<T *>(out), num_tokens, vocab, d, stride_s);
    DLB_LAUNCH_CHECK("embed_gather");
    return DLB_OK;
  }
  const int64_t total = static_cast<int64_t>(num_tokens) * d;
  launch_pdl(embed_gather_scalar_kernel<T>, static_cast<unsigned>(ceil_div<int64_t>(total, kBlock)), kBlock, 0, st, 
      static_cast<const T *>(table), ids, pe, static_cast<T *>(out), num_tokens, vocab, d, seq_len);
  DLB_LAUNCH_CHECK("embed_gather_scalar");
  return DLB_OK;
}

// Dense gradient of the table from the plan of dlb_embed_sort_tokens.
template <typename T>
int scatter_typed(const Plan &p, const void *dy, float *grad, int vocab, int d, cudaStream_t st) {
  constexpr int E = Store<T>::kPerVec;
  const int32_t *perm = p.vals[p.passes & 1];
  // bf16 input: rows of grad and scratch are written 32 bytes at a time (d % 8 == 0 makes row starts 32-byte aligned).
  const bool vec = d % E == 0 && aligned16(dy) && (E == 8 ? aligned32(grad) : aligned16(grad));
  if (!vec) {
    const int64_t total = static_cast<int64_t>(vocab) * d;
    launch_pdl(scatter_scalar_kernel<T>, static_cast<unsigned>(ceil_div<int64_t>(total, kBlock)), kBlock, 0, st,
               static_cast<const T *>(dy), perm, p.seg_start, grad, vocab, d);
    DLB_LAUNCH_CHECK("scatter_scalar");
    return DLB_OK;
  }
  ScatterArgs a{};
  a.perm = perm;
  a.seg_b = p.seg_start;
  a.seg_e = p.seg_start + 1;
  a.long_row = p.long_row;
  a.long_first = p.long_first;
  a.long_b = p.seg_start;
  a.long_e = p.seg_start + 1;
  a.meta = p.meta;
  a.scratch = p.scratch;
  a.out = grad;
  a.out_rows = vocab;
  a.contiguous = 1;
  a.d = d;
  return launch_scatter_rows<T>(dy, a, p.max_sub, 0, st);
}

bool embed_args_ok(int num_tokens, int vocab, int d) {
  return num_tokens >= 0 && vocab > 0 && d > 0 &&
         static_cast<int64_t>(vocab) * d <= INT64_MAX / 8;
}

}  // namespace
}  // namespace dlb

using namespace dlb;

extern "C" int dlb_embed_gather_fwd(const void *table, const int32_t *ids, const float *pe,
                                    int seq_len, void *out, int num_tokens, int vocab, int d,
                                    int dtype, void *stream) {
  DLB_REQUIRE(embed_args_ok(num_tokens, vocab, d), DLB_ERR_INVALID_ARG,
              "embed_gather_fwd: tokens=%d vocab=%d d=%d", num_tokens, vocab, d);
  DLB_REQUIRE(pe == nullptr || seq_len > 0, DLB_ERR_INVALID_ARG,
              "embed_gather_fwd: seq_len=%d with a PE table", seq_len);
  if (num_tokens == 0) return DLB_OK;
  DLB_REQUIRE(table && ids && out, DLB_ERR_INVALID_ARG, "embed_gather_fwd: null pointer");
  if (dtype == DLB_F32)
    return gather_typed<float>(table, ids, pe, seq_len, out, num_tokens, vocab, d, as_stream(stream));
  if (dtype == DLB_BF16)
    return gather_typed<__nv_bfloat16>(table, ids, pe, seq_len, out, num_tokens, vocab, d,
                                       as_stream(stream));
  set_error("embed_gather_fwd: unknown dtype %d", dtype);
  return DLB_ERR_INVALID_ARG;
}

extern "C" size_t dlb_embed_workspace_bytes(int num_tokens, int vocab, int d) {
  if (!embed_args_ok(num_tokens, vocab, d)) return 0;
  return make_plan(nullptr, num_tokens, vocab, d).bytes;
}

extern "C" int dlb_embed_sort_tokens(const int32_t *ids, void *workspace, size_t workspace_bytes,
                                     int num_tokens, int vocab, int d, void *stream) {
  DLB_REQUIRE(embed_args_ok(num_tokens, vocab, d), DLB_ERR_INVALID_ARG,
              "embed_sort_tokens: tokens=%d vocab=%d d=%d", num_tokens, vocab, d);
  DLB_REQUIRE(workspace && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0 &&
                  workspace_bytes >= dlb_embed_workspace_bytes(num_tokens, vocab, d),
              DLB_ERR_WORKSPACE, "embed_sort_tokens: 256-byte aligned workspace of %zu bytes required",
              dlb_embed_workspace_bytes(num_tokens, vocab, d));
  DLB_REQUIRE(ids || num_tokens == 0, DLB_ERR_INVALID_ARG, "embed_sort_tokens: null ids");
  cudaStream_t st = as_stream(stream);
  const Plan p = make_plan(workspace, num_tokens, vocab, d);
  if (num_tokens <= kClusterPlanMaxTokens) {
    // One launch: an 8-CTA cluster runs every phase of the plan.
    ClusterPlanArgs a{};
    a.ids = reinterpret_cast<const uint32_t *>(ids);
    a.keys[0] = p.keys[0]; a.keys[1] = p.keys[1];
    a.vals[0] = p.vals[0]; a.vals[1] = p.vals[1];
    a.seg_start = p.seg_start; a.long_row = p.long_row; a.long_first = p.long_first; a.meta = p.meta;
    a.num_tokens = num_tokens; a.vocab = vocab; a.passes = p.passes; a.sub_len = kSubLen;
    cudaError_t e = cudaFuncSetAttribute(embed_plan_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kClusterPlanSmem));
    DLB_REQUIRE(e == cudaSuccess, DLB_ERR_CUDA, "embed_sort_tokens: shared memory attribute: %s",
                cudaGetErrorString(e));
    // Plain launch: this kernel must not overlap its neighbours (see the kernel's first lines).
    launch_plain(embed_plan_cluster_kernel, kClusterCtas, kClusterThreads, kClusterPlanSmem, st, a);
    DLB_LAUNCH_CHECK("embed_plan_cluster");
    return DLB_OK;
  }
  const uint32_t *kin = reinterpret_cast<const uint32_t *>(ids);
  const int32_t *vin = nullptr;
  for (int pass = 0; pass < p.passes && num_tokens > 0; pass++) {
    const int shift = 8 * pass;
    uint32_t *kout = p.keys[(pass + 1) & 1];
    int32_t *vout = p.vals[(pass + 1) & 1];
    launch_pdl(sort_hist_kernel, p.nblocks, kBlock, 0, st, kin, num_tokens, shift, p.nblocks, p.block_hist);
    DLB_LAUNCH_CHECK("sort_hist");
    launch_pdl(scan_inplace_kernel, 1, 1024, 0, st, p.block_hist, kDigits * p.nblocks);
    DLB_LAUNCH_CHECK("sort_scan");
    launch_pdl(sort_scatter_kernel, p.nblocks, kBlock, 0, st, kin, vin, kout, vout, num_tokens, shift,
                                                      p.nblocks, p.block_hist);
    DLB_LAUNCH_CHECK("sort_scatter");
    kin = kout;
    vin = vout;
  }
  launch_pdl(segment_start_kernel, ceil_div(vocab + 1, kBlock), kBlock, 0, st, 
      p.keys[p.passes & 1], num_tokens, vocab, p.seg_start);
  DLB_LAUNCH_CHECK("segment_start");
  launch_pdl(plan_long_rows_kernel, 1, 1024, 0, st, p.seg_start, vocab, p.long_row, p.long_first, p.meta);
  DLB_LAUNCH_CHECK("plan_long_rows");
  return DLB_OK;
}

extern "C" int dlb_embed_scatter_bwd(const void *dy, const int32_t *ids, float *grad,
                                     void *workspace, size_t workspace_bytes, int num_tokens,
                                     int vocab, int d, int dtype, void *stream) {
  (void)ids;
  DLB_REQUIRE(embed_args_ok(num_tokens, vocab, d), DLB_ERR_INVALID_ARG,
              "embed_scatter_bwd: tokens=%d vocab=%d d=%d", num_tokens, vocab, d);
  DLB_REQUIRE(grad, DLB_ERR_INVALID_ARG, "embed_scatter_bwd: null grad");
  DLB_REQUIRE(workspace && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0 &&
                  workspace_bytes >= dlb_embed_workspace_bytes(num_tokens, vocab, d),
              DLB_ERR_WORKSPACE, "embed_scatter_bwd: 256-byte aligned workspace of %zu bytes required",
              dlb_embed_workspace_bytes(num_tokens, vocab, d));
  DLB_REQUIRE(dy || num_tokens == 0, DLB_ERR_INVALID_ARG, "embed_scatter_bwd: null dy");
  const Plan p = make_plan(workspace, num_tokens, vocab, d);
  if (dtype == DLB_F32) return scatter_typed<float>(p, dy, grad, vocab, d, as_stream(stream));
  if (dtype == DLB_BF16) return scatter_typed<__nv_bfloat16>(p, dy, grad, vocab, d, as_stream(stream));
  set_error("embed_scatter_bwd: unknown dtype %d", dtype);
  return DLB_ERR_INVALID_ARG;
}
