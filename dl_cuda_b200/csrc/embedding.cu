// Token embedding for sm_100a: the gather with the sinusoidal positional-
// encoding add folded in, and the gradient of the table as a deterministic
// sorted-segment sum (no atomics, no memset).
//
// Backward in three steps.
//  1. dlb_embed_sort_tokens: a stable LSD radix sort of (id, token index) pairs
//     (8-bit digits, 2048-token tiles, warp match-any ranking), then per id the
//     start of its run in the sorted list (binary search), then the list of
//     "long" ids (more than kSubLen tokens) with their sub-segment offsets.
//  2. scatter_rows_kernel: one thread group per table row.  A row with at most
//     kSubLen tokens is summed in ascending token order and written once (zero
//     if no token refers to it).  Long rows are cut into sub-segments of
//     kSubLen tokens, each summed by its own thread group into a scratch row.
//  3. combine_long_kernel: adds a long row's scratch rows: 8 contiguous slices of
//     the sub-segments are summed in order, then the 8 slice sums in order.
// The order of every addition is a function of ids alone, so two runs give the
// same bits whatever the scheduling.
#include "common.cuh"
#include "embed_plan_cluster.cuh"

namespace dlb {
namespace {

constexpr int kBlock = 256;
constexpr int kSubLen = 32;  // tokens per sub-segment of a long row

// ------------------------------------------------------------------ gather
// blockDim = (tx, ty): tx threads cover tx column vectors, ty positions per
// CTA.  A thread keeps the PE vector of its (position, column) and walks the
// tokens that share the position (t = s, s+S, s+2S, ...), four gathers in flight.
template <typename T>
__global__ void __launch_bounds__(kBlock)
embed_gather_kernel(const T *table, const int32_t *ids,
                    const float *__restrict__ pe, T *__restrict__ out, int num_tokens, int vocab,
                    int d, int stride_s) {
  pdl_prologue();
  using S = Store<T>;
  constexpr int E = S::kPerVec;
  constexpr int U = 4;
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
  for (int t0 = s; t0 < num_tokens; t0 += U * stride_s) {
    uint4 row[U];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int t = t0 + u * stride_s;
      ok[u] = t < num_tokens;
      if (ok[u]) {
        int id = ld_co(ids + t);
        id = max(0, min(id, vocab - 1));  // out-of-range ids cannot leave the table
        row[u] = ld_keep(table + static_cast<size_t>(id) * d + cv * E);
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
constexpr int kSortItems = 8;                        // keys per thread
constexpr int kSortTile = kBlock * kSortItems;       // 2048 tokens per CTA
constexpr int kDigits = 256;

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
struct Plan {
  uint32_t *keys[2];
  int32_t *vals[2];
  int32_t *block_hist;
  int32_t *seg_start;   // [V+1]
  int32_t *long_row;    // [max_long]
  int32_t *long_first;  // [max_long+1]
  int32_t *meta;        // {n_long, n_sub}
  float *scratch;       // [max_sub][d]
  int passes, nblocks, max_long, max_sub;
  size_t bytes;
};

size_t align_up(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

Plan make_plan(void *workspace, int num_tokens, int vocab, int d) {
  Plan p{};
  int bits = 1;
  while (bits < 32 && (static_cast<uint64_t>(1) << bits) < static_cast<uint64_t>(vocab)) bits++;
  p.passes = (bits + 7) / 8;
  p.nblocks = ceil_div(num_tokens, kSortTile);
  // A long row has more than kSubLen tokens, so there are fewer than T/kSubLen of
  // them, and their sub-segments number at most T/kSubLen + (number of long rows).
  p.max_long = num_tokens / kSubLen + 1;
  p.max_sub = 2 * (num_tokens / kSubLen) + 2;
  char *base = static_cast<char *>(workspace);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    char *ptr = base ? base + off : nullptr;
    off += align_up(bytes);
    return ptr;
  };
  const size_t tok = sizeof(int32_t) * static_cast<size_t>(num_tokens);
  p.keys[0] = reinterpret_cast<uint32_t *>(take(tok));
  p.keys[1] = reinterpret_cast<uint32_t *>(take(tok));
  p.vals[0] = reinterpret_cast<int32_t *>(take(tok));
  p.vals[1] = reinterpret_cast<int32_t *>(take(tok));
  p.block_hist = reinterpret_cast<int32_t *>(take(sizeof(int32_t) * kDigits * p.nblocks));
  p.seg_start = reinterpret_cast<int32_t *>(take(sizeof(int32_t) * (static_cast<size_t>(vocab) + 1)));
  p.long_row = reinterpret_cast<int32_t *>(take(sizeof(int32_t) * p.max_long));
  p.long_first = reinterpret_cast<int32_t *>(take(sizeof(int32_t) * (p.max_long + 1)));
  p.meta = reinterpret_cast<int32_t *>(take(sizeof(int32_t) * 4));
  p.scratch = reinterpret_cast<float *>(take(sizeof(float) * static_cast<size_t>(p.max_sub) * d));
  p.bytes = off;
  return p;
}

// Sum of the dy rows tok(b) .. tok(e-1) over this thread's KV column vectors, in order.
template <typename T, int KV, typename Tok>
__device__ __forceinline__ void sum_tokens(const T *dy, Tok tok, int b, int e, int d, int cv0,
                                           int tx, int ncv, float (&acc)[KV][Store<T>::kPerVec]) {
  using S = Store<T>;
  constexpr int E = S::kPerVec;
#pragma unroll
  for (int k = 0; k < KV; k++)
#pragma unroll
    for (int q = 0; q < E; q++) acc[k][q] = 0.f;
  // UNR token rows in flight per step; the additions stay in token order.
  constexpr int UNR = KV >= 2 ? 2 : 4;
  int j = b;
  for (; j + UNR <= e; j += UNR) {
    uint4 v[UNR][KV];
#pragma unroll
    for (int u = 0; u < UNR; u++) {
      const size_t r = static_cast<size_t>(tok(j + u)) * d;
#pragma unroll
      for (int k = 0; k < KV; k++) {
        const int cv = cv0 + k * tx;
        if (cv < ncv) v[u][k] = ld_stream(dy + r + static_cast<size_t>(cv) * E);
      }
    }
#pragma unroll
    for (int u = 0; u < UNR; u++)
#pragma unroll
      for (int k = 0; k < KV; k++) {
        if (cv0 + k * tx < ncv) {
          float f[E];
          S::unpack(v[u][k], f);
#pragma unroll
          for (int q = 0; q < E; q++) acc[k][q] += f[q];
        }
      }
  }
  for (; j < e; j++) {
    const size_t r0 = static_cast<size_t>(tok(j)) * d;
#pragma unroll
    for (int k = 0; k < KV; k++) {
      const int cv = cv0 + k * tx;
      if (cv < ncv) {
        float f0[E];
        S::unpack(ld_stream(dy + r0 + static_cast<size_t>(cv) * E), f0);
#pragma unroll
        for (int q = 0; q < E; q++) acc[k][q] += f0[q];
      }
    }
  }
}

template <typename T, int KV>
__device__ __forceinline__ void store_row(float *dst, int cv0, int tx, int ncv,
                                          const float (&acc)[KV][Store<T>::kPerVec]) {
  constexpr int E = Store<T>::kPerVec;
#pragma unroll
  for (int k = 0; k < KV; k++) {
    const int cv = cv0 + k * tx;
    if (cv < ncv) {
      if constexpr (E == 8) {
        // dst rows are 32-byte aligned (checked on the host: base and d*4 are)
        st_stream32(dst + static_cast<size_t>(cv) * E, acc[k]);
      } else {
#pragma unroll
        for (int q = 0; q < E / 4; q++) {
          const uint4 o = make_uint4(__float_as_uint(acc[k][4 * q]), __float_as_uint(acc[k][4 * q + 1]),
                                     __float_as_uint(acc[k][4 * q + 2]), __float_as_uint(acc[k][4 * q + 3]));
          st_stream(dst + static_cast<size_t>(cv) * E + 4 * q, o);
        }
      }
    }
  }
}

// blockDim = (tx, ty).  grid.x = sub_groups + row_groups; grid.y tiles columns
// when a row has more than tx*KV vectors.  The sub-segment groups come first so
// that the heaviest work starts first.  A row group is kScatterRowsPerCta (or ty,
// if larger) consecutive table rows: the CTA fetches their segment bounds and the
// token list they share (consecutive rows are consecutive in the sorted list)
// into shared memory once, then each thread row walks its rows, so the only
// dependent global access left per row is the dy load itself.
constexpr int kScatterRowsPerCta = 16;
constexpr int kScatterPermCap = 1024;

// Multi-GPU "peer" output: output row r (a slot of the compacted row list) belongs to rank
// r % n, which sums it.  A rank that has tokens for the row stores its partial sum straight into
// the owner's receive area, laid out [source rank][r / n][d], through the owner's peer mapping;
// rows without local tokens are not sent (the receive area is zero where nothing arrives).
struct PeerOut {
  float *recv[kMaxPeers];  // every rank's receive area as mapped into this GPU's address space
  const int32_t *used;     // device word holding the number of used rows (the compact plan's header)
  int n, me, cap;          // ranks, this rank, rows per source in a receive area
};

template <bool PEER>
__device__ __forceinline__ float *out_row_ptr(float *grad, const PeerOut &po, int r, int d) {
  if constexpr (PEER) {
    return po.recv[r % po.n] + (static_cast<size_t>(po.me) * po.cap + r / po.n) * d;
  } else {
    return grad + static_cast<size_t>(r) * d;
  }
}

template <typename T, int KV, bool PEER>
__global__ void __launch_bounds__(kBlock)
scatter_rows_kernel(const T *dy, const int32_t *perm,
                    const int32_t *seg_start, const int32_t *long_row,
                    const int32_t *long_first, const int32_t *meta,
                    float *__restrict__ grad, float *__restrict__ scratch, int vocab, int d,
                    int sub_groups, const int32_t *row_begin,
                    const int32_t *row_end, int rows_cta, const __grid_constant__ PeerOut po) {
  pdl_prologue();
  using S = Store<T>;
  constexpr int E = S::kPerVec;
  __shared__ int s_b[kBlock], s_e[kBlock];
  __shared__ int s_perm[kScatterPermCap];
  const int tx = blockDim.x, ty = blockDim.y;
  const int ncv = d / E;
  const int cv0 = blockIdx.y * (tx * KV) + threadIdx.x;
  float acc[KV][E];
  if (static_cast<int>(blockIdx.x) < sub_groups) {
    const int n_long = meta[0], n_sub = meta[1];
    for (int idx = blockIdx.x * ty + threadIdx.y; idx < n_sub; idx += sub_groups * ty) {
      int lo = 0, hi = n_long;  // last long row whose first sub-segment is <= idx
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (long_first[mid] <= idx) lo = mid; else hi = mid;
      }
      const int v = long_row[lo];
      const int b = seg_start[v] + (idx - long_first[lo]) * kSubLen;
      const int e = min(seg_start[v + 1], b + kSubLen);
      sum_tokens<T, KV>(dy, [&](int j) { return ld_co(perm + j); }, b, e, d, cv0, tx, ncv, acc);
      store_row<T, KV>(scratch + static_cast<size_t>(idx) * d, cv0, tx, ncv, acc);
    }
    return;
  }
  const int v_first = (blockIdx.x - sub_groups) * rows_cta;
  // Peer mode: the host may have sized the grid from an upper bound of the used rows (it need not
  // wait for the plan); the exact count is read here and surplus CTAs leave.
  if constexpr (PEER) {
    vocab = min(vocab, ld_co(po.used));
    if (v_first >= vocab) return;
  }
  // Output row r takes the sorted tokens [begin, end).  Dense mode: r is the table row and the
  // range is seg_start[r], seg_start[r+1].  Compact mode (row_begin given): r is a slot of the
  // compacted row list, `vocab` is the number of slots, and the ranges come from row_begin/end.
  const int nrows = min(rows_cta, vocab - v_first);
  const int tid = threadIdx.y * tx + threadIdx.x;
  const bool compact = row_begin != nullptr;
  for (int i = tid; i < nrows; i += kBlock) {
    s_b[i] = compact ? ld_co(row_begin + v_first + i) : ld_co(seg_start + v_first + i);
    s_e[i] = compact ? ld_co(row_end + v_first + i) : ld_co(seg_start + v_first + i + 1);
  }
  __syncthreads();
  const int p0 = s_b[0], np = s_e[nrows - 1] - p0;
  const bool staged = !compact && np <= kScatterPermCap;
  if (staged)
    for (int i = tid; i < np; i += kBlock) s_perm[i] = ld_co(perm + p0 + i);
  __syncthreads();
  // Rows with no token or one token (nearly all of them): U rows at a time, every
  // load of the U rows issued before the first store, so that U*KV 16-byte loads per
  // thread are in flight.  A row's sum is still 0.0f + dy (the same bits as the
  // general path below).
  constexpr int U = KV >= 4 ? 2 : 4;
  for (int rl0 = threadIdx.y; rl0 < nrows; rl0 += ty * U) {
    uint4 v[U][KV];
    int state[U];  // -1: not mine or handled below, 0: empty row, 1: one token
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int rl = rl0 + u * ty;
      state[u] = -1;
      if (rl < nrows) {
        const int b = s_b[rl], cnt = s_e[rl] - b;
        if (cnt <= 1) state[u] = cnt;
        if (cnt == 1) {
          const int t = staged ? s_perm[b - p0] : ld_co(perm + b);
          const T *src = dy + static_cast<size_t>(t) * d;
#pragma unroll
          for (int k = 0; k < KV; k++) {
            const int cv = cv0 + k * tx;
            if (cv < ncv) v[u][k] = ld_stream(src + static_cast<size_t>(cv) * E);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      if (state[u] < 0) continue;
      if (PEER && state[u] == 0) continue;  // nothing to send for a row without local tokens
#pragma unroll
      for (int k = 0; k < KV; k++) {
#pragma unroll
        for (int q = 0; q < E; q++) acc[k][q] = 0.f;
        if (state[u] == 1 && cv0 + k * tx < ncv) {
          float f[E];
          S::unpack(v[u][k], f);
#pragma unroll
          for (int q = 0; q < E; q++) acc[k][q] += f[q];
        }
      }
      store_row<T, KV>(out_row_ptr<PEER>(grad, po, v_first + rl0 + u * ty, d), cv0, tx, ncv, acc);
    }
  }
  // Rows with 2..kSubLen tokens.
  for (int rl = threadIdx.y; rl < nrows; rl += ty) {
    const int b = s_b[rl], e = s_e[rl];
    if (e - b < 2 || e - b > kSubLen) continue;  // long rows are written by combine_long_kernel
    if (staged)
      sum_tokens<T, KV>(dy, [&](int j) { return s_perm[j - p0]; }, b, e, d, cv0, tx, ncv, acc);
    else
      sum_tokens<T, KV>(dy, [&](int j) { return ld_co(perm + j); }, b, e, d, cv0, tx, ncv, acc);
    store_row<T, KV>(out_row_ptr<PEER>(grad, po, v_first + rl, d), cv0, tx, ncv, acc);
  }
}

// grad[v,:] = the scratch rows of long row v.  A work item is (long row, block of
// 32 float4 column vectors); CTAs loop over the items.  Each of the CTA's
// kCombineSlices warps adds one contiguous slice of the row's sub-segments in
// order (512 contiguous bytes per sub-segment), then the slice sums are added in
// warp order through shared memory.
constexpr int kCombineSlices = 8;
static_assert(kCombineSlices * 32 == kBlock, "one warp per slice");

template <bool PEER>
__global__ void __launch_bounds__(kBlock)
combine_long_kernel(const float *scratch, const int32_t *long_row,
                    const int32_t *long_first, const int32_t *meta,
                    float *__restrict__ grad, int d, const int32_t *slot_map,
                    const __grid_constant__ PeerOut po) {
  pdl_prologue();
  __shared__ float4 part[kCombineSlices][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = d / 4;
  const int ncb = (nvec + 31) / 32;  // column blocks per row
  const int items = meta[0] * ncb;
  for (int item = blockIdx.x; item < items; item += gridDim.x) {
    const int li = item / ncb, c = ((item % ncb) * 32 + lane) * 4;
    const int s0 = long_first[li], s1 = long_first[li + 1];
    const int per = (s1 - s0 + kCombineSlices - 1) / kCombineSlices;
    const int b = min(s1, s0 + warp * per), e = min(s1, b + per);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < d) {
#pragma unroll 8
      for (int s = b; s < e; s++) {
        const float4 p = __ldcs(reinterpret_cast<const float4 *>(scratch + static_cast<size_t>(s) * d + c));
        acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
      }
    }
    __syncthreads();  // part[] of the previous item has been read
    part[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && c < d) {
      float4 r = part[0][lane];
#pragma unroll
      for (int k = 1; k < kCombineSlices; k++) {
        const float4 p = part[k][lane];
        r.x += p.x; r.y += p.y; r.z += p.z; r.w += p.w;
      }
      const int v = long_row[li];
      const int out_row = slot_map != nullptr ? slot_map[v] : v;  // compact mode: the row's slot
      __stcs(reinterpret_cast<float4 *>(out_row_ptr<PEER>(grad, po, out_row, d) + c), r);
    }
  }
}

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

struct BlockShape {
  int tx, ty;
};
BlockShape shape_for(int ncv) {
  int tx = 1;
  while (tx < kBlock && tx < ncv) tx *= 2;
  return {tx, kBlock / tx};
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
    launch_pdl(embed_gather_kernel<T>, grid, dim3(bs.tx, bs.ty), 0, st, 
        static_cast<const T *>(table), ids, pe, static_cast<T *>(out), num_tokens, vocab, d, stride_s);
    DLB_LAUNCH_CHECK("embed_gather");
    return DLB_OK;
  }
  const int64_t total = static_cast<int64_t>(num_tokens) * d;
  launch_pdl(embed_gather_scalar_kernel<T>, static_cast<unsigned>(ceil_div<int64_t>(total, kBlock)), kBlock, 0, st, 
      static_cast<const T *>(table), ids, pe, static_cast<T *>(out), num_tokens, vocab, d, seq_len);
  DLB_LAUNCH_CHECK("embed_gather_scalar");
  return DLB_OK;
}

// Where the rows of a multi-GPU (compacted) scatter go: the table rows some rank refers to
// ("used" rows) are numbered 0..used-1 in ascending id; everything lives in one workspace.
struct Compact {
  int32_t *header;     // [4]   {used rows, -, -, -}
  int32_t *slot_map;   // [V]   slot of a table row, -1 if no rank refers to it
  int32_t *used_rows;  // [V]   table row of a slot (first `used` entries)
  int32_t *row_begin;  // [V]   this rank's sorted-token range of a slot
  int32_t *row_end;    // [V]
  size_t bytes;
};

Compact make_compact(void *workspace, int vocab) {
  Compact c{};
  char *base = static_cast<char *>(workspace);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    char *ptr = base ? base + off : nullptr;
    off += align_up(bytes);
    return reinterpret_cast<int32_t *>(ptr);
  };
  const size_t per = sizeof(int32_t) * static_cast<size_t>(vocab);
  c.header = take(sizeof(int32_t) * 4);
  c.slot_map = take(per);
  c.used_rows = take(per);
  c.row_begin = take(per);
  c.row_end = take(per);
  c.bytes = off;
  return c;
}

// One CTA: walks the table rows in order, 1024 at a time; a row is used if the GLOBAL plan
// (the tokens of every rank) has a token for it.  Emits the slot numbering and, per slot, the
// LOCAL plan's token range.
__global__ void __launch_bounds__(1024)
compact_rows_kernel(const int32_t *seg_global, const int32_t *seg_local, int vocab,
                    Compact c) {
  pdl_prologue();
  __shared__ int tmp[33];
  int base = 0;
  for (int v0 = 0; v0 < vocab; v0 += 1024) {
    const int v = v0 + threadIdx.x;
    const int used = (v < vocab && seg_global[v + 1] > seg_global[v]) ? 1 : 0;
    int total;
    const int off = cta_exclusive_scan(used, 1024, tmp, &total);
    if (v < vocab) {
      c.slot_map[v] = used ? base + off : -1;
      if (used) {
        c.used_rows[base + off] = v;
        c.row_begin[base + off] = seg_local[v];
        c.row_end[base + off] = seg_local[v + 1];
      }
    }
    base += total;
  }
  if (threadIdx.x == 0) c.header[0] = base;
}

// grad[v,:] = 0 for rows no rank refers to (what & 1); grad[v,:] = compact[slot_map[v],:] for the
// others (what & 2).  blockDim = (tx, ty): ty rows per step, tx float4 column vectors.
__global__ void __launch_bounds__(kBlock)
expand_rows_kernel(const float *compact, const int32_t *slot_map,
                   float *__restrict__ grad, int vocab, int d, int what, int rows_per_cta) {
  pdl_prologue();
  const int nvec = d / 4;
  const int r0 = blockIdx.x * rows_per_cta;
  const int r1 = min(vocab, r0 + rows_per_cta);
  for (int v = r0 + threadIdx.y; v < r1; v += blockDim.y) {
    const int slot = ld_co(slot_map + v);
    if (slot < 0 ? !(what & 1) : !(what & 2)) continue;
    float4 *dst = reinterpret_cast<float4 *>(grad + static_cast<size_t>(v) * d);
    const float4 *src = reinterpret_cast<const float4 *>(compact + static_cast<size_t>(max(slot, 0)) * d);
    for (int c0 = threadIdx.x; c0 < nvec; c0 += 4 * blockDim.x) {
      float4 val[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int c = c0 + u * blockDim.x;
        val[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (slot >= 0 && c < nvec) val[u] = __ldcs(src + c);
      }
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int c = c0 + u * blockDim.x;
        if (c < nvec) __stcs(dst + c, val[u]);
      }
    }
  }
}

// Second half of the peer exchange, run by the owner of a row.  For each owned slot (slots me,
// me+n, me+2n, ... of the compacted row list) the partial sums that arrived from the n source
// ranks are added in rank order (what did not arrive is zero), the receive rows are put back to
// zero for the next step, and the sum is stored into row used_rows[slot] of EVERY rank's dense
// gradient table through the peer mappings: reduction, broadcast and the expansion into the
// dense layout are one pass.  One CTA per owned slot, a thread owns float4 columns.
struct PeerTables {
  float *grad[kMaxPeers];  // every rank's dense [vocab, d] gradient as mapped into this GPU
  int n, me, cap;
};

__global__ void __launch_bounds__(kBlock)
reduce_broadcast_kernel(float *recv, const int32_t *used_rows, const int32_t *header, int d,
                        const __grid_constant__ PeerTables pt) {
  pdl_prologue();
  const int used = ld_co(header);
  const int nvec = d / 4;
  for (int j = blockIdx.x; pt.me + j * pt.n < used; j += gridDim.x) {
    const int v = ld_co(used_rows + pt.me + j * pt.n);
    for (int c = threadIdx.x; c < nvec; c += kBlock) {
      // every source's cell is loaded before the first add, so the n L2 reads are in flight together
      float4 part[kMaxPeers];
#pragma unroll
      for (int src = 0; src < kMaxPeers; src++) {
        if (src < pt.n) {
          // written by a peer: read at L2, never through L1
          part[src] = __ldcg(reinterpret_cast<const float4 *>(recv + (static_cast<size_t>(src) * pt.cap + j) * d) + c);
        }
      }
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int src = 0; src < kMaxPeers; src++) {
        if (src < pt.n) {
          const float4 p = part[src];
          acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
          const bool nonzero = ((__float_as_uint(p.x) | __float_as_uint(p.y) | __float_as_uint(p.z) |
                                 __float_as_uint(p.w)) << 1) != 0;
          if (nonzero)
            __stcg(reinterpret_cast<float4 *>(recv + (static_cast<size_t>(src) * pt.cap + j) * d) + c,
                   make_float4(0.f, 0.f, 0.f, 0.f));
        }
      }
#pragma unroll
      for (int q = 0; q < kMaxPeers; q++) {
        if (q < pt.n) __stcs(reinterpret_cast<float4 *>(pt.grad[q] + static_cast<size_t>(v) * d) + c, acc);
      }
    }
  }
}

template <typename T, int KV>
int launch_scatter(const Plan &p, const void *dy, const int32_t *perm, float *grad, int out_rows, int d,
                   BlockShape bs, const Compact *compact, const PeerOut *peer, cudaStream_t st) {
  constexpr int E = Store<T>::kPerVec;
  const int ncv = d / E;
  // Sub-segment groups loop over the sub-segments, so a few hundred CTAs cover any count.
  const int sub_groups = min(ceil_div(p.max_sub, bs.ty), 4 * sm_count());
  const int rows_cta = bs.ty > kScatterRowsPerCta ? bs.ty : kScatterRowsPerCta;
  const int row_groups = ceil_div(out_rows, rows_cta);
  dim3 grid(sub_groups + row_groups, ceil_div(ncv, bs.tx * KV));
  const PeerOut none{};
  auto go = [&](auto kern) {
    launch_pdl(kern, grid, dim3(bs.tx, bs.ty), 0, st, static_cast<const T *>(dy), perm, p.seg_start, p.long_row,
               p.long_first, p.meta, grad, p.scratch, out_rows, d, sub_groups,
               compact ? compact->row_begin : nullptr, compact ? compact->row_end : nullptr, rows_cta,
               peer ? *peer : none);
  };
  if (peer) go(scatter_rows_kernel<T, KV, true>);
  else go(scatter_rows_kernel<T, KV, false>);
  DLB_LAUNCH_CHECK("scatter_rows");
  return DLB_OK;
}

// out_rows: table rows (dense) or used rows (compact: `grad` is then the [used, d] buffer).
template <typename T>
int scatter_typed(const Plan &p, const void *dy, float *grad, int out_rows, int d, const Compact *compact,
                  cudaStream_t st, const PeerOut *peer = nullptr) {
  constexpr int E = Store<T>::kPerVec;
  const int32_t *perm = p.vals[p.passes & 1];
  // bf16 input: rows of grad and scratch are written 32 bytes at a time (d % 8 == 0 makes row starts 32-byte aligned).
  const bool vec = d % E == 0 && aligned16(dy) && (E == 8 ? aligned32(grad) : aligned16(grad));
  if (!vec) {
    DLB_REQUIRE(compact == nullptr, DLB_ERR_UNSUPPORTED,
                "embed_scatter_bwd_compact: d must be a multiple of %d and the buffers 32-byte aligned", E);
    const int64_t total = static_cast<int64_t>(out_rows) * d;
    launch_pdl(scatter_scalar_kernel<T>, static_cast<unsigned>(ceil_div<int64_t>(total, kBlock)), kBlock, 0, st,
               static_cast<const T *>(dy), perm, p.seg_start, grad, out_rows, d);
    DLB_LAUNCH_CHECK("scatter_scalar");
    return DLB_OK;
  }
  if (out_rows == 0) return DLB_OK;
  const int ncv = d / E;
  const BlockShape bs = shape_for(ncv);
  const int need = ceil_div(ncv, bs.tx);
  int rc;
  // Four vectors per thread only for bf16 input: with fp32 input that variant needs 122 registers (2 CTAs
  // per SM) and two column halves of two vectors each are faster (V 32000, D 4096: 201 against 226 us).
  if (need >= 4 && E == 8) rc = launch_scatter<T, 4>(p, dy, perm, grad, out_rows, d, bs, compact, peer, st);
  else if (need >= 2) rc = launch_scatter<T, 2>(p, dy, perm, grad, out_rows, d, bs, compact, peer, st);
  else rc = launch_scatter<T, 1>(p, dy, perm, grad, out_rows, d, bs, compact, peer, st);
  if (rc != DLB_OK) return rc;
  const int grid = 8 * sm_count();  // 8 CTAs fit an SM; each loops over (long row, column block) items
  if (peer)
    launch_pdl(combine_long_kernel<true>, grid, kBlock, 0, st, p.scratch, p.long_row, p.long_first, p.meta, grad, d,
               compact->slot_map, *peer);
  else
    launch_pdl(combine_long_kernel<false>, grid, kBlock, 0, st, p.scratch, p.long_row, p.long_first, p.meta, grad, d,
               compact ? compact->slot_map : nullptr, PeerOut{});
  DLB_LAUNCH_CHECK("combine_long");
  return DLB_OK;
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
  if (dtype == DLB_F32) return scatter_typed<float>(p, dy, grad, vocab, d, nullptr, as_stream(stream));
  if (dtype == DLB_BF16)
    return scatter_typed<__nv_bfloat16>(p, dy, grad, vocab, d, nullptr, as_stream(stream));
  set_error("embed_scatter_bwd: unknown dtype %d", dtype);
  return DLB_ERR_INVALID_ARG;
}

// ---- multi-GPU: compacted table gradient ------------------------------------------------------

extern "C" size_t dlb_embed_compact_workspace_bytes(int vocab) {
  if (vocab <= 0) return 0;
  return make_compact(nullptr, vocab).bytes;
}

extern "C" int dlb_embed_compact_plan(const void *global_plan, int global_tokens, const void *local_plan,
                                      int local_tokens, void *compact_ws, size_t compact_bytes, int vocab,
                                      int d, void *stream) {
  DLB_REQUIRE(embed_args_ok(global_tokens, vocab, d) && embed_args_ok(local_tokens, vocab, d),
              DLB_ERR_INVALID_ARG, "embed_compact_plan: bad shape");
  DLB_REQUIRE(global_plan && local_plan && compact_ws && (reinterpret_cast<uintptr_t>(compact_ws) & 255u) == 0 &&
                  compact_bytes >= dlb_embed_compact_workspace_bytes(vocab),
              DLB_ERR_WORKSPACE, "embed_compact_plan: plans and a 256-byte aligned workspace of %zu bytes required",
              dlb_embed_compact_workspace_bytes(vocab));
  const Plan pg = make_plan(const_cast<void *>(global_plan), global_tokens, vocab, d);
  const Plan pl = make_plan(const_cast<void *>(local_plan), local_tokens, vocab, d);
  const Compact c = make_compact(compact_ws, vocab);
  launch_pdl(compact_rows_kernel, 1, 1024, 0, as_stream(stream), pg.seg_start, pl.seg_start, vocab, c);
  DLB_LAUNCH_CHECK("compact_rows");
  return DLB_OK;
}

extern "C" int dlb_embed_scatter_bwd_compact(const void *dy, void *local_plan, size_t local_plan_bytes,
                                             const void *compact_ws, float *compact_rows, int used_rows,
                                             int local_tokens, int vocab, int d, int dtype, void *stream) {
  DLB_REQUIRE(embed_args_ok(local_tokens, vocab, d) && used_rows >= 0 && used_rows <= vocab, DLB_ERR_INVALID_ARG,
              "embed_scatter_bwd_compact: tokens=%d vocab=%d d=%d used_rows=%d", local_tokens, vocab, d, used_rows);
  DLB_REQUIRE(local_plan && compact_ws && local_plan_bytes >= dlb_embed_workspace_bytes(local_tokens, vocab, d),
              DLB_ERR_WORKSPACE, "embed_scatter_bwd_compact: plan workspaces required");
  DLB_REQUIRE((compact_rows && (dy || local_tokens == 0)) || used_rows == 0, DLB_ERR_INVALID_ARG,
              "embed_scatter_bwd_compact: null pointer");
  const Plan p = make_plan(local_plan, local_tokens, vocab, d);
  const Compact c = make_compact(const_cast<void *>(compact_ws), vocab);
  if (dtype == DLB_F32) return scatter_typed<float>(p, dy, compact_rows, used_rows, d, &c, as_stream(stream));
  if (dtype == DLB_BF16)
    return scatter_typed<__nv_bfloat16>(p, dy, compact_rows, used_rows, d, &c, as_stream(stream));
  set_error("embed_scatter_bwd_compact: unknown dtype %d", dtype);
  return DLB_ERR_INVALID_ARG;
}

extern "C" int dlb_embed_expand_rows(const float *compact_rows, const void *compact_ws, float *grad, int vocab,
                                     int d, int what, void *stream) {
  DLB_REQUIRE(vocab > 0 && d > 0 && d % 4 == 0 && (what & 3) != 0 && (what & ~3) == 0, DLB_ERR_INVALID_ARG,
              "embed_expand_rows: vocab=%d d=%d (a multiple of 4) what=%d (1 zero, 2 copy, 3 both)", vocab, d, what);
  DLB_REQUIRE(compact_ws && grad && aligned16(grad) && (!(what & 2) || (compact_rows && aligned16(compact_rows))),
              DLB_ERR_INVALID_ARG, "embed_expand_rows: null or unaligned pointer");
  const Compact c = make_compact(const_cast<void *>(compact_ws), vocab);
  int tx = 1;
  while (tx < kBlock && tx < d / 4) tx *= 2;
  const int ty = kBlock / tx;
  const int rows_per_cta = ty > 8 ? ty : 8;
  launch_pdl(expand_rows_kernel, ceil_div(vocab, rows_per_cta), dim3(tx, ty), 0, as_stream(stream), compact_rows,
             c.slot_map, grad, vocab, d, what, rows_per_cta);
  DLB_LAUNCH_CHECK("expand_rows");
  return DLB_OK;
}

// ---- multi-GPU: table gradient exchanged over peer memory ---------------------------------------

static bool peer_args_ok(int n_ranks, int my_rank, int cap_rows) {
  return n_ranks >= 1 && n_ranks <= kMaxPeers && my_rank >= 0 && my_rank < n_ranks && cap_rows >= 0;
}

extern "C" int dlb_embed_scatter_bwd_peer(const void *dy, void *local_plan, size_t local_plan_bytes,
                                          const void *compact_ws, float *const *h_peer_recv, int n_ranks,
                                          int my_rank, int cap_rows, int used_rows, int local_tokens, int vocab,
                                          int d, int dtype, void *stream) {
  DLB_REQUIRE(embed_args_ok(local_tokens, vocab, d) && used_rows >= 0 && used_rows <= vocab, DLB_ERR_INVALID_ARG,
              "embed_scatter_bwd_peer: tokens=%d vocab=%d d=%d used_rows=%d", local_tokens, vocab, d, used_rows);
  DLB_REQUIRE(peer_args_ok(n_ranks, my_rank, cap_rows) && h_peer_recv, DLB_ERR_INVALID_ARG,
              "embed_scatter_bwd_peer: n_ranks=%d (1..%d) my_rank=%d cap_rows=%d", n_ranks, kMaxPeers, my_rank,
              cap_rows);
  DLB_REQUIRE(static_cast<int64_t>(cap_rows) * n_ranks >= used_rows, DLB_ERR_INVALID_ARG,
              "embed_scatter_bwd_peer: %d rows per source hold fewer than the %d used rows", cap_rows, used_rows);
  DLB_REQUIRE(local_plan && compact_ws && local_plan_bytes >= dlb_embed_workspace_bytes(local_tokens, vocab, d),
              DLB_ERR_WORKSPACE, "embed_scatter_bwd_peer: plan workspaces required");
  DLB_REQUIRE(dy || local_tokens == 0, DLB_ERR_INVALID_ARG, "embed_scatter_bwd_peer: null dy");
  PeerOut po{};
  po.n = n_ranks; po.me = my_rank; po.cap = cap_rows;
  for (int r = 0; r < n_ranks; r++) {
    DLB_REQUIRE(h_peer_recv[r] && aligned32(h_peer_recv[r]), DLB_ERR_INVALID_ARG,
                "embed_scatter_bwd_peer: receive area of rank %d is null or not 32-byte aligned", r);
    po.recv[r] = h_peer_recv[r];
  }
  const Plan p = make_plan(local_plan, local_tokens, vocab, d);
  const Compact c = make_compact(const_cast<void *>(compact_ws), vocab);
  po.used = c.header;
  if (dtype == DLB_F32) return scatter_typed<float>(p, dy, nullptr, used_rows, d, &c, as_stream(stream), &po);
  if (dtype == DLB_BF16)
    return scatter_typed<__nv_bfloat16>(p, dy, nullptr, used_rows, d, &c, as_stream(stream), &po);
  set_error("embed_scatter_bwd_peer: unknown dtype %d", dtype);
  return DLB_ERR_INVALID_ARG;
}

extern "C" int dlb_embed_reduce_broadcast_peer(float *my_recv, const void *compact_ws, float *const *h_peer_grad,
                                               int n_ranks, int my_rank, int cap_rows, int vocab, int d,
                                               void *stream) {
  DLB_REQUIRE(vocab > 0 && d > 0 && d % 4 == 0, DLB_ERR_INVALID_ARG,
              "embed_reduce_broadcast_peer: vocab=%d d=%d (a multiple of 4)", vocab, d);
  DLB_REQUIRE(peer_args_ok(n_ranks, my_rank, cap_rows) && h_peer_grad, DLB_ERR_INVALID_ARG,
              "embed_reduce_broadcast_peer: n_ranks=%d (1..%d) my_rank=%d cap_rows=%d", n_ranks, kMaxPeers, my_rank,
              cap_rows);
  DLB_REQUIRE(my_recv && aligned16(my_recv) && compact_ws, DLB_ERR_INVALID_ARG,
              "embed_reduce_broadcast_peer: null or unaligned pointer");
  PeerTables pt{};
  pt.n = n_ranks; pt.me = my_rank; pt.cap = cap_rows;
  for (int r = 0; r < n_ranks; r++) {
    DLB_REQUIRE(h_peer_grad[r] && aligned16(h_peer_grad[r]), DLB_ERR_INVALID_ARG,
                "embed_reduce_broadcast_peer: gradient table of rank %d is null or unaligned", r);
    pt.grad[r] = h_peer_grad[r];
  }
  if (cap_rows == 0) return DLB_OK;
  const Compact c = make_compact(const_cast<void *>(compact_ws), vocab);
  const int grid = min(cap_rows, 16 * sm_count());
  launch_pdl(reduce_broadcast_kernel, grid, kBlock, 0, as_stream(stream), my_recv, c.used_rows, c.header, d, pt);
  DLB_LAUNCH_CHECK("reduce_broadcast");
  return DLB_OK;
}
