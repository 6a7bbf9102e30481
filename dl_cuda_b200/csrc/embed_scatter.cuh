// The sorted-segment sum behind every form of the embedding-table gradient
// (dense single-GPU, compacted for an all-reduce, routed over peer memory).
//
// Input: a list of token indices sorted by table row ("perm") and, per output
// row, its range of that list.  One launch:
//   * rows with at most kSubLen tokens are summed in ascending token order and
//     written once (zeros where no token refers to the row: no memset);
//   * a row with more tokens is cut into sub-segments of kSubLen tokens, each
//     summed by its own thread group into a scratch row; a second kernel
//     (combine_long_kernel, many CTAs per row) adds a row's scratch rows:
//     kCombineSlices contiguous slices of the sub-segments are summed in order,
//     then the slice sums in order.  Measured alternatives, all slower on B200
//     (V 32000 x D 4096, 32768 Zipf tokens, bf16): the CTA that stores a row's
//     last sub-segment adds them all in the same launch (one CTA cannot keep
//     enough loads in flight for a row of 150 sub-segments: 220 against 156 us);
//     the later row CTAs of the bulk-copy form each take a few (row, column
//     block) items once a per-row counter says the sub-segments are stored (CTAs
//     that hold a shared-memory ring are too few to hide this latency-bound work,
//     the kernel of its own runs 8 CTAs per SM: 160 against 149 us); items of 2 or
//     4 column blocks in the second kernel (161 and 173 against 153 us).
// Every addition's order is a function of the ids alone, so two runs give the
// same bits whatever the scheduling; there are no floating-point atomics.
#pragma once

#include "common.cuh"
#include "tma.cuh"

namespace dlb {

constexpr int kEmbBlock = 256;
constexpr int kSubLen = 32;        // tokens per sub-segment of a long row
constexpr int kCombineSlices = 8;  // slices the sub-segment sums of a long row are added in
constexpr int kScatterRowsPerCta = 16;
constexpr int kScatterPermCap = 1024;

inline size_t align_up256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

// ---- the plan dlb_embed_sort_tokens leaves in its workspace ---------------------------------------
constexpr int kSortItems = 8;                      // keys per thread of a radix pass
constexpr int kSortTile = kEmbBlock * kSortItems;  // 2048 tokens per CTA
constexpr int kDigits = 256;

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

inline Plan make_plan(void *workspace, int num_tokens, int vocab, int d) {
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
    off += align_up256(bytes);
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

// ---- flags between the GPUs of one node (see peer.cu) --------------------------------------------
constexpr int kPeerChannels = 4;

// Announces `epoch` on `channel` to every rank once ALL CTAs of the grid have passed this point:
// each CTA fences its (peer) stores and counts itself; the last one stores the flags with release
// semantics at system scope and puts the counter back to zero.  Every CTA of the grid must call it.
struct PeerSignal {
  uint32_t *flags[kMaxPeers];  // every rank's flag words [kPeerChannels][kMaxPeers]
  int32_t *done;               // device counter, zero at launch
  int n, me, channel;
  uint32_t epoch;
};

__device__ __forceinline__ void signal_when_grid_done(const PeerSignal &s) {
  if (s.done == nullptr) return;
  // The CTA's barrier orders every thread's stores before thread 0's fence, and a fence is cumulative:
  // one system-scope fence per CTA covers them all.  (A fence by every thread was measured: it alone
  // added 40 us to a kernel of 900 CTAs.)
  __syncthreads();
  if (threadIdx.x == 0 && threadIdx.y == 0) {
    __threadfence_system();
    const int total = static_cast<int>(gridDim.x * gridDim.y * gridDim.z);
    const int old = atomicAdd(s.done, 1);
    if (old == total - 1) {
      atomicExch(s.done, 0);
      __threadfence_system();
      for (int r = 0; r < s.n; r++) {
        uint32_t *theirs = s.flags[r] + s.channel * kMaxPeers + s.me;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(s.epoch) : "memory");
      }
    }
  }
}

// Waits (whole CTA) until every rank has announced `epoch` on `channel` in this rank's flag words.
// Bounded by wall-clock time: when it runs out bit `channel` of *status is set and the wait ends.
__device__ __forceinline__ void wait_for_peers(const uint32_t *my_flags, int n, int channel, uint32_t epoch,
                                               unsigned long long limit_ns, uint32_t *status) {
  const int t = threadIdx.y * blockDim.x + threadIdx.x;
  if (my_flags != nullptr && t < n) {
    const uint32_t *mine = my_flags + channel * kMaxPeers + t;
    const unsigned long long start = global_ns();
    for (;;) {
      uint32_t seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
      if (static_cast<int32_t>(seen - epoch) >= 0) break;
      if (global_ns() - start > limit_ns) {
        atomicOr(status, 1u << channel);
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
}

// ---- where a summed row goes when the ranks exchange over peer memory ---------------------------------
// A slot is an entry of the list of table rows some rank uses.  If this rank is the only one with
// tokens for it (src_mask[slot] has just this rank's bit) the finished row is stored into row
// used_rows[slot] of EVERY rank's dense table; otherwise the partial sum goes to the receive area of
// the slot's owner (rank slot % n), laid out [source rank][slot / n][d].
struct PeerRoute {
  float *recv[kMaxPeers];
  float *grad[kMaxPeers];
  const int32_t *used_rows;
  const uint32_t *src_mask;
  uint32_t *status;  // bit 31: a slot did not fit the receive area (cap too small)
  int n, me, cap;
};

struct ScatterArgs {
  const int32_t *perm;         // token indices sorted by table row
  const int32_t *seg_b, *seg_e;  // output row r takes perm[seg_b[r] .. seg_e[r])
  const int32_t *long_row;     // rows with more than kSubLen tokens (as indices into long_b/long_e) ...
  const int32_t *long_first;   // ... and the running count of their sub-segments
  const int32_t *long_b, *long_e;  // range of a long row, indexed by long_row[] entries
  const int32_t *long_out;     // output row of a long row (indexed likewise), or null: the entry itself
  const int32_t *meta;         // {number of long rows, number of sub-segments}
  float *scratch;              // [sub-segments][d]
  float *out;                  // output [out_rows][d]
  const int32_t *out_rows_dev; // device word holding the exact number of output rows, or null
  int out_rows;                // number of output rows, or an upper bound when out_rows_dev is given
  int tok_offset;              // subtracted from every perm value (a rank's first token)
  int skip_empty;              // 1: rows without tokens are not written (their contents are never read)
  int contiguous;              // 1: seg_e[r] == seg_b[r + 1] (the plan of dlb_embed_sort_tokens itself)
  int d, sub_groups, rows_cta;
};

// Sum of the dy rows tok(b) .. tok(e-1) over this thread's KV column vectors, in token order.
// UNR token rows are in flight per step, and the token indices of a step are fetched one step
// ahead: where tok() is a load from global memory (rank plans) the chain per step is then one
// row-load latency instead of index load + row load.
template <typename T, int KV, typename Tok>
__device__ __forceinline__ void sum_tokens(const T *dy, Tok tok, int b, int e, int d, int cv0, int tx, int ncv,
                                           float (&acc)[KV][Store<T>::kPerVec]) {
  using S = Store<T>;
  constexpr int E = S::kPerVec;
#pragma unroll
  for (int k = 0; k < KV; k++)
#pragma unroll
    for (int q = 0; q < E; q++) acc[k][q] = 0.f;
  constexpr int UNR = KV >= 4 ? 2 : 4;
  int next_t[UNR];
#pragma unroll
  for (int u = 0; u < UNR; u++) next_t[u] = b + u < e ? tok(b + u) : 0;
  for (int j = b; j < e; j += UNR) {
    uint4 v[UNR][KV];
#pragma unroll
    for (int u = 0; u < UNR; u++) {
      if (j + u < e) {
        const size_t r = static_cast<size_t>(next_t[u]) * d;
#pragma unroll
        for (int k = 0; k < KV; k++) {
          const int cv = cv0 + k * tx;
          if (cv < ncv) v[u][k] = ld_stream(dy + r + static_cast<size_t>(cv) * E);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNR; u++) next_t[u] = j + UNR + u < e ? tok(j + UNR + u) : 0;
#pragma unroll
    for (int u = 0; u < UNR; u++) {
      if (j + u < e) {
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
    }
  }
}

// One row (this thread's KV vectors of it) to dst.  E == 8 (bf16 input): 32-byte stores.
template <int E, int KV>
__device__ __forceinline__ void store_row(float *dst, int cv0, int tx, int ncv, const float (&acc)[KV][E]) {
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

// blockDim = (tx, ty), tx*ty = kEmbBlock.  grid.x = sub_groups + row CTAs; grid.y tiles columns when
// a row has more than tx*KV vectors.  The sub-segment groups come first so that the heaviest work
// starts first.  A row CTA takes groups of rows_cta consecutive output rows (group index strides
// by the number of row CTAs): it fetches their ranges and the token list they share (consecutive
// rows are consecutive in the sorted list) into shared memory once, then each thread row walks
// its rows, so the only dependent global access left per row is the dy load itself.
template <typename T, int KV>
__global__ void __launch_bounds__(kEmbBlock, KV >= 4 ? 1 : 3)
scatter_rows_kernel(const T *dy, const __grid_constant__ ScatterArgs a) {
  pdl_prologue();
  using S = Store<T>;
  constexpr int E = S::kPerVec;
  __shared__ int s_b[kEmbBlock], s_e[kEmbBlock];
  __shared__ int s_perm[kScatterPermCap];
  const int tx = blockDim.x, ty = blockDim.y;
  const int d = a.d;
  const int ncv = d / E;
  const int cv0 = blockIdx.y * (tx * KV) + threadIdx.x;
  const int tid = threadIdx.y * tx + threadIdx.x;
  const int tok_offset = a.tok_offset;
  float acc[KV][E];

  if (static_cast<int>(blockIdx.x) < a.sub_groups) {
    // ------------------------------------------------ sub-segments of long rows
    const int n_long = ld_co(a.meta), n_sub = ld_co(a.meta + 1);
    for (int base = blockIdx.x * ty; base < n_sub; base += a.sub_groups * ty) {
      const int idx = base + threadIdx.y;
      int lo = 0;
      if (idx < n_sub) {
        int hi = n_long;  // last long row whose first sub-segment is <= idx
        while (hi - lo > 1) {
          const int mid = (lo + hi) >> 1;
          if (ld_co(a.long_first + mid) <= idx) lo = mid; else hi = mid;
        }
        const int li = ld_co(a.long_row + lo);
        const int b = ld_co(a.long_b + li) + (idx - ld_co(a.long_first + lo)) * kSubLen;
        const int e = min(ld_co(a.long_e + li), b + kSubLen);
        sum_tokens<T, KV>(dy, [&](int j) { return ld_co(a.perm + j) - tok_offset; }, b, e, d, cv0, tx, ncv, acc);
        store_row<E, KV>(a.scratch + static_cast<size_t>(idx) * d, cv0, tx, ncv, acc);
      }
    }
  } else {
    // ------------------------------------------------ rows with at most kSubLen tokens
    const int out_rows = a.out_rows_dev != nullptr ? min(a.out_rows, ld_co(a.out_rows_dev)) : a.out_rows;
    const int row_ctas = gridDim.x - a.sub_groups;
    const int rows_cta = a.rows_cta;
    for (int v_first = (blockIdx.x - a.sub_groups) * rows_cta; v_first < out_rows; v_first += row_ctas * rows_cta) {
      const int nrows = min(rows_cta, out_rows - v_first);
      for (int i = tid; i < nrows; i += kEmbBlock) {
        s_b[i] = ld_co(a.seg_b + v_first + i);
        s_e[i] = ld_co(a.seg_e + v_first + i);
      }
      __syncthreads();
      // Dense plan: the ranges of consecutive rows are consecutive in the sorted list, so the CTA's
      // whole token list is one span that is fetched once.  Rank plans leave other ranks' tokens (and
      // empty rows) between the ranges: no staging there.
      const int p0 = s_b[0], np = s_e[nrows - 1] - p0;
      const bool staged = a.contiguous != 0 && np <= kScatterPermCap;
      if (staged)
        for (int i = tid; i < np; i += kEmbBlock) s_perm[i] = ld_co(a.perm + p0 + i) - tok_offset;
      __syncthreads();
      // Rows with no token (most of them) first: pure stores, nothing to wait for.
      if (!a.skip_empty) {
        for (int rl = threadIdx.y; rl < nrows; rl += ty) {
          if (s_e[rl] != s_b[rl]) continue;
#pragma unroll
          for (int k = 0; k < KV; k++)
#pragma unroll
            for (int q = 0; q < E; q++) acc[k][q] = 0.f;
          store_row<E, KV>(a.out + static_cast<size_t>(v_first + rl) * d, cv0, tx, ncv, acc);
        }
      }
      // Rows with one token: U rows at a time, every load of the U rows issued before the first store,
      // so that U*KV 16-byte loads per thread are in flight.  A row's sum is still 0.0f + dy (the same
      // bits as the general path below).
      constexpr int U = KV >= 4 ? 2 : 4;
      for (int rl0 = threadIdx.y; rl0 < nrows; rl0 += ty * U) {
        uint4 v[U][KV];
        bool one[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
          const int rl = rl0 + u * ty;
          one[u] = rl < nrows && s_e[rl] - s_b[rl] == 1;
          if (one[u]) {
            const int b = s_b[rl];
            const int t = staged ? s_perm[b - p0] : ld_co(a.perm + b) - tok_offset;
            const T *src = dy + static_cast<size_t>(t) * d;
#pragma unroll
            for (int k = 0; k < KV; k++) {
              const int cv = cv0 + k * tx;
              if (cv < ncv) v[u][k] = ld_stream(src + static_cast<size_t>(cv) * E);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
          if (!one[u]) continue;
#pragma unroll
          for (int k = 0; k < KV; k++) {
#pragma unroll
            for (int q = 0; q < E; q++) acc[k][q] = 0.f;
            if (cv0 + k * tx < ncv) {
              float f[E];
              S::unpack(v[u][k], f);
#pragma unroll
              for (int q = 0; q < E; q++) acc[k][q] += f[q];
            }
          }
          store_row<E, KV>(a.out + static_cast<size_t>(v_first + rl0 + u * ty) * d, cv0, tx, ncv, acc);
        }
      }
      // Rows with 2..kSubLen tokens.
      for (int rl = threadIdx.y; rl < nrows; rl += ty) {
        const int b = s_b[rl], e = s_e[rl];
        if (e - b < 2 || e - b > kSubLen) continue;  // long rows are written by the sub-segment groups
        // one instance of the loop for both sources of the token list (two cost 40 more registers)
        sum_tokens<T, KV>(dy, [&](int j) { return staged ? s_perm[j - p0] : ld_co(a.perm + j) - tok_offset; }, b, e, d,
                          cv0, tx, ncv, acc);
        store_row<E, KV>(a.out + static_cast<size_t>(v_first + rl) * d, cv0, tx, ncv, acc);
      }
      __syncthreads();  // the staging arrays are refilled by the next group
    }
  }
}

// The same sums as a bulk-copy (TMA) pipeline, the other form of scatter_rows_kernel (rows of up to
// 1024 column vectors that fit the ring; launch_scatter_rows says when it is used).
// A CTA takes up to kBulkJobs jobs: a group of consecutive output rows, or (the first sub_groups
// CTAs) sub-segments of long rows.  It first lists the jobs' token indices in shared memory, then
//   producer warp   lane 0 streams the dy rows of those tokens, job after job, into a ring of
//                   shared-memory stages with cp.async.bulk (completion on mbarriers);
//   consumer warps  store the rows without tokens, then per job add the staged rows in token
//                   order into registers and store the sum once.
// No thread holds a dy row in registers while it is in flight and the producer runs ahead over row
// boundaries, so the bytes in flight are set by the ring depth, not by the register file.  The order
// of every row's additions is the one of scatter_rows_kernel: the two forms give the same bits.
constexpr int kBulkConsumers = 256;
constexpr int kBulkThreads = kBulkConsumers + 32;
constexpr int kBulkJobs = 8;  // measured on B200 (V 32000 x D 4096, 32768 Zipf tokens, bf16): 32 -> 154.6, 16 -> 151, 8 -> 146.5, 4 -> 148.5 us

struct ScatterBulkLayout {
  int stages;
  unsigned row_bytes, bar_off, total;
};

template <typename T, int KV>
__global__ void __launch_bounds__(kBulkThreads)
scatter_rows_bulk_kernel(const T *dy, const __grid_constant__ ScatterArgs a, ScatterBulkLayout L,
                         unsigned int *timeouts) {
  pdl_prologue();
  using S = Store<T>;
  constexpr int E = S::kPerVec;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char *ring = smem_raw;
  uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw + L.bar_off);  // [stages]
  uint64_t *empty = full + 16;                                          // [stages]
  volatile int *dead = reinterpret_cast<volatile int *>(empty + 16);
  __shared__ int s_b[kBulkJobs], s_n[kBulkJobs];  // first token (index into perm) and token count; -1: not this CTA's
  __shared__ float *s_dst[kBulkJobs];
  __shared__ int s_tok[kBulkJobs * kSubLen];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int stages = L.stages;
  const int d = a.d;
  const int ncv = d / E;
  if (tid == 0) {
    for (int i = 0; i < stages; i++) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], kBulkConsumers / 32);
    }
    *dead = 0;
    mbar_fence_init();
  }
  __syncthreads();

  const bool sub_cta = static_cast<int>(blockIdx.x) < a.sub_groups;
  int n_long = 0, n_sub = 0, out_rows = 0, rounds;
  if (sub_cta) {
    n_long = ld_co(a.meta);
    n_sub = ld_co(a.meta + 1);
    // sub-segment blockIdx.x + i * sub_groups is job i; kBulkJobs of them per round
    const int mine = (max(n_sub - static_cast<int>(blockIdx.x), 0) + a.sub_groups - 1) / a.sub_groups;
    rounds = (mine + kBulkJobs - 1) / kBulkJobs;
  } else {
    out_rows = a.out_rows_dev != nullptr ? min(a.out_rows, ld_co(a.out_rows_dev)) : a.out_rows;
    const int row_ctas = gridDim.x - a.sub_groups;
    const int groups = (out_rows + kBulkJobs - 1) / kBulkJobs;
    rounds = (max(groups - static_cast<int>(blockIdx.x - a.sub_groups), 0) + row_ctas - 1) / row_ctas;
  }
  int st = 0;           // ring position, the same sequence in the producer and in every consumer
  unsigned phase = 0;
  for (int round = 0; round < rounds; round++) {
    // ---- the jobs of this round
    if (tid < kBulkJobs) {
      int b = 0, n = -1;
      float *dst = nullptr;
      if (sub_cta) {
        const int idx = blockIdx.x + (round * kBulkJobs + tid) * a.sub_groups;
        if (idx < n_sub) {
          int lo = 0, hi = n_long;  // last long row whose first sub-segment is <= idx
          while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (ld_co(a.long_first + mid) <= idx) lo = mid; else hi = mid;
          }
          const int li = ld_co(a.long_row + lo);
          b = ld_co(a.long_b + li) + (idx - ld_co(a.long_first + lo)) * kSubLen;
          n = min(ld_co(a.long_e + li), b + kSubLen) - b;
          dst = a.scratch + static_cast<size_t>(idx) * d;
        }
      } else {
        const int row_ctas = gridDim.x - a.sub_groups;
        const int r = ((blockIdx.x - a.sub_groups) + round * row_ctas) * kBulkJobs + tid;
        if (r < out_rows) {
          b = ld_co(a.seg_b + r);
          n = ld_co(a.seg_e + r) - b;
          if (n > kSubLen || (n == 0 && a.skip_empty)) n = -1;  // long rows are written by the sub-segment CTAs
          dst = a.out + static_cast<size_t>(r) * d;
        }
      }
      s_b[tid] = b;
      s_n[tid] = n;
      s_dst[tid] = dst;
    }
    __syncthreads();
    for (int slot = tid; slot < kBulkJobs * kSubLen; slot += kBulkThreads) {
      const int j = slot / kSubLen, k = slot % kSubLen;
      if (k < s_n[j]) s_tok[slot] = ld_co(a.perm + s_b[j] + k) - a.tok_offset;
    }
    __syncthreads();

    if (warp == kBulkConsumers / 32) {
      // ------------------------------------------------------------ producer
      if (lane == 0) {
        for (int j = 0; j < kBulkJobs; j++) {
          const int n = s_n[j];
          for (int k = 0; k < n; k++) {
            mbar_wait(&empty[st], phase ^ 1, dead, timeouts);
            mbar_expect_tx(&full[st], L.row_bytes);
            bulk_load(ring + static_cast<size_t>(st) * L.row_bytes,
                      dy + static_cast<size_t>(s_tok[j * kSubLen + k]) * d, L.row_bytes, &full[st]);
            if (++st == stages) { st = 0; phase ^= 1; }
          }
        }
      }
    } else {
      // ------------------------------------------------------------ consumers
      float acc[KV][E];
      // Rows with no token (most of them) first: pure stores, nothing to wait for.
      for (int j = 0; j < kBulkJobs; j++) {
        if (s_n[j] != 0) continue;
#pragma unroll
        for (int k = 0; k < KV; k++)
#pragma unroll
          for (int q = 0; q < E; q++) acc[k][q] = 0.f;
        store_row<E, KV>(s_dst[j], tid, kBulkConsumers, ncv, acc);
      }
      for (int j = 0; j < kBulkJobs; j++) {
        const int n = s_n[j];
        if (n <= 0) continue;
#pragma unroll
        for (int k = 0; k < KV; k++)
#pragma unroll
          for (int q = 0; q < E; q++) acc[k][q] = 0.f;
        for (int t = 0; t < n; t++) {
          mbar_wait(&full[st], phase, dead, timeouts);
          const unsigned char *row = ring + static_cast<size_t>(st) * L.row_bytes;
          uint4 raw[KV];
#pragma unroll
          for (int k = 0; k < KV; k++) {
            const int cv = tid + k * kBulkConsumers;
            if (cv < ncv) raw[k] = lds128(row + static_cast<size_t>(cv) * 16);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&empty[st]);  // this warp's reads of the stage have returned
          if (++st == stages) { st = 0; phase ^= 1; }
#pragma unroll
          for (int k = 0; k < KV; k++) {
            if (tid + k * kBulkConsumers < ncv) {
              float f[E];
              S::unpack(raw[k], f);
#pragma unroll
              for (int q = 0; q < E; q++) acc[k][q] += f[q];
            }
          }
        }
        store_row<E, KV>(s_dst[j], tid, kBulkConsumers, ncv, acc);
      }
    }
    // The producer (lanes other than 0 too) must follow the ring position of lane 0.
    if (warp == kBulkConsumers / 32) {
      st = __shfl_sync(0xffffffffu, st, 0);
      phase = __shfl_sync(0xffffffffu, phase, 0);
    }
    __syncthreads();  // the job arrays are refilled by the next round
  }
  // After a wait gave up, copies may still be landing in this CTA's shared memory.
  if (*dead) {
    for (int i = 0; i < 1000; i++) __nanosleep(1000);
  }
}

// Ring depth and shared-memory layout, or stages == 0 when the shape does not fit the kernel.
template <typename T>
ScatterBulkLayout scatter_bulk_layout(int d, int ctas_per_sm) {
  constexpr int E = Store<T>::kPerVec;
  ScatterBulkLayout L{};
  if (d % E != 0 || d / E > 4 * kBulkConsumers) return L;
  L.row_bytes = static_cast<unsigned>(d * sizeof(T));
  const size_t budget = (216 * 1024) / ctas_per_sm - 4096;  // the static arrays take 2.3 KB
  if (2 * static_cast<size_t>(L.row_bytes) + 512 > budget) return L;
  const size_t stages = (budget - 512) / L.row_bytes;
  L.stages = static_cast<int>(stages > 16 ? 16 : stages);
  L.bar_off = L.row_bytes * L.stages;
  L.total = L.bar_off + 512;
  return L;
}

// out[row,:] of every long row = the sum of its scratch rows.  A work item is (long row, block of
// 32 float4 column vectors); CTAs loop over the items.  Each of the CTA's kCombineSlices warps adds
// one contiguous slice of the row's sub-segments in order (512 contiguous bytes per sub-segment),
// then the slice sums are added in warp order through shared memory.
static_assert(kCombineSlices * 32 == kEmbBlock, "one warp per slice");

static __global__ void __launch_bounds__(kEmbBlock) combine_long_kernel(const __grid_constant__ ScatterArgs a) {
  pdl_prologue();
  __shared__ float4 part[kCombineSlices][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int d = a.d;
  const int nvec = d / 4;
  const int ncb = (nvec + 31) / 32;  // column blocks per row
  const int items = ld_co(a.meta) * ncb;
  for (int item = blockIdx.x; item < items; item += gridDim.x) {
    const int row = item / ncb, c = ((item % ncb) * 32 + lane) * 4;
    const int s0 = ld_co(a.long_first + row), s1 = ld_co(a.long_first + row + 1);
    const int per = (s1 - s0 + kCombineSlices - 1) / kCombineSlices;
    const int b = min(s1, s0 + warp * per), e = min(s1, b + per);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < d) {
#pragma unroll 8
      for (int sgm = b; sgm < e; sgm++) {
        const float4 p = __ldcs(reinterpret_cast<const float4 *>(a.scratch + static_cast<size_t>(sgm) * d + c));
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
      const int li = ld_co(a.long_row + row);
      const int out_row = a.long_out != nullptr ? ld_co(a.long_out + li) : li;
      __stcs(reinterpret_cast<float4 *>(a.out + static_cast<size_t>(out_row) * d + c), r);
    }
  }
}

// out[r,:] = 0 for every output row without tokens, as a kernel of its own that runs before the
// summing kernel (which then skips those rows).  An alternative form kept for measurements
// (dlb_set_option "scatter_zero_kernel" = 1): on B200 the two launches took 171 us where the summing
// kernel that also writes the zeros takes 160 us (vocab 32000 x 4096, 32768 Zipf tokens, bf16).
static __global__ void __launch_bounds__(kEmbBlock)
zero_empty_rows_kernel(const int32_t *seg_b, const int32_t *seg_e, float *__restrict__ out, int rows, int d) {
  pdl_prologue();
  const int nv4 = d / 4;
  const int r0 = blockIdx.x * 8;
  int cnt[8];
#pragma unroll
  for (int u = 0; u < 8; u++) cnt[u] = r0 + u < rows ? ld_co(seg_e + r0 + u) - ld_co(seg_b + r0 + u) : 1;
#pragma unroll
  for (int u = 0; u < 8; u++) {
    if (cnt[u] == 0) {
      float4 *dst = reinterpret_cast<float4 *>(out + static_cast<size_t>(r0 + u) * d);
      for (int c = threadIdx.x; c < nv4; c += kEmbBlock) __stcs(dst + c, make_float4(0.f, 0.f, 0.f, 0.f));
    }
  }
}

struct BlockShape {
  int tx, ty;
};
inline BlockShape shape_for(int ncv) {
  int tx = 1;
  while (tx < kEmbBlock && tx < ncv) tx *= 2;
  return {tx, kEmbBlock / tx};
}

// Launches the scatter (and the sum of the long rows) for storage type T.  `max_sub` bounds the number
// of sub-segments the plan can hold; `row_ctas` = 0 means one CTA per group of rows, otherwise that many
// CTAs loop over the groups (for when the exact row count is only known on the device).
template <typename T>
int launch_scatter_rows(const void *dy, ScatterArgs a, int max_sub, int row_ctas, cudaStream_t st) {
  constexpr int E = Store<T>::kPerVec;
  const int ncv = a.d / E;
  const BlockShape bs = shape_for(ncv);
  const int need = ceil_div(ncv, bs.tx);
  // Four vectors per thread only for bf16 input: with fp32 input that variant needs 122 registers (2 CTAs
  // per SM) and two column halves of two vectors each are faster (V 32000, D 4096: 201 against 226 us).
  const int kv = (need >= 4 && E == 8) ? 4 : (need >= 2 ? 2 : 1);
  // Sub-segment groups loop over the sub-segments, so a few hundred CTAs cover any count.
  a.sub_groups = min(ceil_div(max_sub, bs.ty), 4 * sm_count());
  // Rows per CTA: 16 where the rows' token lists are one span fetched once; 4 (one round of the row
  // loop) for a rank plan's rows, which are few and should spread over many CTAs.
  const int want_rows = a.contiguous ? kScatterRowsPerCta : 4;
  a.rows_cta = bs.ty > want_rows ? bs.ty : want_rows;
  const int groups = ceil_div(a.out_rows, a.rows_cta);
  const int row_groups = row_ctas > 0 ? min(groups, row_ctas) : groups;
  dim3 grid(a.sub_groups + row_groups, ceil_div(ncv, bs.tx * kv));
  if (a.contiguous && !a.skip_empty && a.d % 4 == 0 && get_option("scatter_zero_kernel") == 1) {
    launch_pdl(zero_empty_rows_kernel, ceil_div(a.out_rows, 8), kEmbBlock, 0, st, a.seg_b, a.seg_e, a.out, a.out_rows, a.d);
    DLB_LAUNCH_CHECK("zero_empty_rows");
    a.skip_empty = 1;
  }
  // Which form: the bulk-copy pipeline where a dy row keeps all of its consumer threads busy (256 column
  // vectors or more) and the plan is the dense one, whose CTAs each have 8 consecutive rows to work on
  // (V 32000 x D 4096, 32768 Zipf tokens: 147 against 165 us with bf16 input, 190 against 216 us with
  // fp32); rows in registers otherwise.  "scatter_variant" 1 / 2 asks for one form.
  bool launched = false;
  const int want_form = get_option("scatter_variant");
  if (want_form == 2 || (want_form == 0 && a.contiguous && ncv >= kBulkConsumers)) {
    int per_sm = get_option("scatter_bulk_ctas_per_sm");
    if (per_sm < 1 || per_sm > 6) per_sm = 3;
    const ScatterBulkLayout L = scatter_bulk_layout<T>(a.d, per_sm);
    unsigned int *timeouts = wait_timeouts_counter();
    if (L.stages >= 2 && timeouts != nullptr && aligned16(dy)) {
      ScatterArgs b = a;
      b.sub_groups = min(max_sub, 4 * sm_count());
      const int bgroups = ceil_div(a.out_rows, kBulkJobs);
      const int brow = row_ctas > 0 ? min(bgroups, row_ctas) : bgroups;
      const int bkv = ceil_div(ncv, kBulkConsumers);
      auto go_bulk = [&](auto kern) -> int {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(L.total));
        DLB_REQUIRE(e == cudaSuccess, DLB_ERR_CUDA, "scatter_rows_bulk: shared memory attribute: %s", cudaGetErrorString(e));
        launch_pdl(kern, b.sub_groups + brow, kBulkThreads, L.total, st, static_cast<const T *>(dy), b, L, timeouts);
        return DLB_OK;
      };
      int rc;
      if (bkv > 2) rc = go_bulk(scatter_rows_bulk_kernel<T, 4>);
      else if (bkv == 2) rc = go_bulk(scatter_rows_bulk_kernel<T, 2>);
      else rc = go_bulk(scatter_rows_bulk_kernel<T, 1>);
      if (rc != DLB_OK) return rc;
      DLB_LAUNCH_CHECK("scatter_rows_bulk");
      launched = true;
    }
  }
  if (!launched) {
    auto go = [&](auto kern) { launch_pdl(kern, grid, dim3(bs.tx, bs.ty), 0, st, static_cast<const T *>(dy), a); };
    if (kv == 4) go(scatter_rows_kernel<T, 4>);
    else if (kv == 2) go(scatter_rows_kernel<T, 2>);
    else go(scatter_rows_kernel<T, 1>);
    DLB_LAUNCH_CHECK("scatter_rows");
  }
  // 8 CTAs fit an SM; each loops over (long row, column block) items
  launch_pdl(combine_long_kernel, 8 * sm_count(), kEmbBlock, 0, st, a);
  DLB_LAUNCH_CHECK("combine_long");
  return DLB_OK;
}

}  // namespace dlb
