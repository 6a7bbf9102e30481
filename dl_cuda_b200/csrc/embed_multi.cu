// Embedding-table gradient when the token rows are sharded over the GPUs of one node.
//
// Every rank gathers the ids of all ranks and sorts them once (dlb_embed_sort_tokens: the
// "global plan"; rank r holds tokens [r*tpr, (r+1)*tpr) of the gathered list).  The sort is
// stable, so inside a table row's run the token indices ascend and the tokens of one rank are
// contiguous.  dlb_embed_rank_plan derives from it, with no second sort:
//   * the numbering of the table rows ANY rank refers to ("used" rows, slots 0..used-1 in
//     ascending id: the same on every rank);
//   * per slot this rank's range of the sorted list, and the set of ranks that have tokens
//     for it (a bit mask);
//   * this rank's long rows (more than kSubLen local tokens) for the sub-segment sums.
// Two ways to finish from there:
//   * compact + all-reduce: dlb_embed_scatter_bwd_compact sums the local tokens into a dense
//     [used, d] buffer (zeros where this rank has no token), the caller all-reduces it, and
//     dlb_embed_expand_rows writes the dense [vocab, d] gradient;
//   * peer memory (the fused path): dlb_embed_scatter_bwd_peer sums this rank's tokens per
//     row into a local buffer (only rows it has tokens for: HBM-bound, the same kernel as the
//     single-GPU scatter) and then streams those rows out in a copy-shaped kernel that keeps
//     NVLink full: a row that only this rank has tokens for goes straight into row v of EVERY
//     rank's dense table, a row that several ranks share into the receive area of the slot's
//     owner (slot % n).  (Storing to the peers from inside the summing kernel was measured at
//     300 GB/s: its load -> store dependency chains leave the links idle most of the time;
//     the copy-shaped kernel reaches the 700 GB/s a plain peer copy gets.)
//     dlb_embed_reduce_broadcast_peer, on the owner, waits for the ranks' arrival flags, adds
//     the partial rows in rank order and stores the sum into every rank's table.  The kernels
//     signal and wait through flag words in peer memory themselves; rows no rank uses are
//     zeroed locally by dlb_embed_expand_rows(what = 1).
// No atomics on floating-point data anywhere: every rank ends with the same bits.
#include "common.cuh"
#include "embed_scatter.cuh"

namespace dlb {
namespace {

constexpr int kBlock = kEmbBlock;
constexpr int32_t kHistoryMagic = 0x5a11d001;

// header words of a rank plan
enum {
  kHdrUsed = 0, kHdrLong = 1, kHdrSub = 2, kHdrMine = 3, kHdrDonePush = 4, kHdrDoneReduce = 5, kHdrMulti = 6,
  kHdrOwnShared = 7,  // slots this rank owns that several ranks have tokens for
  kHdrNarrow = 8      // slots whose one token lies on ANOTHER rank (it arrives as a row of storage type)
};

struct RankPlan {
  int32_t *header;       // [16]  see kHdr*
  int32_t *slot_map;     // [V]   slot of a table row, -1 if no rank refers to it
  int32_t *used_rows;    // [V]   table row of a slot
  int32_t *row_begin;    // [V]   this rank's range of the global sorted list, per slot
  int32_t *row_end;      // [V]
  uint32_t *src_mask;    // [V]   ranks that have tokens for the slot
  uint32_t *tmp_mask;    // [V]   the same three per TABLE ROW, before the slots are numbered
  int32_t *tmp_begin;    // [V]
  int32_t *tmp_end;      // [V]
  // "my rows": the slots this rank has tokens for, k = 0..mine-1 in ascending id
  int32_t *my_route;     // [max_mine]  where row k goes: v | 0x80000000 if this rank is its only source
                         //             (straight into row v of every table), else its slot (to the owner)
  int32_t *my_src;       // [max_mine]  where row k comes from: the local token index if it has one token,
                         //             else -(m + 1): row m of my_rows
  int32_t *my_slot;      // [max_mine]  slot of row k
  int32_t *own_shared;   // [V]   slots this rank owns (slot % n == me) that two or more ranks have tokens for
  int32_t *narrow;       // [V]   slots with ONE token in all, on another rank: if the storage type is narrower
                         //       than fp32 that rank sends the token's row as it is and this rank widens it
  // "multi rows": my rows with two or more local tokens, m = 0..multi-1 in ascending id
  int32_t *multi_begin;  // [max_multi] range of the global sorted list
  int32_t *multi_end;    // [max_multi]
  int32_t *multi_slot;   // [max_multi] slot of multi row m
  int32_t *long_row;     // [max_long]    multi rows with more than kSubLen tokens
  int32_t *long_first;   // [max_long+1]  running count of their sub-segments
  float *scratch;        // [max_sub][d]
  float *my_rows;        // [max_multi][d] sums of the multi rows (peer exchange only)
  // Survives from one step to the next (dlb_embed_rank_plan does not touch it): the table rows the last
  // exchange wrote, so that the next one clears only those of them it does not write itself.
  int32_t *history;      // [4 + V]  {magic, rows, table address lo, hi, rows...}
  int max_long, max_sub, max_mine, max_multi;
  size_t bytes;
};

RankPlan make_rank_plan(void *workspace, int vocab, int tokens_per_rank, int d) {
  RankPlan r{};
  r.max_long = tokens_per_rank / kSubLen + 1;
  r.max_sub = 2 * (tokens_per_rank / kSubLen) + 2;
  r.max_mine = vocab < tokens_per_rank ? vocab : tokens_per_rank;
  r.max_multi = vocab < tokens_per_rank / 2 ? vocab : tokens_per_rank / 2;
  if (r.max_multi < 1) r.max_multi = 1;
  char *base = static_cast<char *>(workspace);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    char *ptr = base ? base + off : nullptr;
    off += align_up256(bytes);
    return ptr;
  };
  auto ints = [&](size_t n) { return reinterpret_cast<int32_t *>(take(sizeof(int32_t) * n)); };
  const size_t v = static_cast<size_t>(vocab);
  r.header = ints(16);
  r.slot_map = ints(v);
  r.used_rows = ints(v);
  r.row_begin = ints(v);
  r.row_end = ints(v);
  r.src_mask = reinterpret_cast<uint32_t *>(ints(v));
  r.tmp_mask = reinterpret_cast<uint32_t *>(ints(v));
  r.tmp_begin = ints(v);
  r.tmp_end = ints(v);
  r.my_route = ints(r.max_mine);
  r.my_src = ints(r.max_mine);
  r.my_slot = ints(r.max_mine);
  r.own_shared = ints(v);
  r.narrow = ints(v);
  r.multi_begin = ints(r.max_multi);
  r.multi_end = ints(r.max_multi);
  r.multi_slot = ints(r.max_multi);
  r.long_row = ints(r.max_long);
  r.long_first = ints(r.max_long + 1);
  r.scratch = reinterpret_cast<float *>(take(sizeof(float) * static_cast<size_t>(r.max_sub) * d));
  r.my_rows = reinterpret_cast<float *>(take(sizeof(float) * static_cast<size_t>(r.max_multi) * d));
  r.history = ints(v + 4);
  r.bytes = off;
  return r;
}

// Phase 1: clear what the next phase fills with atomics / sparse stores.
__global__ void __launch_bounds__(kBlock) rank_plan_clear_kernel(RankPlan r, int vocab) {
  pdl_prologue();
  const int v = blockIdx.x * kBlock + threadIdx.x;
  if (v < vocab) {
    r.tmp_mask[v] = 0u;
    r.tmp_begin[v] = 0;
    r.tmp_end[v] = 0;
  }
  if (v < 16) r.header[v] = 0;
}

// Phase 2: one thread per position of the sorted list.  A maximal run of one (table row, rank)
// pair marks the rank in the row's mask; this rank's run gives the row's local range.
__global__ void __launch_bounds__(kBlock)
rank_plan_runs_kernel(const uint32_t *keys, const int32_t *vals, int n, int tokens_per_rank, int me, int vocab,
                      RankPlan r) {
  pdl_prologue();
  const int j = blockIdx.x * kBlock + threadIdx.x;
  if (j >= n) return;
  const uint32_t k = ld_co(keys + j);
  if (k >= static_cast<uint32_t>(vocab)) return;  // ids outside the table belong to no row
  const int rank = ld_co(vals + j) / tokens_per_rank;
  const bool first = j == 0 || ld_co(keys + j - 1) != k || ld_co(vals + j - 1) / tokens_per_rank != rank;
  const bool last = j == n - 1 || ld_co(keys + j + 1) != k || ld_co(vals + j + 1) / tokens_per_rank != rank;
  if (first) {
    atomicOr(r.tmp_mask + k, 1u << rank);  // integer bits: order-free
    if (rank == me) r.tmp_begin[k] = j;
  }
  if (last && rank == me) r.tmp_end[k] = j + 1;
}

// Exclusive scans of three 64-bit values per thread over the 1024 threads of the CTA at once (one set
// of barriers); tmp holds 3 x 33 values.  v[] is replaced by the exclusive prefixes, total[] gets the sums.
__device__ __forceinline__ void cta_scan3_u64(unsigned long long (&v)[3], unsigned long long (*tmp)[33],
                                              unsigned long long (&total)[3]) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned long long incl[3];
#pragma unroll
  for (int i = 0; i < 3; i++) {
    incl[i] = v[i];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long t = __shfl_up_sync(0xffffffffu, incl[i], o);
      if (lane >= o) incl[i] += t;
    }
  }
  __syncthreads();
  if (lane == 31) {
#pragma unroll
    for (int i = 0; i < 3; i++) tmp[i][warp] = incl[i];
  }
  __syncthreads();
  if (warp < 3) {
    const unsigned long long w = tmp[warp][lane];
    unsigned long long wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    tmp[warp][lane] = wi - w;
    if (lane == 31) tmp[warp][32] = wi;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 3; i++) {
    total[i] = tmp[i][32];
    v[i] = tmp[i][warp] + incl[i] - v[i];
  }
}

// Phase 3, one CTA: walks the table rows in order, 1024 at a time, and numbers the used rows
// (slots), this rank's rows, its rows with several tokens, its long rows, the shared slots it owns
// and the slots whose single token lies on another rank.  The counts ride in three 64-bit scans:
//   A {used rows (bits 0..19), long rows (20..39), sub-segments (40..63)}
//   B {my rows (0..19), multi rows (20..39)}
//   C {owned shared slots (0..19), narrow slots (20..39)}   -- needs the slot, so it trails A by a chunk
// A thread takes kNumberRows consecutive rows per step and the CTA scans the threads' sums, so the
// barriers of a scan are paid once per 4096 rows.
constexpr int kNumberRows = 4;  // table rows per thread and step: 4096 rows per step of the CTA

__global__ void __launch_bounds__(1024)
rank_plan_number_kernel(const int32_t *seg_global, const int32_t *vals, int tok_offset, int me, int n_ranks, int vocab,
                        RankPlan r) {
  pdl_prologue();
  __shared__ unsigned long long tmp[3][33];
  unsigned long long base[3] = {0, 0, 0};
  for (int v0 = 0; v0 < vocab; v0 += 1024 * kNumberRows) {
    const int first = v0 + threadIdx.x * kNumberRows;
    int seg[kNumberRows + 1], b[kNumberRows], e[kNumberRows];
    uint32_t mask[kNumberRows];
#pragma unroll
    for (int i = 0; i <= kNumberRows; i++) seg[i] = first + i <= vocab ? ld_co(seg_global + first + i) : 0;
#pragma unroll
    for (int i = 0; i < kNumberRows; i++) {
      const int v = first + i;
      b[i] = v < vocab ? ld_co(r.tmp_begin + v) : 0;
      e[i] = v < vocab ? ld_co(r.tmp_end + v) : 0;
      mask[i] = v < vocab ? ld_co(r.tmp_mask + v) : 0u;
    }
    // A: {used rows (bits 0..19), long rows (20..39), sub-segments (40..63)}; B: {my rows, multi rows}
    unsigned long long in_a[kNumberRows], in_b[kNumberRows];
    unsigned long long val[3] = {0ull, 0ull, 0ull}, total[3];
#pragma unroll
    for (int i = 0; i < kNumberRows; i++) {
      const bool used = first + i < vocab && seg[i + 1] > seg[i];
      const int cnt = used ? e[i] - b[i] : 0;
      const bool is_long = cnt > kSubLen;
      const unsigned long long nsub = is_long ? static_cast<unsigned long long>((cnt + kSubLen - 1) / kSubLen) : 0ull;
      in_a[i] = (used ? 1ull : 0ull) | (is_long ? (1ull << 20) : 0ull) | (nsub << 40);
      in_b[i] = (cnt > 0 ? 1ull : 0ull) | (cnt > 1 ? (1ull << 20) : 0ull);
      val[0] += in_a[i];
      val[1] += in_b[i];
    }
    cta_scan3_u64(val, tmp, total);
    unsigned long long at_a = base[0] + val[0], at_b = base[1] + val[1];
    base[0] += total[0];
    base[1] += total[1];
    // C needs the slot numbers A has just produced: {shared slots this rank owns, narrow slots}
    unsigned long long in_c[kNumberRows], pre_a[kNumberRows], pre_b[kNumberRows];
    unsigned long long val_c[3] = {0ull, 0ull, 0ull}, total_c[3];
#pragma unroll
    for (int i = 0; i < kNumberRows; i++) {
      pre_a[i] = at_a;
      pre_b[i] = at_b;
      const bool used = (in_a[i] & 1ull) != 0;
      const int slot = static_cast<int>(at_a & 0xfffffull);
      const int sources = __popc(mask[i]);
      const bool own_shared = used && sources >= 2 && slot % n_ranks == me;
      const bool narrow = used && sources == 1 && mask[i] != (1u << me) && seg[i + 1] - seg[i] == 1;
      in_c[i] = (own_shared ? 1ull : 0ull) | (narrow ? (1ull << 20) : 0ull);
      val_c[0] += in_c[i];
      at_a += in_a[i];
      at_b += in_b[i];
    }
    cta_scan3_u64(val_c, tmp, total_c);
    unsigned long long at_c = base[2] + val_c[0];
    base[2] += total_c[0];
#pragma unroll
    for (int i = 0; i < kNumberRows; i++) {
      const int v = first + i;
      if (v >= vocab) continue;
      const bool used = (in_a[i] & 1ull) != 0;
      const int slot = static_cast<int>(pre_a[i] & 0xfffffull);
      r.slot_map[v] = used ? slot : -1;
      if (used) {
        const int cnt = e[i] - b[i];
        r.used_rows[slot] = v;
        r.row_begin[slot] = b[i];
        r.row_end[slot] = e[i];
        r.src_mask[slot] = mask[i];
        if (in_c[i] & 1ull) r.own_shared[at_c & 0xfffffull] = slot;
        if (in_c[i] >> 20) r.narrow[(at_c >> 20) & 0xfffffull] = slot;
        if (cnt > 0) {
          const int k = static_cast<int>(pre_b[i] & 0xfffffull);
          const int m = static_cast<int>((pre_b[i] >> 20) & 0xfffffull);
          r.my_route[k] = mask[i] == (1u << me) ? static_cast<int32_t>(static_cast<uint32_t>(v) | 0x80000000u) : slot;
          r.my_src[k] = cnt == 1 ? ld_co(vals + b[i]) - tok_offset : -(m + 1);
          r.my_slot[k] = slot;
          if (cnt > 1) {
            r.multi_begin[m] = b[i];
            r.multi_end[m] = e[i];
            r.multi_slot[m] = slot;
          }
          if (cnt > kSubLen) {
            const int li = static_cast<int>((pre_a[i] >> 20) & 0xfffffull);
            r.long_row[li] = m;
            r.long_first[li] = static_cast<int>(pre_a[i] >> 40);
          }
        }
      }
      at_c += in_c[i];
    }
  }
  if (threadIdx.x == 0) {
    const int n_long = static_cast<int>((base[0] >> 20) & 0xfffffull);
    r.header[kHdrUsed] = static_cast<int>(base[0] & 0xfffffull);
    r.header[kHdrLong] = n_long;
    r.header[kHdrSub] = static_cast<int>(base[0] >> 40);
    r.header[kHdrMine] = static_cast<int>(base[1] & 0xfffffull);
    r.header[kHdrMulti] = static_cast<int>((base[1] >> 20) & 0xfffffull);
    r.header[kHdrOwnShared] = static_cast<int>(base[2] & 0xfffffull);
    r.header[kHdrNarrow] = static_cast<int>((base[2] >> 20) & 0xfffffull);
    r.long_first[n_long] = static_cast<int>(base[0] >> 40);
  }
}

// grad[v,:] = 0 for rows no rank refers to (what & 1); grad[v,:] = compact[slot_map[v],:] for the
// others (what & 2).  blockDim = (tx, ty): ty rows per step, tx float4 column vectors.
__global__ void __launch_bounds__(kBlock)
expand_rows_kernel(const float *compact, const int32_t *slot_map, float *__restrict__ grad, int vocab, int d,
                   int what, int rows_per_cta) {
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

// Scatter arguments from a rank plan.  by_slot: one output row per used row (zeros where this rank
// has no token: the form an all-reduce needs); otherwise one output row per row this rank has
// SEVERAL tokens for, in the plan's own buffer (rows with one token need no sum).
ScatterArgs rank_scatter_args(const Plan &pg, const RankPlan &r, int tokens_per_rank, int my_rank, int max_rows, int d,
                              bool by_slot) {
  ScatterArgs a{};
  a.perm = pg.vals[pg.passes & 1];
  a.seg_b = by_slot ? r.row_begin : r.multi_begin;
  a.seg_e = by_slot ? r.row_end : r.multi_end;
  a.long_row = r.long_row;
  a.long_first = r.long_first;
  a.long_b = r.multi_begin;
  a.long_e = r.multi_end;
  a.long_out = by_slot ? r.multi_slot : nullptr;
  a.meta = r.header + kHdrLong;
  a.scratch = r.scratch;
  a.out_rows_dev = by_slot ? r.header + kHdrUsed : r.header + kHdrMulti;
  a.out_rows = max_rows;
  a.tok_offset = my_rank * tokens_per_rank;
  a.d = d;
  return a;
}

// Streams this rank's rows to where they belong and zeroes, in this rank's own table, the rows no
// rank refers to.  Copy-shaped on purpose: nothing a store needs waits on another store, so the
// links (and, for the zero rows, HBM) stay full.
//   Pushers (one CTA in kPushPeriod, about one per SM): row k of "my rows" is the token's gradient
//     itself (one token: read from dy, widened to fp32) or its sum from the local scatter.  Its
//     only source: stored into row v of every rank's table.  Shared with other ranks: stored into
//     the receive area of the slot's owner.  The small-gradient buffer goes into slot `me` of every
//     rank's area first.
//   The other CTAs write zeros into the table rows that have no slot.
// Why the split: a warp whose stores go out over NVLink stalls at the link's pace, and its zero
// stores would queue behind them; with MANY pushing CTAs the clearing CTAs do not even get onto
// the SMs.  Measured on two B200s (64 MB pushed, 422 MB cleared): 162 us with 1184 pushing CTAs
// beside the clearing ones, 118 us with 148 (alone: 102 and 75 us).
// When the last CTA has issued its stores the grid announces `sig`.
struct SmallPush {
  const float *src;
  float *dst[kMaxPeers];  // every rank's [n ranks][small_n] area
  int small_n;
};

struct PushArgs {
  const float *my_rows;     // [multi rows][d]
  const int32_t *my_route;  // see RankPlan
  const int32_t *my_src;
  const int32_t *my_slot;
  void *stage[kMaxPeers];   // every rank's [slots][d] rows of the storage type (null: rows always travel as fp32)
  int clear;                // 1: this launch also clears the rows nobody uses; 2: only those of them that
                            //    the previous exchange wrote (falls back to 1 if there is no valid history)
  const int32_t *history;   // see RankPlan
  const int32_t *n_mine;    // device word: number of my rows
  const int32_t *slot_map;
  int d, vocab;
  int skip;    // measurements only: 1 no pushes, 2 no zero rows
  int which;   // rows pushed: 1 those with one token (read from dy), 2 the summed ones, 3 both
  int period;  // one CTA in `period` pushes
};

template <int E>
__device__ __forceinline__ void store_vec(float *p, const float (&f)[E]) {
  if constexpr (E == 8) {
    st_stream32(p, f);  // one whole 32-byte sector per lane: 16-byte stores at a 32-byte stride halve the link rate
  } else {
    st_stream(p, make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3])));
  }
}

constexpr int kPushPeriod = 6;  // one CTA in six pushes; six CTAs fit an SM, so every SM hosts about one pusher

template <typename T>
__global__ void __launch_bounds__(kBlock, kPushPeriod)
push_rows_kernel(const T *dy, const __grid_constant__ PushArgs a, const __grid_constant__ PeerRoute pr,
                 const __grid_constant__ SmallPush sp, const __grid_constant__ PeerSignal sig) {
  pdl_prologue();
  using S = Store<T>;
  constexpr int E = S::kPerVec;
  const int d = a.d;
  const int nv4 = d / 4;
  const int period = a.period;
  const int pushers = (gridDim.x + period - 1) / period;
  if (blockIdx.x % period == 0) {
    // ------------------------------------------------------------------ pusher
    const int me = blockIdx.x / period;
    if (sp.src != nullptr) {
      const int n4 = sp.small_n / 4;
      for (int i = me * kBlock + threadIdx.x; i < n4; i += pushers * kBlock) {
        const float4 v = *reinterpret_cast<const float4 *>(sp.src + 4 * static_cast<size_t>(i));
        for (int q = 0; q < pr.n; q++)
          __stcs(reinterpret_cast<float4 *>(sp.dst[q] + static_cast<size_t>(pr.me) * sp.small_n) + i, v);
      }
    }
    const int n_mine = a.skip == 1 ? 0 : ld_co(a.n_mine);
    const int ncv = d / E;
    int k = me;
    int src = k < n_mine ? ld_co(a.my_src + k) : 0;
    int32_t route = k < n_mine ? ld_co(a.my_route + k) : 0;
    while (k < n_mine) {
      // the next row's two words are fetched while this row moves
      const int k_next = k + pushers;
      const int src_next = k_next < n_mine ? ld_co(a.my_src + k_next) : 0;
      const int32_t route_next = k_next < n_mine ? ld_co(a.my_route + k_next) : 0;
      const bool everywhere = route < 0;
      size_t off = 0;
      float *single = nullptr;
      bool ok = (a.which & (src >= 0 ? 1 : 2)) != 0;
      if (!ok) {
      } else if (everywhere) {
        off = static_cast<size_t>(static_cast<uint32_t>(route) & 0x7fffffffu) * d;
      } else {
        const int j = route / pr.n;
        if (j >= pr.cap) {
          if (threadIdx.x == 0) atomicOr(pr.status, 1u << 31);
          ok = false;
        } else {
          single = pr.recv[route % pr.n] + (static_cast<size_t>(pr.me) * pr.cap + j) * d;
        }
      }
      if (ok && src >= 0) {
        // one token: the row is dy[src,:] widened to fp32 (0.0f + x carries x's bits)
        const T *row = dy + static_cast<size_t>(src) * d;
        // one token here and this rank the only source = one token in all
        const bool narrow_ok = sizeof(T) < 4 && a.stage[0] != nullptr;
        const int slot_k = narrow_ok && everywhere ? ld_co(a.my_slot + k) : 0;
        for (int cv0 = threadIdx.x; cv0 < ncv; cv0 += 2 * kBlock) {
          uint4 raw[2];
#pragma unroll
          for (int u = 0; u < 2; u++)
            if (cv0 + u * kBlock < ncv) raw[u] = ld_stream(row + static_cast<size_t>(cv0 + u * kBlock) * E);
#pragma unroll
          for (int u = 0; u < 2; u++) {
            const int cv = cv0 + u * kBlock;
            if (cv >= ncv) continue;
            float f[E];
            S::unpack(raw[u], f);
#pragma unroll
            for (int e = 0; e < E; e++) f[e] = 0.0f + f[e];
            if (everywhere && narrow_ok) {
              // The one token of this row anywhere: the peers get the row as it is stored (half the bytes
              // for bf16) and widen it themselves; only this rank's own table gets the fp32 row here.
              store_vec<E>(pr.grad[pr.me] + off + static_cast<size_t>(cv) * E, f);
#pragma unroll 1
              for (int q = 0; q < pr.n; q++) {
                if (q != pr.me)
                  __stcs(reinterpret_cast<uint4 *>(static_cast<T *>(a.stage[q]) + static_cast<size_t>(slot_k) * d) + cv, raw[u]);
              }
            } else if (everywhere) {
#pragma unroll 1
              for (int q = 0; q < pr.n; q++) store_vec<E>(pr.grad[q] + off + static_cast<size_t>(cv) * E, f);
            } else {
              store_vec<E>(single + static_cast<size_t>(cv) * E, f);
            }
          }
        }
      } else if (ok) {
        const float4 *row = reinterpret_cast<const float4 *>(a.my_rows + static_cast<size_t>(-src - 1) * d);
        for (int c0 = threadIdx.x; c0 < nv4; c0 += 4 * kBlock) {
          float4 v[4];
#pragma unroll
          for (int u = 0; u < 4; u++)
            if (c0 + u * kBlock < nv4) v[u] = __ldcs(row + c0 + u * kBlock);
#pragma unroll
          for (int u = 0; u < 4; u++) {
            const int c = c0 + u * kBlock;
            if (c >= nv4) continue;
            if (everywhere) {
#pragma unroll 1
              for (int q = 0; q < pr.n; q++) __stcs(reinterpret_cast<float4 *>(pr.grad[q] + off) + c, v[u]);
            } else {
              __stcs(reinterpret_cast<float4 *>(single) + c, v[u]);
            }
          }
        }
      }
      k = k_next;
      src = src_next;
      route = route_next;
    }
  } else if (a.skip != 2 && a.clear) {
    // ------------------------------------------------------------------ clears the rows nobody uses
    const int zeroers = gridDim.x - pushers;
    const int me = blockIdx.x - blockIdx.x / period - 1;
    float *mine = pr.grad[pr.me];
    const unsigned long long addr = reinterpret_cast<unsigned long long>(mine);
    const bool by_history = a.clear == 2 && ld_co(a.history) == kHistoryMagic &&
                            static_cast<uint32_t>(ld_co(a.history + 2)) == static_cast<uint32_t>(addr) &&
                            static_cast<uint32_t>(ld_co(a.history + 3)) == static_cast<uint32_t>(addr >> 32);
    if (by_history) {
      // Everything outside the rows the last exchange wrote is zero already: clear only those of them
      // that no rank uses this time.
      const int count = min(ld_co(a.history + 1), a.vocab);
      for (int i0 = me * 8; i0 < count; i0 += 8 * zeroers) {
        int row[8], slot[8];
#pragma unroll
        for (int u = 0; u < 8; u++) row[u] = i0 + u < count ? ld_co(a.history + 4 + i0 + u) : -1;
#pragma unroll
        for (int u = 0; u < 8; u++) slot[u] = (row[u] >= 0 && row[u] < a.vocab) ? ld_co(a.slot_map + row[u]) : 0;
#pragma unroll
        for (int u = 0; u < 8; u++) {
          if (slot[u] < 0) {
            float4 *dst = reinterpret_cast<float4 *>(mine + static_cast<size_t>(row[u]) * d);
            for (int c = threadIdx.x; c < nv4; c += kBlock) __stcs(dst + c, make_float4(0.f, 0.f, 0.f, 0.f));
          }
        }
      }
    } else {
      // Blocks of eight consecutive rows per CTA, the CTAs' blocks side by side: the rows being written
      // at any moment form one compact window of the table.
      for (int v0 = me * 8; v0 < a.vocab; v0 += 8 * zeroers) {
        int slot[8];
#pragma unroll
        for (int u = 0; u < 8; u++) slot[u] = v0 + u < a.vocab ? ld_co(a.slot_map + v0 + u) : 0;
#pragma unroll
        for (int u = 0; u < 8; u++) {
          if (slot[u] < 0) {
            float4 *dst = reinterpret_cast<float4 *>(mine + static_cast<size_t>(v0 + u) * d);
            for (int c = threadIdx.x; c < nv4; c += kBlock) __stcs(dst + c, make_float4(0.f, 0.f, 0.f, 0.f));
          }
        }
      }
    }
  }
  signal_when_grid_done(sig);
}

// Second half of the peer exchange.  Every CTA first waits until all ranks have announced (wait
// channel) that their rows are out.  Then, from lists the rank plan prepared (no searching):
//   * shared slots this rank owns: the partial rows of the ranks in the slot's mask are added in rank
//     order and the sum is stored into row used_rows[slot] of every rank's dense table; a work item
//     is (slot, block of kBlock float4 columns);
//   * narrow slots (one token in all, on another rank, sent as a row of the storage type): widened to
//     fp32 into this rank's own table row;
//   * the small-gradient buffers that arrived from the ranks are added in rank order into small_out.
// The last CTA announces the signal channel.
struct ReduceArgs {
  const float *recv;         // this rank's receive area [n][cap][d]
  float *grad[kMaxPeers];    // every rank's dense table
  const float *small_recv;   // this rank's [n][small_n] area
  float *small_out;
  const void *stage;         // this rank's [slots][d] rows of the storage type, or null
  const uint32_t *my_flags;
  uint32_t *status;
  const int32_t *header, *used_rows, *own_shared, *narrow;
  int32_t *history;          // receives the table rows this exchange wrote (see RankPlan)
  const uint32_t *src_mask;
  int n, me, cap, d, small_n, wait_channel;
  uint32_t wait_epoch;
  unsigned long long limit_ns;
};

template <typename T>
__global__ void __launch_bounds__(kBlock, 4)
reduce_broadcast_kernel(const __grid_constant__ ReduceArgs a, const __grid_constant__ PeerSignal sig) {
  pdl_prologue();
  wait_for_peers(a.my_flags, a.n, a.wait_channel, a.wait_epoch, a.limit_ns, a.status);
  using S = Store<T>;
  constexpr int E = S::kPerVec;
  const int d = a.d;
  const int nvec = d / 4;
  const int chunks = (nvec + kBlock - 1) / kBlock;
  const int shared = ld_co(a.header + kHdrOwnShared);
  for (int item = blockIdx.x; item < shared * chunks; item += gridDim.x) {
    const int slot = ld_co(a.own_shared + item / chunks);
    const int c = (item % chunks) * kBlock + threadIdx.x;
    const int j = slot / a.n;
    if (j >= a.cap) {
      if (threadIdx.x == 0) atomicOr(a.status, 1u << 31);
      continue;
    }
    if (c >= nvec) continue;
    const uint32_t mask = ld_co(a.src_mask + slot);
    const size_t row_off = static_cast<size_t>(ld_co(a.used_rows + slot)) * d;
    // the cells of eight sources are loaded before the first of their adds, so the reads are in flight together
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    bool any = false;
#pragma unroll 1
    for (int base = 0; base < a.n; base += 8) {
      float4 part[8];
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int src = base + u;
        if (src < a.n && ((mask >> src) & 1u)) {
          // written by a peer: read at L2, never through L1
          part[u] = __ldcg(reinterpret_cast<const float4 *>(a.recv + (static_cast<size_t>(src) * a.cap + j) * d) + c);
        }
      }
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int src = base + u;
        if (src < a.n && ((mask >> src) & 1u)) {
          const float4 p = part[u];
          if (!any) {
            acc = p;
            any = true;
          } else {
            acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
          }
        }
      }
    }
#pragma unroll 1
    for (int q = 0; q < a.n; q++) __stcs(reinterpret_cast<float4 *>(a.grad[q] + row_off) + c, acc);
  }
  if (a.stage != nullptr) {
    // Two rows per step (their loads in flight together); the slots and table rows of the next step
    // are fetched while these move.
    const int narrow = ld_co(a.header + kHdrNarrow);
    const int ncv = d / E;
    const T *stage = static_cast<const T *>(a.stage);
    float *mine = a.grad[a.me];
    int item = 2 * blockIdx.x;
    int slot[2], row[2];
#pragma unroll
    for (int u = 0; u < 2; u++) slot[u] = item + u < narrow ? ld_co(a.narrow + item + u) : 0;
#pragma unroll
    for (int u = 0; u < 2; u++) row[u] = item + u < narrow ? ld_co(a.used_rows + slot[u]) : 0;
    while (item < narrow) {
      const int item_next = item + 2 * gridDim.x;
      int slot_next[2];
#pragma unroll
      for (int u = 0; u < 2; u++) slot_next[u] = item_next + u < narrow ? ld_co(a.narrow + item_next + u) : 0;
      for (int cv0 = threadIdx.x; cv0 < ncv; cv0 += 2 * kBlock) {
        uint4 raw[2][2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
          const uint4 *src = reinterpret_cast<const uint4 *>(stage + static_cast<size_t>(slot[r]) * d);
#pragma unroll
          for (int u = 0; u < 2; u++)
            if (item + r < narrow && cv0 + u * kBlock < ncv) raw[r][u] = __ldcg(src + cv0 + u * kBlock);  // written by a peer
        }
#pragma unroll
        for (int r = 0; r < 2; r++) {
          float *dst = mine + static_cast<size_t>(row[r]) * d;
#pragma unroll
          for (int u = 0; u < 2; u++) {
            if (item + r >= narrow || cv0 + u * kBlock >= ncv) continue;
            float f[E];
            S::unpack(raw[r][u], f);
#pragma unroll
            for (int e = 0; e < E; e++) f[e] = 0.0f + f[e];
            store_vec<E>(dst + static_cast<size_t>(cv0 + u * kBlock) * E, f);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 2; u++) {
        row[u] = item_next + u < narrow ? ld_co(a.used_rows + slot_next[u]) : 0;
        slot[u] = slot_next[u];
      }
      item = item_next;
    }
  }
  {
    // what the next exchange may have to clear: the rows written into this rank's table this time
    const int used = ld_co(a.header + kHdrUsed);
    for (int i = blockIdx.x * kBlock + threadIdx.x; i < used; i += gridDim.x * kBlock)
      a.history[4 + i] = ld_co(a.used_rows + i);
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      const unsigned long long addr = reinterpret_cast<unsigned long long>(a.grad[a.me]);
      a.history[0] = kHistoryMagic;
      a.history[1] = used;
      a.history[2] = static_cast<int32_t>(static_cast<uint32_t>(addr));
      a.history[3] = static_cast<int32_t>(static_cast<uint32_t>(addr >> 32));
    }
  }
  if (a.small_out != nullptr) {
    const int n4 = a.small_n / 4;
    for (int i = blockIdx.x * kBlock + threadIdx.x; i < n4; i += gridDim.x * kBlock) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
      for (int base = 0; base < a.n; base += 8) {
        float4 part[8];
#pragma unroll
        for (int u = 0; u < 8; u++)
          if (base + u < a.n)
            part[u] = __ldcg(reinterpret_cast<const float4 *>(a.small_recv + static_cast<size_t>(base + u) * a.small_n) + i);
#pragma unroll
        for (int u = 0; u < 8; u++) {
          if (base + u >= a.n) continue;
          if (base + u == 0) {
            acc = part[u];
          } else {
            acc.x += part[u].x; acc.y += part[u].y; acc.z += part[u].z; acc.w += part[u].w;
          }
        }
      }
      reinterpret_cast<float4 *>(a.small_out)[i] = acc;
    }
  }
  signal_when_grid_done(sig);
}

bool shape_ok(int tokens, int vocab, int d) {
  return tokens >= 0 && vocab > 0 && d > 0 && static_cast<int64_t>(vocab) * d <= INT64_MAX / 8;
}

bool group_ok(const dlb_peer_group *g) {
  return g != nullptr && g->n_ranks >= 1 && g->n_ranks <= kMaxPeers && g->my_rank >= 0 && g->my_rank < g->n_ranks &&
         g->cap_rows >= 0 && g->small_n >= 0 && g->small_n % 4 == 0 && g->timeout_ms > 0 && g->timeout_ms <= 10000 &&
         g->status != nullptr;
}

}  // namespace
}  // namespace dlb

using namespace dlb;

extern "C" size_t dlb_embed_rank_plan_bytes(int vocab, int tokens_per_rank, int d) {
  if (!shape_ok(tokens_per_rank, vocab, d)) return 0;
  return make_rank_plan(nullptr, vocab, tokens_per_rank, d).bytes;
}

extern "C" int dlb_embed_rank_plan(const void *global_plan, int global_tokens, int tokens_per_rank, int n_ranks,
                                   int my_rank, void *rank_plan, size_t rank_plan_bytes, int vocab, int d,
                                   void *stream) {
  DLB_REQUIRE(shape_ok(global_tokens, vocab, d) && tokens_per_rank > 0, DLB_ERR_INVALID_ARG,
              "embed_rank_plan: tokens=%d tokens_per_rank=%d vocab=%d d=%d", global_tokens, tokens_per_rank, vocab, d);
  DLB_REQUIRE(n_ranks >= 1 && n_ranks <= kMaxPeers && my_rank >= 0 && my_rank < n_ranks &&
                  static_cast<int64_t>(n_ranks) * tokens_per_rank >= global_tokens,
              DLB_ERR_INVALID_ARG, "embed_rank_plan: n_ranks=%d (1..%d) my_rank=%d: %d ranks of %d tokens must cover %d",
              n_ranks, kMaxPeers, my_rank, n_ranks, tokens_per_rank, global_tokens);
  DLB_REQUIRE(vocab < (1 << 20) && global_tokens < (1 << 24), DLB_ERR_UNSUPPORTED,
              "embed_rank_plan: at most 2^20 table rows and 2^24 tokens");
  DLB_REQUIRE(global_plan && rank_plan && (reinterpret_cast<uintptr_t>(rank_plan) & 255u) == 0 &&
                  rank_plan_bytes >= dlb_embed_rank_plan_bytes(vocab, tokens_per_rank, d),
              DLB_ERR_WORKSPACE, "embed_rank_plan: the global plan and a 256-byte aligned workspace of %zu bytes required",
              dlb_embed_rank_plan_bytes(vocab, tokens_per_rank, d));
  cudaStream_t st = as_stream(stream);
  const Plan pg = make_plan(const_cast<void *>(global_plan), global_tokens, vocab, d);
  const RankPlan r = make_rank_plan(rank_plan, vocab, tokens_per_rank, d);
  const int cells = vocab > 16 ? vocab : 16;
  launch_pdl(rank_plan_clear_kernel, ceil_div(cells, kBlock), kBlock, 0, st, r, vocab);
  DLB_LAUNCH_CHECK("rank_plan_clear");
  if (global_tokens > 0) {
    launch_pdl(rank_plan_runs_kernel, ceil_div(global_tokens, kBlock), kBlock, 0, st, pg.keys[pg.passes & 1],
               pg.vals[pg.passes & 1], global_tokens, tokens_per_rank, my_rank, vocab, r);
    DLB_LAUNCH_CHECK("rank_plan_runs");
  }
  launch_pdl(rank_plan_number_kernel, 1, 1024, 0, st, pg.seg_start, pg.vals[pg.passes & 1], my_rank * tokens_per_rank,
             my_rank, n_ranks, vocab, r);
  DLB_LAUNCH_CHECK("rank_plan_number");
  return DLB_OK;
}

extern "C" int dlb_embed_scatter_bwd_compact(const void *dy, const void *global_plan, int global_tokens,
                                             void *rank_plan, int tokens_per_rank, int my_rank, float *compact_rows,
                                             int max_rows, int vocab, int d, int dtype, void *stream) {
  DLB_REQUIRE(shape_ok(global_tokens, vocab, d) && tokens_per_rank > 0 && my_rank >= 0 && max_rows >= 0 &&
                  max_rows <= vocab,
              DLB_ERR_INVALID_ARG, "embed_scatter_bwd_compact: tokens=%d tokens_per_rank=%d my_rank=%d max_rows=%d",
              global_tokens, tokens_per_rank, my_rank, max_rows);
  DLB_REQUIRE(global_plan && rank_plan, DLB_ERR_WORKSPACE, "embed_scatter_bwd_compact: plan workspaces required");
  DLB_REQUIRE((compact_rows && dy) || max_rows == 0, DLB_ERR_INVALID_ARG, "embed_scatter_bwd_compact: null pointer");
  if (max_rows == 0) return DLB_OK;
  const Plan pg = make_plan(const_cast<void *>(global_plan), global_tokens, vocab, d);
  const RankPlan r = make_rank_plan(rank_plan, vocab, tokens_per_rank, d);
  ScatterArgs a = rank_scatter_args(pg, r, tokens_per_rank, my_rank, max_rows, d, true);
  a.out = compact_rows;
  const int e = dtype == DLB_BF16 ? 8 : 4;
  DLB_REQUIRE(d % e == 0 && aligned16(dy) && (e == 8 ? aligned32(compact_rows) : aligned16(compact_rows)),
              DLB_ERR_UNSUPPORTED, "embed_scatter_bwd_compact: d must be a multiple of %d and the buffers 32-byte aligned", e);
  if (dtype == DLB_F32) return launch_scatter_rows<float>(dy, a, r.max_sub, 0, as_stream(stream));
  if (dtype == DLB_BF16) return launch_scatter_rows<__nv_bfloat16>(dy, a, r.max_sub, 0, as_stream(stream));
  set_error("embed_scatter_bwd_compact: unknown dtype %d", dtype);
  return DLB_ERR_INVALID_ARG;
}

extern "C" int dlb_embed_expand_rows(const float *compact_rows, const void *rank_plan, int tokens_per_rank, float *grad,
                                     int vocab, int d, int what, void *stream) {
  DLB_REQUIRE(vocab > 0 && d > 0 && d % 4 == 0 && tokens_per_rank > 0 && (what & 3) != 0 && (what & ~3) == 0,
              DLB_ERR_INVALID_ARG, "embed_expand_rows: vocab=%d d=%d (a multiple of 4) what=%d (1 zero, 2 copy, 3 both)",
              vocab, d, what);
  DLB_REQUIRE(rank_plan && grad && aligned16(grad) && (!(what & 2) || (compact_rows && aligned16(compact_rows))),
              DLB_ERR_INVALID_ARG, "embed_expand_rows: null or unaligned pointer");
  const RankPlan r = make_rank_plan(const_cast<void *>(rank_plan), vocab, tokens_per_rank, d);
  int tx = 1;
  while (tx < kBlock && tx < d / 4) tx *= 2;
  const int ty = kBlock / tx;
  const int rows_per_cta = ty > 8 ? ty : 8;
  launch_pdl(expand_rows_kernel, ceil_div(vocab, rows_per_cta), dim3(tx, ty), 0, as_stream(stream), compact_rows,
             r.slot_map, grad, vocab, d, what, rows_per_cta);
  DLB_LAUNCH_CHECK("expand_rows");
  return DLB_OK;
}

// ---- table gradient exchanged over peer memory ------------------------------------------------------

static void fill_signal(PeerSignal *s, const dlb_peer_group *g, int32_t *done, int channel, uint32_t epoch) {
  for (int q = 0; q < g->n_ranks; q++) s->flags[q] = g->flags[q];
  s->done = done;
  s->n = g->n_ranks;
  s->me = g->my_rank;
  s->channel = channel;
  s->epoch = epoch;
}

extern "C" int dlb_embed_scatter_bwd_peer(const void *dy, const void *global_plan, int global_tokens, void *rank_plan,
                                          int tokens_per_rank, const dlb_peer_group *peers, const float *small,
                                          int max_rows, int clear_unused, int part, int vocab, int d, int dtype,
                                          int signal_channel, uint32_t signal_epoch, void *stream) {
  DLB_REQUIRE(part >= 0 && part <= 3, DLB_ERR_INVALID_ARG, "embed_scatter_bwd_peer: part=%d (0 all, 1 sums, 2 first push, "
              "3 second push)", part);
  DLB_REQUIRE(shape_ok(global_tokens, vocab, d) && tokens_per_rank > 0 && max_rows >= 0 && max_rows <= vocab,
              DLB_ERR_INVALID_ARG, "embed_scatter_bwd_peer: tokens=%d tokens_per_rank=%d vocab=%d d=%d max_rows=%d",
              global_tokens, tokens_per_rank, vocab, d, max_rows);
  DLB_REQUIRE(group_ok(peers), DLB_ERR_INVALID_ARG, "embed_scatter_bwd_peer: bad peer group (1..%d ranks, my_rank, "
              "cap_rows >= 0, small_n a multiple of 4, timeout_ms 1..10000, status)", kMaxPeers);
  DLB_REQUIRE(signal_channel >= 0 && signal_channel < kPeerChannels && clear_unused >= 0 && clear_unused <= 2,
              DLB_ERR_INVALID_ARG, "embed_scatter_bwd_peer: channel=%d (0..%d) clear_unused=%d (0, 1 or 2)", signal_channel,
              kPeerChannels - 1, clear_unused);
  DLB_REQUIRE(static_cast<int64_t>(peers->cap_rows) * peers->n_ranks >= max_rows, DLB_ERR_INVALID_ARG,
              "embed_scatter_bwd_peer: %d rows per source hold fewer than the %d rows asked for", peers->cap_rows,
              max_rows);
  DLB_REQUIRE(global_plan && rank_plan, DLB_ERR_WORKSPACE, "embed_scatter_bwd_peer: plan workspaces required");
  DLB_REQUIRE(dy || global_tokens == 0, DLB_ERR_INVALID_ARG, "embed_scatter_bwd_peer: null dy");
  const int e = dtype == DLB_BF16 ? 8 : 4;
  DLB_REQUIRE(dtype == DLB_F32 || dtype == DLB_BF16, DLB_ERR_INVALID_ARG, "embed_scatter_bwd_peer: unknown dtype %d", dtype);
  DLB_REQUIRE(d % e == 0 && aligned16(dy), DLB_ERR_UNSUPPORTED,
              "embed_scatter_bwd_peer: d must be a multiple of %d and dy 16-byte aligned", e);
  PeerRoute route{};
  SmallPush push{};
  route.n = peers->n_ranks;
  route.me = peers->my_rank;
  route.cap = peers->cap_rows;
  route.status = peers->status;
  for (int q = 0; q < peers->n_ranks; q++) {
    DLB_REQUIRE(peers->flags[q] && peers->recv[q] && peers->grad[q] && aligned32(peers->recv[q]) && aligned32(peers->grad[q]),
                DLB_ERR_INVALID_ARG, "embed_scatter_bwd_peer: a buffer of rank %d is null or not 32-byte aligned", q);
    DLB_REQUIRE(small == nullptr || (peers->small[q] && aligned16(peers->small[q])), DLB_ERR_INVALID_ARG,
                "embed_scatter_bwd_peer: the small-gradient area of rank %d is null or unaligned", q);
    DLB_REQUIRE(peers->stage[0] == nullptr || (peers->stage[q] && aligned16(peers->stage[q])), DLB_ERR_INVALID_ARG,
                "embed_scatter_bwd_peer: the staging area of rank %d is null or unaligned (all ranks or none)", q);
    route.recv[q] = peers->recv[q];
    route.grad[q] = peers->grad[q];
    push.dst[q] = peers->small[q];
  }
  DLB_REQUIRE(small == nullptr || (peers->small_n > 0 && aligned16(small)), DLB_ERR_INVALID_ARG,
              "embed_scatter_bwd_peer: small gradients given but the group has small_n = 0 (or the buffer is unaligned)");
  push.src = small;
  push.small_n = peers->small_n;
  const Plan pg = make_plan(const_cast<void *>(global_plan), global_tokens, vocab, d);
  const RankPlan r = make_rank_plan(rank_plan, vocab, tokens_per_rank, d);
  route.used_rows = r.used_rows;
  route.src_mask = r.src_mask;
  cudaStream_t st = as_stream(stream);
  // 1. the sums of the rows this rank has SEVERAL tokens for, into the plan's own buffer (local,
  //    HBM-bound).  A looping grid: the exact number of rows is read on the device, so the host neither
  //    waits for the plan nor launches CTAs for rows that do not exist.
  int multi_bound = max_rows < r.max_multi ? max_rows : r.max_multi;
  if (multi_bound < 1) multi_bound = 1;
  ScatterArgs a = rank_scatter_args(pg, r, tokens_per_rank, peers->my_rank, multi_bound, d, false);
  a.out = r.my_rows;
  const int phases = get_option("embed_peer_phases");  // measurements only: 1 sums, 2 push
  if ((part == 0 || part == 1) && (phases == 0 || phases == 1)) {
    const int row_ctas = 8 * sm_count();
    const int rc = dtype == DLB_F32 ? launch_scatter_rows<float>(dy, a, r.max_sub, row_ctas, st)
                                    : launch_scatter_rows<__nv_bfloat16>(dy, a, r.max_sub, row_ctas, st);
    if (rc != DLB_OK) return rc;
  }
  if (phases == 1 || part == 1) return DLB_OK;
  // 2. every row out to the tables / the owners, the small gradients along with them, zeros into the
  //    rows nobody uses, then the flag.  In parts: first the rows with one token (they need no sum),
  //    the clearing and the small gradients; then the summed rows and the flag.
  PushArgs pa{};
  pa.my_rows = r.my_rows;
  pa.my_route = r.my_route;
  pa.my_src = r.my_src;
  pa.my_slot = r.my_slot;
  pa.which = part == 2 ? 1 : (part == 3 ? 2 : 3);
  pa.clear = part == 3 ? 0 : clear_unused;
  pa.history = r.history;
  if (part == 3) push.src = nullptr;  // went out with the first push
  for (int q = 0; q < peers->n_ranks; q++) pa.stage[q] = peers->stage[0] != nullptr ? peers->stage[q] : nullptr;
  pa.n_mine = r.header + kHdrMine;
  pa.slot_map = r.slot_map;
  pa.d = d;
  pa.vocab = vocab;
  pa.skip = phases == 3 ? 2 : (phases == 4 ? 1 : 0);
  pa.period = get_option("embed_push_period") > 0 ? get_option("embed_push_period") : kPushPeriod;
  if (!pa.clear) pa.period = 1;  // nothing to clear: every CTA pushes
  PeerSignal sig{};
  if (part != 2) fill_signal(&sig, peers, r.header + kHdrDonePush, signal_channel, signal_epoch);  // the first push of two is silent
  const int grid = kPushPeriod * sm_count();
  if (dtype == DLB_F32)
    launch_pdl(push_rows_kernel<float>, grid, kBlock, 0, st, static_cast<const float *>(dy), pa, route, push, sig);
  else
    launch_pdl(push_rows_kernel<__nv_bfloat16>, grid, kBlock, 0, st, static_cast<const __nv_bfloat16 *>(dy), pa, route,
               push, sig);
  DLB_LAUNCH_CHECK("push_rows");
  return DLB_OK;
}

extern "C" int dlb_embed_reduce_broadcast_peer(void *rank_plan, int tokens_per_rank, const dlb_peer_group *peers,
                                               float *small_out, int vocab, int d, int dtype, int wait_channel,
                                               uint32_t wait_epoch, int signal_channel, uint32_t signal_epoch,
                                               void *stream) {
  DLB_REQUIRE(dtype == DLB_F32 || dtype == DLB_BF16, DLB_ERR_INVALID_ARG, "embed_reduce_broadcast_peer: unknown dtype %d",
              dtype);
  DLB_REQUIRE(vocab > 0 && d > 0 && d % 4 == 0 && tokens_per_rank > 0, DLB_ERR_INVALID_ARG,
              "embed_reduce_broadcast_peer: vocab=%d d=%d (a multiple of 4) tokens_per_rank=%d", vocab, d, tokens_per_rank);
  DLB_REQUIRE(group_ok(peers), DLB_ERR_INVALID_ARG, "embed_reduce_broadcast_peer: bad peer group");
  DLB_REQUIRE(wait_channel >= 0 && wait_channel < kPeerChannels && signal_channel >= 0 && signal_channel < kPeerChannels,
              DLB_ERR_INVALID_ARG, "embed_reduce_broadcast_peer: channels %d, %d (0..%d)", wait_channel, signal_channel,
              kPeerChannels - 1);
  DLB_REQUIRE(rank_plan, DLB_ERR_WORKSPACE, "embed_reduce_broadcast_peer: rank plan required");
  ReduceArgs a{};
  for (int q = 0; q < peers->n_ranks; q++) {
    DLB_REQUIRE(peers->flags[q] && peers->grad[q] && aligned16(peers->grad[q]), DLB_ERR_INVALID_ARG,
                "embed_reduce_broadcast_peer: a buffer of rank %d is null or unaligned", q);
    a.grad[q] = peers->grad[q];
  }
  const int me = peers->my_rank;
  DLB_REQUIRE(peers->recv[me] && aligned16(peers->recv[me]), DLB_ERR_INVALID_ARG,
              "embed_reduce_broadcast_peer: this rank's receive area is null or unaligned");
  DLB_REQUIRE(small_out == nullptr || (peers->small_n > 0 && peers->small[me] && aligned16(small_out)), DLB_ERR_INVALID_ARG,
              "embed_reduce_broadcast_peer: small_out given without a small-gradient area");
  const RankPlan r = make_rank_plan(rank_plan, vocab, tokens_per_rank, d);
  a.recv = peers->recv[me];
  a.small_recv = peers->small[me];
  a.small_out = small_out;
  a.my_flags = peers->flags[me];
  a.status = peers->status;
  a.header = r.header;
  a.used_rows = r.used_rows;
  a.own_shared = r.own_shared;
  a.narrow = r.narrow;
  a.history = r.history;
  a.src_mask = r.src_mask;
  a.stage = (dtype == DLB_BF16 && peers->stage[0] != nullptr) ? peers->stage[me] : nullptr;
  DLB_REQUIRE(d % (dtype == DLB_BF16 ? 8 : 4) == 0 && aligned32(peers->grad[me]), DLB_ERR_UNSUPPORTED,
              "embed_reduce_broadcast_peer: d must be a multiple of %d and the tables 32-byte aligned",
              dtype == DLB_BF16 ? 8 : 4);
  a.n = peers->n_ranks;
  a.me = me;
  a.cap = peers->cap_rows;
  a.d = d;
  a.small_n = peers->small_n;
  a.wait_channel = wait_channel;
  a.wait_epoch = wait_epoch;
  a.limit_ns = static_cast<unsigned long long>(peers->timeout_ms) * 1000000ull;
  PeerSignal sig{};
  fill_signal(&sig, peers, r.header + kHdrDoneReduce, signal_channel, signal_epoch);
  const int grid = 4 * sm_count();  // what fits the GPU at once: one wave
  if (dtype == DLB_BF16)
    launch_pdl(reduce_broadcast_kernel<__nv_bfloat16>, grid, kBlock, 0, as_stream(stream), a, sig);
  else
    launch_pdl(reduce_broadcast_kernel<float>, grid, kBlock, 0, as_stream(stream), a, sig);
  DLB_LAUNCH_CHECK("reduce_broadcast");
  return DLB_OK;
}
