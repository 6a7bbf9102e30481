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
//   * peer memory (the fused path): dlb_embed_scatter_bwd_peer stores a row that only this
//     rank has tokens for straight into row v of EVERY rank's dense table, and a row that
//     several ranks share into the receive area of the slot's owner (slot % n);
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

struct RankPlan {
  int32_t *header;     // [16]  {used rows, long rows, sub-segments, -, done counters x4, ...}
  int32_t *slot_map;   // [V]   slot of a table row, -1 if no rank refers to it
  int32_t *used_rows;  // [V]   table row of a slot
  int32_t *row_begin;  // [V]   this rank's range of the global sorted list, per slot
  int32_t *row_end;    // [V]
  uint32_t *src_mask;  // [V]   ranks that have tokens for the slot
  uint32_t *tmp_mask;  // [V]   the same three per TABLE ROW, before the slots are numbered
  int32_t *tmp_begin;  // [V]
  int32_t *tmp_end;    // [V]
  int32_t *long_row;   // [max_long]    slots with more than kSubLen local tokens
  int32_t *long_first; // [max_long+1]  running count of their sub-segments
  float *scratch;      // [max_sub][d]
  int max_long, max_sub;
  size_t bytes;
};

RankPlan make_rank_plan(void *workspace, int vocab, int tokens_per_rank, int d) {
  RankPlan r{};
  r.max_long = tokens_per_rank / kSubLen + 1;
  r.max_sub = 2 * (tokens_per_rank / kSubLen) + 2;
  char *base = static_cast<char *>(workspace);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    char *ptr = base ? base + off : nullptr;
    off += align_up256(bytes);
    return ptr;
  };
  const size_t per = sizeof(int32_t) * static_cast<size_t>(vocab);
  r.header = reinterpret_cast<int32_t *>(take(sizeof(int32_t) * 16));
  r.slot_map = reinterpret_cast<int32_t *>(take(per));
  r.used_rows = reinterpret_cast<int32_t *>(take(per));
  r.row_begin = reinterpret_cast<int32_t *>(take(per));
  r.row_end = reinterpret_cast<int32_t *>(take(per));
  r.src_mask = reinterpret_cast<uint32_t *>(take(per));
  r.tmp_mask = reinterpret_cast<uint32_t *>(take(per));
  r.tmp_begin = reinterpret_cast<int32_t *>(take(per));
  r.tmp_end = reinterpret_cast<int32_t *>(take(per));
  r.long_row = reinterpret_cast<int32_t *>(take(sizeof(int32_t) * r.max_long));
  r.long_first = reinterpret_cast<int32_t *>(take(sizeof(int32_t) * (r.max_long + 1)));
  r.scratch = reinterpret_cast<float *>(take(sizeof(float) * static_cast<size_t>(r.max_sub) * d));
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

// Exclusive scan of one 64-bit value per thread over the 1024 threads of the CTA; tmp holds 33 values.
__device__ __forceinline__ unsigned long long cta_scan_u64(unsigned long long v, unsigned long long *tmp,
                                                           unsigned long long *total) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned long long incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  __syncthreads();
  if (lane == 31) tmp[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const unsigned long long w = tmp[lane];
    unsigned long long wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    tmp[lane] = wi - w;
    if (lane == 31) tmp[32] = wi;
  }
  __syncthreads();
  *total = tmp[32];
  return tmp[warp] + incl - v;
}

// Phase 3, one CTA: walks the table rows in order, 1024 at a time, and numbers the used rows and
// this rank's long rows.  Three counts ride in one 64-bit scan: used rows (bits 0..19), long rows
// (20..39), sub-segments (40..63).
__global__ void __launch_bounds__(1024)
rank_plan_number_kernel(const int32_t *seg_global, int vocab, RankPlan r) {
  pdl_prologue();
  __shared__ unsigned long long tmp[33];
  unsigned long long base = 0;
  for (int v0 = 0; v0 < vocab; v0 += 1024) {
    const int v = v0 + threadIdx.x;
    const bool used = v < vocab && ld_co(seg_global + v + 1) > ld_co(seg_global + v);
    int b = 0, e = 0;
    if (used) {
      b = ld_co(r.tmp_begin + v);
      e = ld_co(r.tmp_end + v);
    }
    const int cnt = e - b;
    const bool is_long = cnt > kSubLen;
    const unsigned long long nsub = is_long ? static_cast<unsigned long long>((cnt + kSubLen - 1) / kSubLen) : 0ull;
    const unsigned long long mine = (used ? 1ull : 0ull) | (is_long ? (1ull << 20) : 0ull) | (nsub << 40);
    unsigned long long total;
    const unsigned long long at = base + cta_scan_u64(mine, tmp, &total);
    if (v < vocab) {
      const int slot = static_cast<int>(at & 0xfffffull);
      r.slot_map[v] = used ? slot : -1;
      if (used) {
        r.used_rows[slot] = v;
        r.row_begin[slot] = b;
        r.row_end[slot] = e;
        r.src_mask[slot] = ld_co(r.tmp_mask + v);
        if (is_long) {
          const int li = static_cast<int>((at >> 20) & 0xfffffull);
          r.long_row[li] = slot;
          r.long_first[li] = static_cast<int>(at >> 40);
        }
      }
    }
    base += total;
  }
  if (threadIdx.x == 0) {
    const int n_long = static_cast<int>((base >> 20) & 0xfffffull);
    r.header[0] = static_cast<int>(base & 0xfffffull);
    r.header[1] = n_long;
    r.header[2] = static_cast<int>(base >> 40);
    r.long_first[n_long] = static_cast<int>(base >> 40);
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

// Second half of the peer exchange, run by the owner of a slot.  Every CTA first waits until all
// ranks have announced (wait channel) that their partial rows are out.  Work items are (owned
// slot, block of kBlock float4 columns); a slot that fewer than two ranks have tokens for is
// skipped (its only source stored the finished row itself).  The partial rows of the ranks in the
// slot's mask are added in rank order and the sum is stored into row used_rows[slot] of every
// rank's dense table.  The small-gradient buffers that arrived from the ranks are added the same
// way into small_out.  The last CTA announces the signal channel.
struct ReduceArgs {
  const float *recv;         // this rank's receive area [n][cap][d]
  float *grad[kMaxPeers];    // every rank's dense table
  const float *small_recv;   // this rank's [n][small_n] area
  float *small_out;
  const uint32_t *my_flags;
  uint32_t *status;
  const int32_t *header, *used_rows;
  const uint32_t *src_mask;
  int n, me, cap, d, small_n, wait_channel;
  uint32_t wait_epoch;
  unsigned long long limit_ns;
};

__global__ void __launch_bounds__(kBlock)
reduce_broadcast_kernel(const __grid_constant__ ReduceArgs a, const __grid_constant__ PeerSignal sig) {
  pdl_prologue();
  wait_for_peers(a.my_flags, a.n, a.wait_channel, a.wait_epoch, a.limit_ns, a.status);
  const int used = ld_co(a.header);
  const int nvec = a.d / 4;
  const int chunks = (nvec + kBlock - 1) / kBlock;
  const int owned = used > a.me ? (used - a.me + a.n - 1) / a.n : 0;
  for (int item = blockIdx.x; item < owned * chunks; item += gridDim.x) {
    const int j = item / chunks;
    const int slot = a.me + j * a.n;
    const uint32_t mask = ld_co(a.src_mask + slot);
    if (__popc(mask) < 2) continue;
    if (j >= a.cap) {
      if (threadIdx.x == 0) atomicOr(a.status, 1u << 31);
      continue;
    }
    const int c = (item % chunks) * kBlock + threadIdx.x;
    if (c >= nvec) continue;
    const size_t row_off = static_cast<size_t>(ld_co(a.used_rows + slot)) * a.d;
    // every source's cell is loaded before the first add, so the reads are in flight together
    float4 part[kMaxPeers];
#pragma unroll
    for (int src = 0; src < kMaxPeers; src++) {
      if (src < a.n && ((mask >> src) & 1u)) {
        // written by a peer: read at L2, never through L1
        part[src] = __ldcg(reinterpret_cast<const float4 *>(a.recv + (static_cast<size_t>(src) * a.cap + j) * a.d) + c);
      }
    }
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    bool any = false;
#pragma unroll
    for (int src = 0; src < kMaxPeers; src++) {
      if (src < a.n && ((mask >> src) & 1u)) {
        const float4 p = part[src];
        if (!any) {
          acc = p;
          any = true;
        } else {
          acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
        }
      }
    }
#pragma unroll 1
    for (int q = 0; q < a.n; q++) __stcs(reinterpret_cast<float4 *>(a.grad[q] + row_off) + c, acc);
  }
  if (a.small_out != nullptr) {
    const int n4 = a.small_n / 4;
    for (int i = blockIdx.x * kBlock + threadIdx.x; i < n4; i += gridDim.x * kBlock) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int src = 0; src < a.n; src++) {
        const float4 p = __ldcg(reinterpret_cast<const float4 *>(a.small_recv + static_cast<size_t>(src) * a.small_n) + i);
        if (src == 0) {
          acc = p;
        } else {
          acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
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

// The arguments every rank-plan scatter shares.
ScatterArgs rank_scatter_args(const Plan &pg, const RankPlan &r, int tokens_per_rank, int my_rank, int max_rows, int d) {
  ScatterArgs a{};
  a.perm = pg.vals[pg.passes & 1];
  a.seg_b = r.row_begin;
  a.seg_e = r.row_end;
  a.long_row = r.long_row;
  a.long_first = r.long_first;
  a.long_b = r.row_begin;
  a.long_e = r.row_end;
  a.long_out = nullptr;
  a.meta = r.header + 1;
  a.scratch = r.scratch;
  a.out_rows_dev = r.header;
  a.out_rows = max_rows;
  a.tok_offset = my_rank * tokens_per_rank;
  a.d = d;
  return a;
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
  launch_pdl(rank_plan_number_kernel, 1, 1024, 0, st, pg.seg_start, vocab, r);
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
  ScatterArgs a = rank_scatter_args(pg, r, tokens_per_rank, my_rank, max_rows, d);
  a.out = compact_rows;
  const int e = dtype == DLB_BF16 ? 8 : 4;
  DLB_REQUIRE(d % e == 0 && aligned16(dy) && (e == 8 ? aligned32(compact_rows) : aligned16(compact_rows)),
              DLB_ERR_UNSUPPORTED, "embed_scatter_bwd_compact: d must be a multiple of %d and the buffers 32-byte aligned", e);
  if (dtype == DLB_F32) return launch_scatter_rows<float>(dy, a, r.max_sub, 0, nullptr, nullptr, nullptr, as_stream(stream));
  if (dtype == DLB_BF16)
    return launch_scatter_rows<__nv_bfloat16>(dy, a, r.max_sub, 0, nullptr, nullptr, nullptr, as_stream(stream));
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
                                          int max_rows, int vocab, int d, int dtype, int signal_channel,
                                          uint32_t signal_epoch, void *stream) {
  DLB_REQUIRE(shape_ok(global_tokens, vocab, d) && tokens_per_rank > 0 && max_rows >= 0 && max_rows <= vocab,
              DLB_ERR_INVALID_ARG, "embed_scatter_bwd_peer: tokens=%d tokens_per_rank=%d vocab=%d d=%d max_rows=%d",
              global_tokens, tokens_per_rank, vocab, d, max_rows);
  DLB_REQUIRE(group_ok(peers), DLB_ERR_INVALID_ARG, "embed_scatter_bwd_peer: bad peer group (1..%d ranks, my_rank, "
              "cap_rows >= 0, small_n a multiple of 4, timeout_ms 1..10000, status)", kMaxPeers);
  DLB_REQUIRE(signal_channel >= 0 && signal_channel < kPeerChannels, DLB_ERR_INVALID_ARG,
              "embed_scatter_bwd_peer: channel=%d (0..%d)", signal_channel, kPeerChannels - 1);
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
  ScatterArgs a = rank_scatter_args(pg, r, tokens_per_rank, peers->my_rank, max_rows > 0 ? max_rows : 1, d);
  PeerSignal sig{};
  fill_signal(&sig, peers, r.header + 4, signal_channel, signal_epoch);
  // A persistent grid: the exact number of used rows is read on the device, so the host neither waits
  // for the plan nor launches CTAs for rows that do not exist.
  const int row_ctas = 8 * sm_count();
  if (dtype == DLB_F32) return launch_scatter_rows<float>(dy, a, r.max_sub, row_ctas, &route, &push, &sig, as_stream(stream));
  return launch_scatter_rows<__nv_bfloat16>(dy, a, r.max_sub, row_ctas, &route, &push, &sig, as_stream(stream));
}

extern "C" int dlb_embed_reduce_broadcast_peer(void *rank_plan, int tokens_per_rank, const dlb_peer_group *peers,
                                               float *small_out, int vocab, int d, int wait_channel,
                                               uint32_t wait_epoch, int signal_channel, uint32_t signal_epoch,
                                               void *stream) {
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
  a.src_mask = r.src_mask;
  a.n = peers->n_ranks;
  a.me = me;
  a.cap = peers->cap_rows;
  a.d = d;
  a.small_n = peers->small_n;
  a.wait_channel = wait_channel;
  a.wait_epoch = wait_epoch;
  a.limit_ns = static_cast<unsigned long long>(peers->timeout_ms) * 1000000ull;
  PeerSignal sig{};
  fill_signal(&sig, peers, r.header + 5, signal_channel, signal_epoch);
  const int grid = 4 * sm_count();
  launch_pdl(reduce_broadcast_kernel, grid, kBlock, 0, as_stream(stream), a, sig);
  DLB_LAUNCH_CHECK("reduce_broadcast");
  return DLB_OK;
}
