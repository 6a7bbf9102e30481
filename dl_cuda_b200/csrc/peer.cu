// Barrier between the GPUs of one node over peer-mapped flag words, for the steps of
// the table-gradient exchange that one rank's kernels write into another rank's
// memory (csrc/embedding.cu).
//
// Every rank owns a flag array flags[channel][source rank] in memory that all ranks
// have mapped.  To pass barrier number `epoch` of a channel a rank stores `epoch`
// into its own slot of every rank's array (release, system scope) and then waits
// until every slot of its own array has reached `epoch` (acquire, system scope).
// Epochs only grow, so no flag is ever reset.  The kernel runs after everything the
// rank launched before it in the stream (its stores to peers included) and before
// everything after it, so "all ranks passed barrier e" means "all ranks finished the
// kernels they launched before it".
//
// The wait is bounded by a wall-clock limit: when it runs out the kernel records
// the channel in *status and returns; nothing traps and the context stays usable.
// Each rank runs on its own GPU; several ranks of one barrier must never share one.
//
// dlb_peer_wait is the waiting half alone (for kernels that announce a channel
// themselves when their last CTA finishes, see embed_scatter.cuh); dlb_peer_put
// is an all-gather by pushes: copy a buffer into this rank's slot on every rank,
// announce, wait.
#include "common.cuh"
#include "embed_scatter.cuh"

namespace dlb {
namespace {

struct PeerFlags {
  uint32_t *flags[kMaxPeers];
};

__global__ void __launch_bounds__(32)
peer_barrier_kernel(const __grid_constant__ PeerFlags pf, int n, int me, int channel, uint32_t epoch,
                    unsigned long long limit_ns, uint32_t *status, int do_signal) {
  pdl_prologue();
  const int r = threadIdx.x;
  if (do_signal && r < n) {
    __threadfence_system();
    uint32_t *theirs = pf.flags[r] + channel * kMaxPeers + me;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
  }
  wait_for_peers(pf.flags[me], n, channel, epoch, limit_ns, status);
}

// One CTA copies `n16` 16-byte words from src into this rank's slot of every rank's buffer, then
// announces the channel, then (optionally) waits until every rank has done the same: an
// all-gather by pushes, complete on this rank when the kernel ends.
struct PutArgs {
  const uint4 *src;
  uint4 *dst[kMaxPeers];  // already offset to this rank's slot
  size_t n16;
};

__global__ void __launch_bounds__(1024)
peer_put_kernel(const __grid_constant__ PutArgs a, const __grid_constant__ PeerFlags pf, int n, int me, int channel,
                uint32_t epoch, unsigned long long limit_ns, uint32_t *status, int wait) {
  pdl_prologue();
  for (int q = 0; q < n; q++)
    for (size_t i = threadIdx.x; i < a.n16; i += 1024) a.dst[q][i] = a.src[i];
  __syncthreads();  // orders every thread's stores before the fences below (a fence is cumulative)
  if (threadIdx.x < n) {
    __threadfence_system();
    uint32_t *theirs = pf.flags[threadIdx.x] + channel * kMaxPeers + me;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
  }
  if (wait) wait_for_peers(pf.flags[me], n, channel, epoch, limit_ns, status);
}

bool flags_ok(uint32_t *const *h_peer_flags, int n_ranks, PeerFlags *pf) {
  for (int r = 0; r < n_ranks; r++) {
    if (h_peer_flags[r] == nullptr) return false;
    pf->flags[r] = h_peer_flags[r];
  }
  return true;
}

}  // namespace
}  // namespace dlb

using namespace dlb;

extern "C" size_t dlb_peer_flags_bytes(void) { return sizeof(uint32_t) * kMaxPeers * kPeerChannels; }

static int barrier_like(const char *what, uint32_t *const *h_peer_flags, int n_ranks, int my_rank, int channel,
                        uint32_t epoch, int timeout_ms, uint32_t *d_status, int do_signal, void *stream) {
  DLB_REQUIRE(n_ranks >= 1 && n_ranks <= kMaxPeers && my_rank >= 0 && my_rank < n_ranks, DLB_ERR_INVALID_ARG,
              "%s: n_ranks=%d (1..%d) my_rank=%d", what, n_ranks, kMaxPeers, my_rank);
  DLB_REQUIRE(channel >= 0 && channel < kPeerChannels && timeout_ms > 0 && timeout_ms <= 10000, DLB_ERR_INVALID_ARG,
              "%s: channel=%d (0..%d) timeout_ms=%d (1..10000)", what, channel, kPeerChannels - 1, timeout_ms);
  DLB_REQUIRE(h_peer_flags && d_status, DLB_ERR_INVALID_ARG, "%s: null pointer", what);
  PeerFlags pf{};
  DLB_REQUIRE(flags_ok(h_peer_flags, n_ranks, &pf), DLB_ERR_INVALID_ARG, "%s: the flags of a rank are null", what);
  launch_pdl(peer_barrier_kernel, 1, 32, 0, as_stream(stream), pf, n_ranks, my_rank, channel, epoch,
             static_cast<unsigned long long>(timeout_ms) * 1000000ull, d_status, do_signal);
  DLB_LAUNCH_CHECK(what);
  return DLB_OK;
}

extern "C" int dlb_peer_barrier(uint32_t *const *h_peer_flags, int n_ranks, int my_rank, int channel,
                                uint32_t epoch, int timeout_ms, uint32_t *d_status, void *stream) {
  return barrier_like("peer_barrier", h_peer_flags, n_ranks, my_rank, channel, epoch, timeout_ms, d_status, 1, stream);
}

extern "C" int dlb_peer_wait(uint32_t *const *h_peer_flags, int n_ranks, int my_rank, int channel, uint32_t epoch,
                             int timeout_ms, uint32_t *d_status, void *stream) {
  return barrier_like("peer_wait", h_peer_flags, n_ranks, my_rank, channel, epoch, timeout_ms, d_status, 0, stream);
}

extern "C" int dlb_peer_put(const void *src, size_t bytes, void *const *h_peer_dst, uint32_t *const *h_peer_flags,
                            int n_ranks, int my_rank, int channel, uint32_t epoch, int wait, int timeout_ms,
                            uint32_t *d_status, void *stream) {
  DLB_REQUIRE(n_ranks >= 1 && n_ranks <= kMaxPeers && my_rank >= 0 && my_rank < n_ranks, DLB_ERR_INVALID_ARG,
              "peer_put: n_ranks=%d (1..%d) my_rank=%d", n_ranks, kMaxPeers, my_rank);
  DLB_REQUIRE(channel >= 0 && channel < kPeerChannels && timeout_ms > 0 && timeout_ms <= 10000, DLB_ERR_INVALID_ARG,
              "peer_put: channel=%d (0..%d) timeout_ms=%d (1..10000)", channel, kPeerChannels - 1, timeout_ms);
  DLB_REQUIRE(h_peer_dst && h_peer_flags && d_status && (src || bytes == 0), DLB_ERR_INVALID_ARG, "peer_put: null pointer");
  DLB_REQUIRE(bytes % 16 == 0 && aligned16(src), DLB_ERR_INVALID_ARG,
              "peer_put: %zu bytes: a multiple of 16 from a 16-byte aligned buffer required", bytes);
  PeerFlags pf{};
  DLB_REQUIRE(flags_ok(h_peer_flags, n_ranks, &pf), DLB_ERR_INVALID_ARG, "peer_put: the flags of a rank are null");
  PutArgs a{};
  a.src = static_cast<const uint4 *>(src);
  a.n16 = bytes / 16;
  for (int r = 0; r < n_ranks; r++) {
    DLB_REQUIRE(h_peer_dst[r] && aligned16(h_peer_dst[r]), DLB_ERR_INVALID_ARG,
                "peer_put: the destination of rank %d is null or unaligned", r);
    a.dst[r] = reinterpret_cast<uint4 *>(static_cast<char *>(h_peer_dst[r]) + static_cast<size_t>(my_rank) * bytes);
  }
  launch_pdl(peer_put_kernel, 1, 1024, 0, as_stream(stream), a, pf, n_ranks, my_rank, channel, epoch,
             static_cast<unsigned long long>(timeout_ms) * 1000000ull, d_status, wait);
  DLB_LAUNCH_CHECK("peer_put");
  return DLB_OK;
}
