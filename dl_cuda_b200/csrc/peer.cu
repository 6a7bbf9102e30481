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
#include "common.cuh"

namespace dlb {
namespace {

constexpr int kChannels = 4;

struct PeerFlags {
  uint32_t *flags[kMaxPeers];
};

__global__ void __launch_bounds__(32)
peer_barrier_kernel(const __grid_constant__ PeerFlags pf, int n, int me, int channel, uint32_t epoch,
                    unsigned long long limit_ns, uint32_t *status) {
  pdl_prologue();
  const int r = threadIdx.x;
  if (r >= n) return;
  __threadfence_system();
  uint32_t *theirs = pf.flags[r] + channel * kMaxPeers + me;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
  const uint32_t *mine = pf.flags[me] + channel * kMaxPeers + r;
  const unsigned long long start = global_ns();
  for (;;) {
    uint32_t seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
    if (static_cast<int32_t>(seen - epoch) >= 0) break;
    if (global_ns() - start > limit_ns) {
      atomicOr(status, 1u << channel);
      break;
    }
    __nanosleep(200);
  }
}

}  // namespace
}  // namespace dlb

using namespace dlb;

extern "C" size_t dlb_peer_flags_bytes(void) { return sizeof(uint32_t) * kMaxPeers * kChannels; }

extern "C" int dlb_peer_barrier(uint32_t *const *h_peer_flags, int n_ranks, int my_rank, int channel,
                                uint32_t epoch, int timeout_ms, uint32_t *d_status, void *stream) {
  DLB_REQUIRE(n_ranks >= 1 && n_ranks <= kMaxPeers && my_rank >= 0 && my_rank < n_ranks, DLB_ERR_INVALID_ARG,
              "peer_barrier: n_ranks=%d (1..%d) my_rank=%d", n_ranks, kMaxPeers, my_rank);
  DLB_REQUIRE(channel >= 0 && channel < kChannels && timeout_ms > 0 && timeout_ms <= 10000, DLB_ERR_INVALID_ARG,
              "peer_barrier: channel=%d (0..%d) timeout_ms=%d (1..10000)", channel, kChannels - 1, timeout_ms);
  DLB_REQUIRE(h_peer_flags && d_status, DLB_ERR_INVALID_ARG, "peer_barrier: null pointer");
  PeerFlags pf{};
  for (int r = 0; r < n_ranks; r++) {
    DLB_REQUIRE(h_peer_flags[r] != nullptr, DLB_ERR_INVALID_ARG, "peer_barrier: flags of rank %d are null", r);
    pf.flags[r] = h_peer_flags[r];
  }
  launch_pdl(peer_barrier_kernel, 1, 32, 0, as_stream(stream), pf, n_ranks, my_rank, channel, epoch,
             static_cast<unsigned long long>(timeout_ms) * 1000000ull, d_status);
  DLB_LAUNCH_CHECK("peer_barrier");
  return DLB_OK;
}
