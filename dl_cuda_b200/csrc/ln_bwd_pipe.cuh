// Layer-norm backward as a bulk-copy (TMA) pipeline, for rows wide enough that
// holding them in registers across a CTA costs occupancy.
//
// Persistent CTAs, three roles that meet only at mbarriers (no CTA-wide barrier
// inside the loop):
//   producer (1 thread)  streams tiles of RT whole rows of dy (one or two
//                        gradient streams) and xhat into a ring of shared-memory
//                        stages with cp.async.bulk;
//   column warps (CT threads)  each thread owns KV 16-byte column vectors for the
//                        whole kernel.  Per tile it makes two passes over its
//                        columns in shared memory.  Pass A (one tile ahead):
//                        partial row sums of dy*gamma and dy*gamma*xhat, reduced
//                        inside the warp and published per warp, plus the
//                        dgamma/dbeta sums of its columns, kept in registers.
//                        Pass B: dx, once the row sums are complete;
//   reducer (1 warp)     adds the per-warp partial sums of a tile in warp order
//                        and leaves, per row, inv_std and the two sums already
//                        scaled by it.
// Pass A of tile i+1 overlaps the wait for the row sums of tile i, so no warp
// idles on another; the bytes in flight are set by the ring depth, not by the
// register file.  dx = (g - c1 - xhat*c2)*inv_std is evaluated as
// g*inv_std - c1*inv_std - xhat*(c2*inv_std).  Each CTA ends by writing one
// partial row [2*d]; colsum_finalize adds the partial rows in CTA order.
#pragma once

#include "common.cuh"
#include "tma.cuh"

namespace dlb {

constexpr int kPipeMaxStages = 8;
constexpr size_t kPipeSmemPerSm = 216 * 1024;

struct PipeLayout {
  int stages;
  unsigned op_bytes, stage_bytes;              // one operand of a tile; all operands of a tile
  unsigned psum_off, stats_off, bar_off, total;
};

// Sums N values (N a power of two <= 32) across the warp with N+3 shuffles
// instead of 5N: each step halves the number of values a lane carries.  Lane l
// ends with the total of value l >> (5 - log2 N); the order of the additions is
// fixed.
template <int N>
__device__ __forceinline__ float warp_sum_many(float (&v)[N], int lane) {
  int o = 16;
#pragma unroll
  for (int n = N; n > 1; n >>= 1, o >>= 1) {
    const int half = n >> 1;
    const bool up = (lane & o) != 0;
#pragma unroll
    for (int i = 0; i < half; i++) {
      const float send = up ? v[i] : v[i + half];
      const float keep = up ? v[i + half] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
    }
  }
  float r = v[0];
#pragma unroll
  for (; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  return r;
}

template <int N>
struct Log2;
template <> struct Log2<1> { static constexpr int v = 0; };
template <> struct Log2<2> { static constexpr int v = 1; };
template <> struct Log2<4> { static constexpr int v = 2; };
template <> struct Log2<8> { static constexpr int v = 3; };
template <> struct Log2<16> { static constexpr int v = 4; };

template <typename T, int CT, int KV, int RT, int MINB>
__global__ void __launch_bounds__(CT + 64, MINB)
ln_bwd_pipe_kernel(const T *dy_a, const T *dy_b, const T *xhat,
                   const float *inv_std, const float *gamma, T *dx,
                   float *__restrict__ partial, int rows, int d, PipeLayout L,
                   unsigned int *timeouts) {
  pdl_prologue();
  using S = Store<T>;
  constexpr int E = S::kPerVec;
  constexpr int kColWarps = CT / 32;
  constexpr int NS = 2 * RT;  // row sums per tile
  extern __shared__ __align__(128) unsigned char smem_raw[];

  const bool has_b = dy_b != nullptr;
  const int nops = has_b ? 3 : 2;
  unsigned char *ring = smem_raw;
  float *psum = reinterpret_cast<float *>(smem_raw + L.psum_off);       // [stages][kColWarps][NS]
  float4 *stats = reinterpret_cast<float4 *>(smem_raw + L.stats_off);   // [stages][RT] {inv_std, c1*is, c2*is, -}
  uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw + L.bar_off);  // [kPipeMaxStages] each
  uint64_t *sums = full + kPipeMaxStages;
  uint64_t *ready = sums + kPipeMaxStages;
  uint64_t *empty = ready + kPipeMaxStages;
  volatile int *dead = reinterpret_cast<volatile int *>(empty + kPipeMaxStages);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int stages = L.stages;
  const int ntiles = (rows + RT - 1) / RT;
  const int ncv = d / E;

  if (tid == 0) {
    for (int s = 0; s < stages; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&sums[s], kColWarps);
      mbar_init(&ready[s], 1);
      mbar_init(&empty[s], kColWarps);
    }
    *dead = 0;
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == kColWarps + 1) {
    // ---------------------------------------------------------- producer
    if (lane == 0) {
      int it = 0;
      for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
        const int s = it % stages;
        // First lap: the barrier is fresh, waiting for parity 1 returns at once.
        mbar_wait(&empty[s], ((it / stages) & 1) ^ 1, dead, timeouts);
        const int row0 = tile * RT;
        const int nrows = min(RT, rows - row0);
        const unsigned bytes = static_cast<unsigned>(static_cast<size_t>(nrows) * d * sizeof(T));
        const size_t goff = static_cast<size_t>(row0) * d;
        unsigned char *dst = ring + static_cast<size_t>(L.stage_bytes) * s;
        mbar_expect_tx(&full[s], bytes * nops);
        bulk_load(dst, dy_a + goff, bytes, &full[s]);
        bulk_load(dst + L.op_bytes, xhat + goff, bytes, &full[s]);
        if (has_b) bulk_load(dst + 2 * L.op_bytes, dy_b + goff, bytes, &full[s]);
      }
    }
    return;
  }

  if (warp == kColWarps) {
    // ----------------------------------------------------------- reducer
    // Lane j < NS owns row sum j (j = 2r: sum of g, j = 2r+1: sum of g*xhat).
    int it = 0;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
      const int s = it % stages;
      const int row = tile * RT + (lane >> 1);
      const float is = (lane < NS && row < rows) ? ld_co(inv_std + row) : 0.f;
      mbar_wait(&sums[s], (it / stages) & 1, dead, timeouts);
      if (lane < NS) {
        const float *p = psum + (static_cast<size_t>(s) * kColWarps) * NS + lane;
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < kColWarps; w++) t += p[w * NS];
        float *out = reinterpret_cast<float *>(&stats[s * RT + (lane >> 1)]);
        const float scaled = (t / d) * is;
        if ((lane & 1) == 0) {
          out[0] = is;
          out[1] = scaled;
        } else {
          out[2] = scaled;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&ready[s]);
    }
    return;
  }

  // --------------------------------------------------------- column warps
  float gv[KV][E];
#pragma unroll
  for (int k = 0; k < KV; k++) {
    const int cv = tid + k * CT;
#pragma unroll
    for (int q = 0; q < E / 4; q++) {
      float4 g4 = make_float4(0.f, 0.f, 0.f, 0.f);
      if (cv < ncv) g4 = ld_keep_f4(gamma + cv * E + 4 * q);
      gv[k][4 * q] = g4.x; gv[k][4 * q + 1] = g4.y; gv[k][4 * q + 2] = g4.z; gv[k][4 * q + 3] = g4.w;
    }
  }
  float accg[KV][E], accb[KV][E];
#pragma unroll
  for (int k = 0; k < KV; k++)
#pragma unroll
    for (int e = 0; e < E; e++) accg[k][e] = accb[k][e] = 0.f;

  // Pass A over the tile in stage s: row sums (published per warp) and column sums.
  auto pass_a = [&](int s, int nrows) {
    const unsigned char *src = ring + static_cast<size_t>(L.stage_bytes) * s;
    float c[NS];
#pragma unroll
    for (int j = 0; j < NS; j++) c[j] = 0.f;
#pragma unroll
    for (int r = 0; r < RT; r++) {
      if (r < nrows) {
        const unsigned char *row = src + static_cast<size_t>(r) * d * sizeof(T);
#pragma unroll
        for (int k = 0; k < KV; k++) {
          const int cv = tid + k * CT;
          if (cv < ncv) {
            float dyv[E], xv[E];
            S::unpack(lds128(row + static_cast<size_t>(cv) * 16), dyv);
            S::unpack(lds128(row + L.op_bytes + static_cast<size_t>(cv) * 16), xv);
            if (has_b) {
              float t[E];
              S::unpack(lds128(row + 2 * L.op_bytes + static_cast<size_t>(cv) * 16), t);
#pragma unroll
              for (int e = 0; e < E; e++) dyv[e] += t[e];
            }
#pragma unroll
            for (int e = 0; e < E; e++) {
              const float g = dyv[e] * gv[k][e];
              c[2 * r] += g;
              c[2 * r + 1] += g * xv[e];
              accg[k][e] += dyv[e] * xv[e];
              accb[k][e] += dyv[e];
            }
          }
        }
      }
    }
    const float total = warp_sum_many<NS>(c, lane);
    constexpr int kShift = 5 - Log2<NS>::v;
    if ((lane & ((1 << kShift) - 1)) == 0)
      psum[(static_cast<size_t>(s) * kColWarps + warp) * NS + (lane >> kShift)] = total;
    __syncwarp();
    if (lane == 0) mbar_arrive(&sums[s]);
  };

  int it = 0;
  const int tile0 = blockIdx.x;
  if (tile0 < ntiles) {
    mbar_wait(&full[0], 0, dead, timeouts);
    pass_a(0, min(RT, rows - tile0 * RT));
  }
  for (int tile = tile0; tile < ntiles; tile += gridDim.x, ++it) {
    const int next = tile + gridDim.x;
    if (next < ntiles) {
      const int s1 = (it + 1) % stages;
      mbar_wait(&full[s1], ((it + 1) / stages) & 1, dead, timeouts);
      pass_a(s1, min(RT, rows - next * RT));
    }
    const int s = it % stages;
    const int row0 = tile * RT;
    const int nrows = min(RT, rows - row0);
    mbar_wait(&ready[s], (it / stages) & 1, dead, timeouts);
    const unsigned char *src = ring + static_cast<size_t>(L.stage_bytes) * s;
#pragma unroll
    for (int r = 0; r < RT; r++) {
      if (r < nrows) {
        const float4 st = stats[s * RT + r];  // {inv_std, c1*inv_std, c2*inv_std}
        const unsigned char *row = src + static_cast<size_t>(r) * d * sizeof(T);
#pragma unroll
        for (int k = 0; k < KV; k++) {
          const int cv = tid + k * CT;
          if (cv < ncv) {
            float dyv[E], xv[E], o[E];
            S::unpack(lds128(row + static_cast<size_t>(cv) * 16), dyv);
            S::unpack(lds128(row + L.op_bytes + static_cast<size_t>(cv) * 16), xv);
            if (has_b) {
              float t[E];
              S::unpack(lds128(row + 2 * L.op_bytes + static_cast<size_t>(cv) * 16), t);
#pragma unroll
              for (int e = 0; e < E; e++) dyv[e] += t[e];
            }
#pragma unroll
            for (int e = 0; e < E; e++) {
              const float g = dyv[e] * gv[k][e];
              o[e] = fmaf(-xv[e], st.z, fmaf(g, st.x, -st.y));
            }
            st_stream(dx + static_cast<size_t>(row0 + r) * d + static_cast<size_t>(cv) * E, S::pack(o));
          }
        }
      }
    }
    // This warp is done with the stage (its reads have returned): hand it back.
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
  }

  // After a wait gave up, copies may still be landing in this CTA's shared
  // memory: let them finish before the CTA retires.
  if (*dead) {
    for (int i = 0; i < 1000; i++) __nanosleep(1000);
  }

  // Thread-owned columns: the CTA's partial row needs no further reduction.
#pragma unroll
  for (int k = 0; k < KV; k++) {
    const int cv = tid + k * CT;
    if (cv < ncv) {
      float *pg = partial + (static_cast<size_t>(blockIdx.x) * 2) * d + cv * E;
      float *pbeta = pg + d;
#pragma unroll
      for (int q = 0; q < E / 4; q++) {
        *reinterpret_cast<float4 *>(pg + 4 * q) =
            make_float4(accg[k][4 * q], accg[k][4 * q + 1], accg[k][4 * q + 2], accg[k][4 * q + 3]);
        *reinterpret_cast<float4 *>(pbeta + 4 * q) =
            make_float4(accb[k][4 * q], accb[k][4 * q + 1], accb[k][4 * q + 2], accb[k][4 * q + 3]);
      }
    }
  }
}

struct PipeShape {
  int ct = 0, kv = 0, rt = 0, ctas_per_sm = 1;
  PipeLayout layout{};
};

// Picks column threads, vectors per thread, rows per tile, CTAs per SM and ring
// depth, or ct == 0 when the row is too narrow or too wide for this kernel.
template <typename T>
PipeShape pick_pipe_shape(int rows, int d, bool two_grads, bool aligned) {
  constexpr int E = Store<T>::kPerVec;
  PipeShape p;
  if (!aligned || d % E != 0) return p;
  const int ncv = d / E;
  if (ncv < 128) return p;
  // Column threads per CTA, measured on B200: bf16 rows of 512 vectors and more run best with 512
  // threads, one vector each, one CTA per SM (32768 x 4096: 133 against 138 us); fp32 rows of 256
  // vectors with 128 threads, two vectors each (65536 x 1024: 128 against 140 us).
  int ct = ncv >= 256 ? 256 : 128;
  if (E == 8 && ncv >= 512) ct = 512;
  if (E == 4 && ncv == 256) ct = 128;
  const int want_ct = get_option("ln_bwd_pipe_threads");
  if ((want_ct == 128 || want_ct == 256 || want_ct == 512) && want_ct <= ncv) ct = want_ct;
  int kv = 1;
  while (kv * ct < ncv) kv *= 2;
  if (kv > 4) return p;
  const size_t row_bytes = static_cast<size_t>(d) * sizeof(T) * (two_grads ? 3 : 2);
  // Rows per tile: a stage of about 32 KB, bounded by what the kernels are built for.
  const int rt_max = kv == 1 ? 8 : (kv == 2 ? 4 : 2);
  int rt = rt_max;
  while (rt > 1 && rt * row_bytes > 40 * 1024) rt /= 2;
  if (kv == 1 && rt < 2) rt = 2;
  if (ct == 512 && kv == 1 && !two_grads && 4 * row_bytes <= 64 * 1024) rt = 4;  // 64 KB stages, three of them
  const int want_rt = get_option("ln_bwd_pipe_rows_per_tile");
  if ((want_rt == 1 || want_rt == 2 || want_rt == 4 || want_rt == 8) && want_rt <= rt_max && !(kv == 1 && want_rt < 2))
    rt = want_rt;
  int max_stages = kPipeMaxStages;
  int ctas = (kv <= 2 || sizeof(T) == 4) ? 2 : 1;  // all but the widest bf16 variant fit two CTAs per SM in registers
  if (ct == 512) ctas = 1;  // 576 threads: one CTA per SM keeps 18 warps and the whole ring
  const int want_ctas = get_option("ln_bwd_pipe_ctas_per_sm");
  if (want_ctas == 1) ctas = 1;
  PipeLayout &L = p.layout;
  L.op_bytes = static_cast<unsigned>(static_cast<size_t>(rt) * d * sizeof(T));
  L.stage_bytes = L.op_bytes * (two_grads ? 3 : 2);
  const size_t fixed = sizeof(float) * kPipeMaxStages * (ct / 32) * 2 * rt + sizeof(float4) * kPipeMaxStages * rt +
                       sizeof(uint64_t) * 4 * kPipeMaxStages + 64 + 1024 /* per-CTA reserve of the driver */;
  for (; ctas >= 1; ctas--) {
    const size_t budget = kPipeSmemPerSm / ctas;
    if (static_cast<size_t>(L.stage_bytes) * 3 + fixed <= budget || (ctas == 1 && static_cast<size_t>(L.stage_bytes) * 2 + fixed <= budget)) {
      int stages = static_cast<int>((budget - fixed) / L.stage_bytes);
      L.stages = stages > max_stages ? max_stages : stages;
      break;
    }
  }
  if (ctas < 1) return p;
  L.psum_off = L.stage_bytes * L.stages;
  L.stats_off = L.psum_off + static_cast<unsigned>(sizeof(float)) * kPipeMaxStages * (ct / 32) * 2 * rt;
  L.bar_off = L.stats_off + static_cast<unsigned>(sizeof(float4)) * kPipeMaxStages * rt;
  L.total = L.bar_off + static_cast<unsigned>(sizeof(uint64_t)) * 4 * kPipeMaxStages + 64;
  // Worth it only when every CTA gets a few tiles.
  const int mode = get_option("ln_bwd_pipe");
  if (mode == 1) return p;
  if (mode != 2 && ceil_div(rows, rt) < 2 * sm_count() * ctas) return p;
  p.ct = ct;
  p.kv = kv;
  p.rt = rt;
  p.ctas_per_sm = ctas;
  return p;
}

template <typename T, int CT, int KV, int RT>
int launch_ln_bwd_pipe(const PipeShape &p, const void *dy_a, const void *dy_b, const void *xhat,
                       const float *inv_std, const float *gamma, void *dx, float *partial,
                       int *n_partial, int rows, int d, cudaStream_t st) {
  constexpr int MINB = (CT <= 256 && (KV <= 2 || sizeof(T) == 4)) ? 2 : 1;
  auto kern = ln_bwd_pipe_kernel<T, CT, KV, RT, MINB>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(p.layout.total));
  DLB_REQUIRE(e == cudaSuccess, DLB_ERR_CUDA, "ln_bwd: shared memory attribute: %s", cudaGetErrorString(e));
  unsigned int *timeouts = wait_timeouts_counter();
  DLB_REQUIRE(timeouts != nullptr, DLB_ERR_CUDA, "ln_bwd: no timeout counter on this device");
  const int grid = min(sm_count() * p.ctas_per_sm, ceil_div(rows, RT));
  launch_pdl(kern, grid, CT + 64, p.layout.total, st, 
      static_cast<const T *>(dy_a), static_cast<const T *>(dy_b), static_cast<const T *>(xhat), inv_std,
      gamma, static_cast<T *>(dx), partial, rows, d, p.layout, timeouts);
  DLB_LAUNCH_CHECK("ln_bwd_pipe");
  *n_partial = grid;
  return DLB_OK;
}

// (CT, KV, RT) combinations pick_pipe_shape can return.
#define DLB_PIPE_CASES(M)                                         \
  M(128, 1, 2) M(128, 1, 4) M(128, 1, 8) M(128, 2, 1) M(128, 2, 2) M(128, 2, 4) M(128, 4, 1) M(128, 4, 2) \
  M(256, 1, 2) M(256, 1, 4) M(256, 1, 8) M(256, 2, 1) M(256, 2, 2) M(256, 2, 4) M(256, 4, 1) M(256, 4, 2) \
  M(512, 1, 2) M(512, 1, 4) M(512, 1, 8) M(512, 2, 1) M(512, 2, 2) M(512, 2, 4)

}  // namespace dlb
