/*
 * dlcuda_b200.h -- C ABI of the B200 (sm_100a) fused layer kernels.
 *
 * Every entry point takes raw DEVICE pointers (unless a parameter is named
 * h_*), plain integer sizes, a storage-type tag and a CUDA stream passed as
 * void* (a cudaStream_t; NULL = the legacy default stream).  Nothing here
 * allocates, frees, synchronises or exits: scratch memory is passed in by the
 * caller (its size comes from the matching *_workspace_bytes query) and every
 * call returns a dlb_status.  dlb_last_error() gives the text of the last
 * failure on the calling thread.
 *
 * Storage types.  DLB_F32: every tensor is float.  DLB_BF16: activation-sized
 * tensors (a, b, y, xhat, dy, dx, x, cache, embedding table, gather output)
 * are bfloat16, while parameters (gamma, beta, bias), the positional-encoding
 * table, inv_std, every gradient of a parameter and all arithmetic stay fp32.
 *
 * Each declaration cites the interface of Cameron-Lyons/dl-cuda that it
 * replaces (path inside that project : lines).
 */
#ifndef DLCUDA_B200_H
#define DLCUDA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define DLB_API __attribute__((visibility("default")))
#else
#define DLB_API
#endif

typedef enum dlb_status {
  DLB_OK = 0,
  DLB_ERR_INVALID_ARG = 1, /* null pointer, negative size, unknown enum      */
  DLB_ERR_WORKSPACE = 2,   /* workspace missing or smaller than required     */
  DLB_ERR_UNSUPPORTED = 3, /* shape outside what the kernels were built for  */
  DLB_ERR_CUDA = 4,        /* a CUDA runtime call or launch failed           */
  DLB_ERR_NO_DEVICE = 5    /* no CUDA device: there is no CPU fallback       */
} dlb_status;

typedef enum dlb_dtype { DLB_F32 = 0, DLB_BF16 = 1 } dlb_dtype;

typedef enum dlb_act {
  DLB_ACT_RELU = 0,
  DLB_ACT_SIGMOID = 1,
  DLB_ACT_TANH = 2,
  DLB_ACT_GELU = 3
} dlb_act;

/* ---- library ----------------------------------------------------------- */

DLB_API int dlb_version(void);
DLB_API const char *dlb_status_string(int status);
DLB_API const char *dlb_last_error(void);
/* Number of kernels this library has launched from the calling process since
 * load (every stream, every thread).  Used by benchmarks to report launches. */
DLB_API uint64_t dlb_launch_count(void);

/* Kernel-variant overrides for measurements: where a kernel exists in more than one form,
 * the heuristic's choice can be replaced so that both forms are timed in one process on the
 * same buffers.  value 0 gives the choice back to the heuristic; an override that does not
 * fit a call's shape is ignored for that call.  Results are the same whatever the choice
 * (except where an option says otherwise).
 *   "gather_rows_in_flight"      4 | 8   table rows a thread loads before its first store
 *   "gather_variant"             1 rows in registers | 2 the bulk-copy (TMA) pipeline
 *   "gather_bulk_ctas_per_sm"    1 one CTA per SM with a deeper ring (default 2)
 *   "gather_bulk_waves"          1..16: grid of the bulk-copy gather in units of the CTAs that fit the GPU
 *                                (default: about 450 KB of table rows per CTA)
 *   "ln_bwd_pipe"                1 never the bulk-copy pipeline | 2 whenever the shape allows
 *   "ln_bwd_pipe_threads"        128 | 256 | 512 column threads per CTA
 *   "ln_bwd_pipe_ctas_per_sm"    1 | 2
 *   "ln_bwd_pipe_rows_per_tile"  1 | 2 | 4 | 8
 *   "act_bwd_partial_rows"       upper bound of the partial rows of a fused bias gradient
 *   "scatter_variant"            1 rows in registers | 2 the bulk-copy (TMA) pipeline, for the
 *                                sorted-segment sums
 *   "scatter_bulk_ctas_per_sm"   1..6: its ring is sized for this many CTAs per SM (default 3)
 *   "scatter_zero_kernel"        1 the rows without tokens are cleared by a kernel of their own
 *                                that runs before the scatter-add
 *   "embed_push_period"          1..6: one CTA in this many of dlb_embed_scatter_bwd_peer's
 *                                second kernel pushes rows to the peers, the others clear rows
 *   "embed_peer_phases"          1 only the local sums | 2 only the push of
 *                                dlb_embed_scatter_bwd_peer (for timing the halves; results are
 *                                incomplete while it is set)
 * Process-wide, not synchronised with calls in flight.  No counterpart in the reference. */
DLB_API int dlb_set_option(const char *name, int value);

/* The pipelined kernels wait on shared-memory barriers for at most one second of
 * wall-clock time each; a wait that gives up lets the kernel finish (with wrong
 * results) and bumps a per-device counter instead of hanging the GPU.  This
 * call synchronises the whole device (cudaDeviceSynchronize: every stream,
 * non-blocking ones included) and returns that counter: 0 means every result
 * since load is good.  The layer classes call it from clip_grad_norm and
 * save_weights and exit when it is non-zero.  No counterpart in the reference. */
DLB_API int dlb_pipeline_timeouts(unsigned int *h_count);

/* ---- residual add -------------------------------------------------------
 * out[i] = a[i] + b[i].  out may alias a or b.
 * Replaces transformerResidualAddKernel (src/transformer.cuh:216-222) and
 * addVectorsKernel (src/layers.cuh:256-262) where they are used on their own;
 * the adds that feed a layer norm are folded into the calls below instead. */
DLB_API int dlb_residual_add(const void *a, const void *b, void *out, int64_t n,
                             int dtype, void *stream);

/* ---- layer norm with the residual add folded in --------------------------
 * Forward: s = a + b (b may be NULL: s = a); per row of d features
 *   mean = sum(s)/d; var = sum((s-mean)^2)/d (biased, two-pass);
 *   inv_std = 1/sqrtf(var+eps); xhat = (s-mean)*inv_std; y = gamma*xhat+beta.
 * xhat [rows,d] and inv_std [rows] are the caches backward needs; pass both
 * NULL for inference.  y may alias a or b.
 * Replaces transformerResidualAddKernel + layerNormForwardCachingKernel
 * (src/transformer.cuh:216-222, 136-164; call sites :499-507, :526-533). */
DLB_API int dlb_ln_residual_fwd(const void *a, const void *b, const float *gamma,
                                const float *beta, void *y, void *xhat,
                                float *inv_std, int rows, int d, float eps,
                                int dtype, void *stream);

/* Backward: dy = dy_a + dy_b (dy_b may be NULL);
 *   g = dy*gamma; c1 = mean(g); c2 = mean(g*xhat);
 *   dx = (g - c1 - xhat*c2)*inv_std;
 *   dgamma[j] = sum_rows dy*xhat; dbeta[j] = sum_rows dy   (overwritten).
 * One pass over dy/xhat; the column sums are reduced through `workspace` in a
 * fixed order, so results are bitwise reproducible.  dx may alias dy_a.
 * Replaces layerNormBackwardKernel + layerNormParamGradKernel and the gradient
 * residual add in front of them (src/transformer.cuh:166-207; call sites
 * :557-560, :583-585, :594-598). */
DLB_API size_t dlb_ln_bwd_workspace_bytes(int rows, int d);
DLB_API int dlb_ln_bwd(const void *dy_a, const void *dy_b, const void *xhat,
                       const float *inv_std, const float *gamma, void *dx,
                       float *dgamma, float *dbeta, void *workspace,
                       size_t workspace_bytes, int rows, int d, int dtype,
                       void *stream);

/* Layer-norm backward for callers that cannot allocate: same arguments and
 * results as dlb_ln_bwd, minus the workspace.  It is meant for hosts that are
 * handed their buffers by someone else and must not call cudaMalloc themselves
 * (a plugin inside another framework's memory pool, a latency-critical path, a
 * process with a memory budget fixed at start-up).  The scratch is a 16 MiB
 * array inside the library's device image (dlb_ln_bwd_noalloc_max_bytes()):
 * every GPU that loads the library holds it until the process exits.  Shapes
 * whose dlb_ln_bwd_workspace_bytes(rows, d) exceeds it (d > 2048 for up to
 * 262144 rows) are refused with DLB_ERR_UNSUPPORTED.  The call itself asks for
 * no memory: no cudaMalloc, no cudaFree, no allocating library routine.  The
 * first call on a device looks up the array's device address
 * (cudaGetSymbolAddress) and caches it; under CUDA's lazy module loading that
 * first lookup is also the moment the driver materialises the library's device
 * image, array included, on that GPU.  Make that first call before any stream
 * capture.  All calls share the one array and it keeps the
 * last call's contents; nothing in it has to start at zero (every partial row
 * is written before it is read), but two calls that overlap on the GPU (two
 * streams, two host threads) race on it -- order them.
 * This entry point has no counterpart in the reference. */
DLB_API size_t dlb_ln_bwd_noalloc_max_bytes(void);
DLB_API int dlb_ln_bwd_noalloc(const void *dy_a, const void *dy_b, const void *xhat,
                               const float *inv_std, const float *gamma, void *dx,
                               float *dgamma, float *dbeta, int rows, int d,
                               int dtype, void *stream);

/* ---- sinusoidal positional encoding --------------------------------------
 * h_table[pos*d + i] = (i even ? sinf : cosf)(pos / powf(10000, 2*(i/2)/d)),
 * built on the HOST with the C library's float functions, exactly as
 * PositionalEncoding's constructor does (src/positional_encoding.cuh:33-41). */
DLB_API int dlb_pe_build_table_host(float *h_table, int seq_len, int d);

/* out[i] = in[i] + pe[i mod (seq_len*d)] over batch*seq_len*d elements.
 * Replaces addPositionalEncodingKernel (src/positional_encoding.cuh:7-17). */
DLB_API int dlb_pe_add_fwd(const void *in, const float *pe, void *out, int batch,
                           int seq_len, int d, int dtype, void *stream);
/* dx = dy (identity).  Replaces the device-to-device copy in
 * PositionalEncoding::backward (src/positional_encoding.cuh:66-70). */
DLB_API int dlb_pe_add_bwd(const void *dy, void *dx, int64_t n, int dtype,
                           void *stream);

/* ---- token embedding ------------------------------------------------------
 * Gather with the positional-encoding add folded in:
 *   out[t,:] = table[ids[t],:] + (pe ? pe[(t mod seq_len),:] : 0).
 * ids are int32 in [0,vocab); the call does not validate them on the device.
 * Replaces embeddingForwardKernel (src/embedding.cuh:8-17) followed by
 * addPositionalEncodingKernel (src/positional_encoding.cuh:7-17). */
DLB_API int dlb_embed_gather_fwd(const void *table, const int32_t *ids,
                                 const float *pe, int seq_len, void *out,
                                 int num_tokens, int vocab, int d, int dtype,
                                 void *stream);

/* Gradient of the table: grad[v,:] = sum over tokens t with ids[t]==v of
 * dy[t,:]; rows no token refers to are written as zero (no separate memset).
 * The tokens are sorted by id (stable radix sort) and each output row is
 * summed in ascending token order, long rows through fixed-size sub-segments,
 * so the result does not depend on scheduling: two runs give identical bits.
 * grad is always fp32.  Replaces cudaMemset + embeddingBackwardKernel
 * (src/embedding.cuh:19-30, 82-92), whose fp32 atomicAdd order is arbitrary.
 *
 * dlb_embed_sort_tokens builds the sorted-segment plan from ids alone into
 * `workspace`; dlb_embed_scatter_bwd consumes it.  A plan stays valid for as
 * long as ids do, so a layer builds it once per batch. */
DLB_API size_t dlb_embed_workspace_bytes(int num_tokens, int vocab, int d);
DLB_API int dlb_embed_sort_tokens(const int32_t *ids, void *workspace,
                                  size_t workspace_bytes, int num_tokens,
                                  int vocab, int d, void *stream);
DLB_API int dlb_embed_scatter_bwd(const void *dy, const int32_t *ids,
                                  float *grad, void *workspace,
                                  size_t workspace_bytes, int num_tokens,
                                  int vocab, int d, int dtype, void *stream);

/* Multi-GPU form of the table gradient (token rows sharded over the ranks of one node; the
 * reference has no multi-GPU path, so these have no counterpart there -- they serve the
 * all-reduce of what src/embedding.cuh:82-92 produces).  Every rank gathers the ids of all
 * ranks (rank r holds tokens [r*tokens_per_rank, (r+1)*tokens_per_rank) of the gathered
 * list; the last rank may hold fewer) and sorts them once:
 *   dlb_embed_sort_tokens on the gathered ids  -> global plan (the same on every rank)
 *   dlb_embed_rank_plan(global plan, my_rank)  -> rank plan: the table rows ANY rank
 *       refers to ("used" rows) numbered 0..used-1 in ascending id ("slots", the same
 *       numbering on every rank), per slot this rank's tokens and the set of ranks that
 *       have tokens for it.  No second sort: a stable sort leaves each rank's tokens of a
 *       row contiguous.  The first int32 of the rank plan (device memory) is `used`.
 * Instead of all-reducing the dense [vocab, d] gradient, either
 *   dlb_embed_scatter_bwd_compact -> [used, d] buffer of this rank's sums (zeros for rows
 *       only other ranks use); all-reduce its first used*d floats; then
 *   dlb_embed_expand_rows(compact_rows, rank plan, grad, what): what&1 zero the rows no
 *       rank uses, what&2 copy the used rows (the zeroing needs only the plan, so it can
 *       run beside the all-reduce);
 * or the peer-memory exchange further down.  max_rows bounds the rows written (pass
 * min(vocab, all tokens) or the exact count); the exact count is read on the device, so
 * the host need not wait for the plan. */
DLB_API size_t dlb_embed_rank_plan_bytes(int vocab, int tokens_per_rank, int d);
DLB_API int dlb_embed_rank_plan(const void *global_plan, int global_tokens, int tokens_per_rank,
                                int n_ranks, int my_rank, void *rank_plan, size_t rank_plan_bytes,
                                int vocab, int d, void *stream);
DLB_API int dlb_embed_scatter_bwd_compact(const void *dy, const void *global_plan, int global_tokens,
                                          void *rank_plan, int tokens_per_rank, int my_rank,
                                          float *compact_rows, int max_rows, int vocab, int d,
                                          int dtype, void *stream);
DLB_API int dlb_embed_expand_rows(const float *compact_rows, const void *rank_plan,
                                  int tokens_per_rank, float *grad, int vocab, int d, int what,
                                  void *stream);

/* ---- bias + activation epilogues -------------------------------------------
 * Forward: pre = x + (bias ? bias[col] : 0); y = act(pre) over [rows,cols].
 *   RELU    y = pre>0 ? pre : 0           cache = 1 bit per element (pre>0)
 *   SIGMOID y = 1/(1+expf(-pre))          cache = y
 *   TANH    y = tanhf(pre)                cache = y
 *   GELU    y = pre*0.5*(1+tanhf(k(pre+0.044715 pre^3)))   cache = pre
 * `cache` is owned by the layer (dlb_act_cache_bytes), written in the same
 * pass, and may be NULL for inference.  y may alias x.
 * Backward: RELU dx = dy*(bit?1.0f:0.0f); SIGMOID dx = dy*s*(1-s);
 *   TANH dx = dy*(1-t*t); GELU as geluBackwardKernel.  When dbias is non-NULL
 *   dbias[col] = sum_rows dx (overwritten) is produced in the same pass through
 *   `workspace` (fixed order, reproducible).  dx may alias dy.
 * Replaces reluKernel/sigmoidKernel/tanhActivationKernel/geluForwardKernel and
 * their backward kernels with the cudaMemcpy cache copies around them
 * (src/activation.cuh:5-55, 75-118, 203-226, 278-289), tanhBackwardElementKernel
 * (src/layers.cuh:247-254), the bias add at the end of linearLayerKernel
 * (src/layers.cuh:34) and linearBackwardBiasKernel (src/layers.cuh:70-82). */
DLB_API size_t dlb_act_cache_bytes(int kind, int64_t n, int dtype);
DLB_API int dlb_act_fwd(int kind, const void *x, const float *bias, void *y,
                        void *cache, int64_t rows, int64_t cols, int dtype,
                        void *stream);
DLB_API size_t dlb_act_bwd_workspace_bytes(int kind, int64_t rows, int64_t cols);
DLB_API int dlb_act_bwd(int kind, const void *dy, const void *cache, void *dx,
                        float *dbias, void *workspace, size_t workspace_bytes,
                        int64_t rows, int64_t cols, int dtype, void *stream);

/* dbias[col] = sum_rows dy[row,col] on its own (fixed order, reproducible).
 * Replaces linearBackwardBiasKernel (src/layers.cuh:70-82). */
DLB_API size_t dlb_bias_grad_workspace_bytes(int64_t rows, int64_t cols);
DLB_API int dlb_bias_grad(const void *dy, float *dbias, void *workspace,
                          size_t workspace_bytes, int64_t rows, int64_t cols,
                          int dtype, void *stream);

/* ---- parameter update used by the layers themselves ------------------------
 * p[i] -= lr*g[i].  Replaces sgdUpdateKernel (src/layers.cuh:84-90), which
 * EmbeddingLayer::update_weights calls (src/embedding.cuh:94-99). */
DLB_API int dlb_sgd_update(float *params, const float *grads, float lr,
                           int64_t n, void *stream);

/* ---- optimizer steps and gradient clipping over a list of parameter groups ----
 * The h_* arrays are HOST arrays of n_groups device pointers / sizes (the
 * reference's ParamGroup list, src/sequential.cuh:19-23); one launch covers up
 * to 64 groups.
 *   DLB_OPT_SGD      p -= lr*g                                   (h_m, h_v unused)
 *   DLB_OPT_ADAM     m = b1*m+(1-b1)*g; v = b2*v+(1-b2)*g*g;
 *                    p -= lr * (m*inv_bc1) / (sqrtf(v*inv_bc2)+eps)
 *   DLB_OPT_ADAMW    ... p -= lr * (m_hat/(sqrtf(v_hat)+eps) + weight_decay*p)
 *   DLB_OPT_RMSPROP  s = b1*s+(1-b1)*g*g (s in h_m, decay in beta1);
 *                    p -= lr*g/(sqrtf(s)+eps)
 * inv_bias_correction{1,2} = 1/(1-beta^t) are computed by the caller, as the
 * reference's optimizer classes do.
 * Replaces sgdUpdateKernel (src/layers.cuh:84-90), updateRMSprop / updateAdam /
 * updateAdamW (src/optimizers.cuh:6-48) and the per-group launch loops of
 * src/optimizer.cuh:28-33, 78-92, 139-153, 187-195. */
typedef enum dlb_opt { DLB_OPT_SGD = 0, DLB_OPT_ADAM = 1, DLB_OPT_ADAMW = 2, DLB_OPT_RMSPROP = 3 } dlb_opt;
DLB_API int dlb_optim_step(int kind, int n_groups, float *const *h_params,
                           float *const *h_grads, float *const *h_m, float *const *h_v,
                           const int *h_sizes, float lr, float beta1, float beta2,
                           float eps, float weight_decay, float inv_bias_correction1,
                           float inv_bias_correction2, void *stream);

/* Global gradient norm and clipping without a host round trip:
 *   d_result[0] = sum of g*g over every group (fixed order, reproducible),
 *   d_result[1] = its square root, d_result[2] = the scale applied,
 * and, when max_norm > 0 and the norm exceeds it, every gradient is multiplied
 * by max_norm/(norm + 1e-6f) in place.  d_result is DEVICE memory (3 floats);
 * the caller reads d_result[1] back only if it wants the number.
 * Replaces the per-group thrust::transform_reduce + host sum and
 * clipGradsKernel of Sequential::clip_grad_norm (src/optimizer.cuh:205-233,
 * src/optimizers.cuh:50-55). */
DLB_API size_t dlb_grad_norm_workspace_bytes(void);
DLB_API int dlb_grad_norm_clip(int n_groups, float *const *h_grads, const int *h_sizes,
                               float max_norm, void *workspace, size_t workspace_bytes,
                               float *d_result, void *stream);

/* ---- checkpoint staging -----------------------------------------------------
 * The body of a DLCU weights file (everything after the 12-byte header 'DLCU',
 * int32 version, int32 group count; src/sequential.cuh:161-205) is, per
 * parameter group, one int32 size followed by that many floats.  pack writes
 * exactly those bytes into one device buffer in a single launch, so that saving
 * is ONE device-to-host copy instead of the reference's one per group
 * (src/sequential.cuh:190-200); unpack scatters a body that was uploaded with
 * ONE host-to-device copy back into the groups (the reference: :245-262).  The
 * size words of the body are written by pack and ignored by unpack (the host
 * validates them before uploading).  h_params / h_sizes are HOST arrays. */
DLB_API size_t dlb_checkpoint_body_bytes(int n_groups, const int *h_sizes);
DLB_API int dlb_checkpoint_pack(int n_groups, float *const *h_params, const int *h_sizes,
                                void *d_body, size_t body_bytes, void *stream);
DLB_API int dlb_checkpoint_unpack(int n_groups, float *const *h_params, const int *h_sizes,
                                  const void *d_body, size_t body_bytes, void *stream);

/* ---- multi-GPU: table gradient exchanged over peer memory (one node) ----------
 * No counterpart in the reference (it is single-GPU).  Alternative to the all-reduce of
 * the compacted rows: the scatter-add, the exchange and the expansion into the dense
 * table are fused into two kernels that signal and wait through flag words themselves.
 *
 * Every rank allocates, in memory that all ranks of the node have mapped (CUDA IPC,
 * cuMem fabric handles, torch symmetric memory ...):
 *   flags  dlb_peer_flags_bytes() bytes, zero before the first use
 *   recv   [n_ranks sources][cap_rows][d] fp32, the partial rows other ranks push
 *          (cap_rows * n_ranks must cover the used rows; no initial contents required)
 *   grad   the dense [vocab, d] fp32 table gradient (the result)
 *   small  [n_ranks][small_n] fp32 (optional): every rank's small parameter gradients
 * and fills a dlb_peer_group with the addresses of all ranks' buffers AS MAPPED ON THE
 * CALLING GPU (its own at index my_rank) plus a device status word of its own.
 *
 * dlb_embed_scatter_bwd_peer: (1) sums the rows this rank has several tokens for into a
 * buffer inside the rank plan (local, HBM-bound); (2) streams every row this rank has tokens
 * for to where it belongs, in a copy-shaped kernel that keeps NVLink full.  A row that ONLY
 * this rank has tokens for is final: it is stored straight into row v of every rank's grad
 * (a row with one token is read from dy itself).  A row several ranks share goes to the
 * receive area of the slot's owner (slot % n_ranks) at recv[my_rank][slot / n_ranks].  Rows
 * without local tokens send nothing.  With bf16 storage and staging areas given, a row whose
 * ONE token in all lies on this rank travels narrow: the peers get the token's bf16 row (half
 * the bytes) in stage[q][slot] and widen it themselves in the second call (0.0f + x is exact).
 * clear_unused = 1: the same kernel writes zeros into the rows of THIS rank's grad that no
 * rank uses.  clear_unused = 2: it clears only those of them that the PREVIOUS exchange wrote
 * (the rank plan workspace remembers them across steps; dlb_embed_reduce_broadcast_peer records
 * them): valid when nothing but these two calls writes the table between steps and the rank
 * plan workspace was zero-filled once before its first use; without a matching record it clears
 * everything, as 1 does.  clear_unused = 0: the caller clears (dlb_embed_expand_rows(what = 1)
 * on any stream once the rank plan is ready).  If `small` is given, its small_n floats are copied to
 * small[q][my_rank] on every rank q.  When the last CTA has issued its stores the kernel
 * announces (signal_channel, signal_epoch).  part = 0 does all of this in stream order.  To
 * overlap the sums with the pushes that do not need them, call it three times with the same
 * arguments: part = 1 (the sums alone) on a second stream, part = 2 (rows with one token, the
 * clearing, the small gradients; announces nothing) on the first, and, once part 1 has
 * finished (an event), part = 3 (the summed rows, then the announcement) on the first.
 *
 * dlb_embed_reduce_broadcast_peer: waits (bounded by timeout_ms) until every rank has
 * announced (wait_channel, wait_epoch); for each slot it owns that several ranks share it
 * adds the partial rows in rank order and stores the sum into row v of every rank's grad;
 * rows that arrived narrow are widened into this rank's own grad;
 * if small_out is given it receives the rank-order sum of the n_ranks small buffers (the
 * same bits on every rank).  Then it announces (signal_channel, signal_epoch); follow it
 * with dlb_peer_wait on that channel: after it every rank's table is complete.
 *
 * Epochs per channel grow by one per use, the same on all ranks.  A rank may start the
 * next step's dlb_embed_scatter_bwd_peer only when every rank is done with the tables of
 * this step (its consumer has run): the all-gather of the next step's ids (dlb_peer_put
 * with wait, stream-ordered after the consumer) is that barrier.  Status bits: bit c =
 * a wait on channel c gave up; bit 31 = cap_rows was too small for a slot (row dropped). */
#define DLB_MAX_PEERS 16
typedef struct dlb_peer_group {
  int n_ranks;                    /* 1..DLB_MAX_PEERS */
  int my_rank;
  int cap_rows;                   /* rows per source rank in a receive area */
  int small_n;                    /* floats per small-gradient buffer, a multiple of 4 (0: none) */
  int timeout_ms;                 /* bound of every wait inside the kernels, 1..10000 */
  int reserved;
  uint32_t *flags[DLB_MAX_PEERS]; /* per rank, as mapped on the calling GPU */
  float *recv[DLB_MAX_PEERS];
  float *grad[DLB_MAX_PEERS];
  float *small[DLB_MAX_PEERS];    /* may be NULL when small_n == 0 */
  void *stage[DLB_MAX_PEERS];     /* optional (all ranks or none): [cap_rows * n_ranks][d] rows of the
                                     STORAGE type, for rows that travel narrow (see below) */
  uint32_t *status;               /* this rank's device status word (zero before the first use) */
} dlb_peer_group;

DLB_API int dlb_embed_scatter_bwd_peer(const void *dy, const void *global_plan, int global_tokens,
                                       void *rank_plan, int tokens_per_rank,
                                       const dlb_peer_group *peers, const float *small, int max_rows,
                                       int clear_unused, int part, int vocab, int d, int dtype,
                                       int signal_channel, uint32_t signal_epoch, void *stream);
DLB_API int dlb_embed_reduce_broadcast_peer(void *rank_plan, int tokens_per_rank,
                                            const dlb_peer_group *peers, float *small_out, int vocab,
                                            int d, int dtype, int wait_channel, uint32_t wait_epoch,
                                            int signal_channel, uint32_t signal_epoch, void *stream);

/* Flags between the ranks' streams.  Every rank owns dlb_peer_flags_bytes() bytes of
 * zero-initialised memory that all ranks have mapped (h_peer_flags: HOST array of n_ranks
 * device addresses).  Per channel (0..3) epochs must be 1, 2, 3, ... in call order, the
 * same on all ranks.  Every wait gives up after timeout_ms: bit `channel` of *d_status
 * (device memory) is then set and the kernel returns; the caller checks it after
 * synchronising.  One rank per GPU: kernels that wait for one another must never share one.
 *   dlb_peer_barrier  announces `epoch` to every rank and waits until every rank has.
 *   dlb_peer_wait     the waiting half alone (the announcement came from a kernel).
 *   dlb_peer_put      an all-gather by pushes: copies `bytes` (a multiple of 16) from src
 *                     into h_peer_dst[q] + my_rank*bytes on every rank q, announces, and
 *                     with wait != 0 waits for every rank's announcement, so that this
 *                     rank's gathered buffer is complete when the kernel ends. */
DLB_API size_t dlb_peer_flags_bytes(void);
DLB_API int dlb_peer_barrier(uint32_t *const *h_peer_flags, int n_ranks, int my_rank,
                             int channel, uint32_t epoch, int timeout_ms, uint32_t *d_status,
                             void *stream);
DLB_API int dlb_peer_wait(uint32_t *const *h_peer_flags, int n_ranks, int my_rank, int channel,
                          uint32_t epoch, int timeout_ms, uint32_t *d_status, void *stream);
DLB_API int dlb_peer_put(const void *src, size_t bytes, void *const *h_peer_dst,
                         uint32_t *const *h_peer_flags, int n_ranks, int my_rank, int channel,
                         uint32_t epoch, int wait, int timeout_ms, uint32_t *d_status, void *stream);

/* ---- pass-through dense ops (fp32 only, correctness implementations) ----------
 * The matrix products, row softmax and loss kernels that the reference's
 * TransformerLayer / LinearLayer / SoftmaxActivation / loss helpers run between
 * the bandwidth-bound kernels above.  They are here so that a model built on
 * the reference's layer API runs end to end on this library; they use the fp32
 * pipes (no tensor cores) and keep the reference's per-element arithmetic: one
 * fused multiply-add per k in ascending k from 0, then alpha, bias, accumulate.
 *
 * dlb_gemm_f32: for every batch z (zo = z / batch_inner, zi = z % batch_inner)
 *   C[i*ldc + j] (+)= alpha * sum_kk A[i*a_row + kk*a_col] * B[kk*b_row + j*b_col] + bias[j]
 * with A, B, C offset by zo*x_outer + zi*x_inner elements; bias may be NULL;
 * accumulate != 0 adds the result to what C holds.  The strides let one launch
 * serve X*W (linearLayerKernel, src/layers.cuh:23-36), dY*W^T
 * (linearBackwardInputKernel :38-52, matMulBTKernel src/transformer.cuh:84-95),
 * X^T*dY (linearBackwardWeightKernel :54-68, matMulATKernel :97-108), and the
 * per-(batch, head) products of attnScoresKernel / attnApplyKernel (:8-19,
 * :47-58) over all heads at once, addressing heads inside [tokens, d_model]
 * by stride instead of through reshapeToHeadsKernel / reshapeFromHeadsKernel
 * (:110-134). */
DLB_API int dlb_gemm_f32(const float *a, const float *b, const float *bias, float *c,
                         int m, int n, int k, int64_t a_row, int64_t a_col,
                         int64_t b_row, int64_t b_col, int64_t ldc, int batch,
                         int batch_inner, int64_t a_outer, int64_t a_inner,
                         int64_t b_outer, int64_t b_inner, int64_t c_outer,
                         int64_t c_inner, float alpha, int accumulate, void *stream);

/* Row softmax, out may alias in.  causal_period > 0 keeps only the first
 * (row % causal_period) + 1 entries of each row and writes exact zeros after
 * them (applyCausalMaskKernel + softmaxForwardKernel, src/transformer.cuh:21-45);
 * 0 is the plain softmax of softmaxForwardGeneralKernel (src/activation.cuh:121-143). */
DLB_API int dlb_softmax_fwd(const float *in, float *out, int64_t rows, int width,
                            int causal_period, void *stream);
/* dx = s * (dy - sum_j dy_j*s_j) * scale; dx may alias dy.  Replaces
 * softmaxBackwardKernel + scaleBufferKernel (src/transformer.cuh:60-82, :209-214)
 * and softmaxBackwardGeneralKernel (src/activation.cuh:145-165). */
DLB_API int dlb_softmax_bwd(const float *dy, const float *s, float *dx, int64_t rows,
                            int width, float scale, void *stream);

/* Per-sample losses and their gradients, src/loss.cuh:18-109 (computeLoss /
 * computeLossBackward :146-202): error[n], grad[n] (grad[n*classes] for the
 * categorical loss), clamp epsilon 1e-10 as in the reference. */
typedef enum dlb_loss {
  DLB_LOSS_SQUARED = 0,
  DLB_LOSS_ABSOLUTE = 1,
  DLB_LOSS_BCE = 2,
  DLB_LOSS_CCE = 3
} dlb_loss;
DLB_API int dlb_loss_fwd(int kind, const float *y, const float *y_pred, float *error,
                         int64_t n, int classes, void *stream);
DLB_API int dlb_loss_bwd(int kind, const float *y, const float *y_pred, float *grad,
                         int64_t n, int classes, void *stream);
/* Cross entropy against integer targets: error[i] = -logf(max(p[i,target[i]], eps)),
 * grad[i,c] = c == target[i] ? -1/(max(p,eps)*n) : 0.  Replaces
 * categoricalCrossEntropyFromIdsKernel / ...BackwardFromIdsKernel
 * (src/loss.cuh:111-144, wrappers :204-221). */
DLB_API int dlb_ce_from_ids_fwd(const int32_t *target_ids, const float *y_pred,
                                float *error, int n, int classes, float epsilon,
                                void *stream);
DLB_API int dlb_ce_from_ids_bwd(const int32_t *target_ids, const float *y_pred,
                                float *grad, int n, int classes, float epsilon,
                                void *stream);

#ifdef __cplusplus
}
#endif
#endif /* DLCUDA_B200_H */
