"""torch-tensor front end of the C ABI, for tests and benchmarks.

Each function forwards to one entry point of libdlcuda_b200.so on the current
CUDA stream.  Outputs and workspaces can be passed in (benchmarks do, so that
nothing is allocated inside a timed region) or are allocated here.
"""
from __future__ import annotations

import torch

from . import capi
from .capi import check, current_stream, dtype_of, ptr


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("device tensors required: the kernels have no CPU path")
        if t is not None and not t.is_contiguous():
            raise ValueError("contiguous tensors required")


def _workspace(nbytes: int, device) -> torch.Tensor:
    # 256-byte aligned by the caching allocator (512-byte granularity).
    return torch.empty(max(nbytes, 16), dtype=torch.uint8, device=device)


def residual_add(a, b, out=None):
    _need_cuda(a, b, out)
    out = torch.empty_like(a) if out is None else out
    check(capi.lib().dlb_residual_add(ptr(a), ptr(b), ptr(out), a.numel(), dtype_of(a), current_stream()))
    return out


def ln_residual_fwd(a, b, gamma, beta, eps=1e-5, y=None, xhat=None, inv_std=None, cache=True):
    """Returns (y, xhat, inv_std); xhat/inv_std are None when cache is False."""
    _need_cuda(a, b, gamma, beta, y, xhat, inv_std)
    rows, d = a.shape
    y = torch.empty_like(a) if y is None else y
    if cache:
        xhat = torch.empty_like(a) if xhat is None else xhat
        inv_std = torch.empty(rows, dtype=torch.float32, device=a.device) if inv_std is None else inv_std
    else:
        xhat = inv_std = None
    check(capi.lib().dlb_ln_residual_fwd(ptr(a), ptr(b), ptr(gamma), ptr(beta), ptr(y), ptr(xhat),
                                         ptr(inv_std), rows, d, eps, dtype_of(a), current_stream()))
    return y, xhat, inv_std


def ln_bwd_workspace(rows, d, device):
    return _workspace(capi.lib().dlb_ln_bwd_workspace_bytes(rows, d), device)


def ln_bwd(dy_a, dy_b, xhat, inv_std, gamma, dx=None, dgamma=None, dbeta=None, workspace=None):
    """Returns (dx, dgamma, dbeta)."""
    _need_cuda(dy_a, dy_b, xhat, inv_std, gamma, dx, dgamma, dbeta)
    rows, d = dy_a.shape
    dx = torch.empty_like(dy_a) if dx is None else dx
    dgamma = torch.empty(d, dtype=torch.float32, device=dy_a.device) if dgamma is None else dgamma
    dbeta = torch.empty(d, dtype=torch.float32, device=dy_a.device) if dbeta is None else dbeta
    workspace = ln_bwd_workspace(rows, d, dy_a.device) if workspace is None else workspace
    check(capi.lib().dlb_ln_bwd(ptr(dy_a), ptr(dy_b), ptr(xhat), ptr(inv_std), ptr(gamma), ptr(dx),
                                ptr(dgamma), ptr(dbeta), ptr(workspace), workspace.numel(), rows, d,
                                dtype_of(dy_a), current_stream()))
    return dx, dgamma, dbeta


def pe_table(seq_len: int, d: int) -> torch.Tensor:
    """The sinusoidal table, built on the host (float powf/sinf/cosf), as a CPU tensor."""
    t = torch.empty(seq_len, d, dtype=torch.float32)
    check(capi.lib().dlb_pe_build_table_host(t.data_ptr(), seq_len, d))
    return t


def pe_add_fwd(x, pe, out=None):
    _need_cuda(x, pe, out)
    batch, seq_len, d = x.shape
    out = torch.empty_like(x) if out is None else out
    check(capi.lib().dlb_pe_add_fwd(ptr(x), ptr(pe), ptr(out), batch, seq_len, d, dtype_of(x), current_stream()))
    return out


def pe_add_bwd(dy, dx=None):
    _need_cuda(dy, dx)
    dx = torch.empty_like(dy) if dx is None else dx
    check(capi.lib().dlb_pe_add_bwd(ptr(dy), ptr(dx), dy.numel(), dtype_of(dy), current_stream()))
    return dx


def embed_gather_fwd(table, ids, pe=None, seq_len=0, out=None):
    _need_cuda(table, ids, pe, out)
    vocab, d = table.shape
    n = ids.numel()
    out = torch.empty(n, d, dtype=table.dtype, device=table.device) if out is None else out
    check(capi.lib().dlb_embed_gather_fwd(ptr(table), ptr(ids), ptr(pe), seq_len, ptr(out), n, vocab, d,
                                          dtype_of(table), current_stream()))
    return out


def embed_workspace(num_tokens, vocab, d, device):
    return _workspace(capi.lib().dlb_embed_workspace_bytes(num_tokens, vocab, d), device)


def embed_sort_tokens(ids, vocab, d, workspace=None):
    _need_cuda(ids)
    n = ids.numel()
    workspace = embed_workspace(n, vocab, d, ids.device) if workspace is None else workspace
    check(capi.lib().dlb_embed_sort_tokens(ptr(ids), ptr(workspace), workspace.numel(), n, vocab, d,
                                           current_stream()))
    return workspace


def embed_scatter_bwd(dy, ids, vocab, workspace, grad=None):
    """workspace must hold the plan embed_sort_tokens built for these ids."""
    _need_cuda(dy, ids, grad, workspace)
    n, d = dy.shape
    grad = torch.empty(vocab, d, dtype=torch.float32, device=dy.device) if grad is None else grad
    check(capi.lib().dlb_embed_scatter_bwd(ptr(dy), ptr(ids), ptr(grad), ptr(workspace), workspace.numel(),
                                           n, vocab, d, dtype_of(dy), current_stream()))
    return grad


def embed_rank_plan_workspace(vocab, tokens_per_rank, d, device):
    """Zero-filled: the workspace carries a record from one exchange to the next (see clear_unused = 2)."""
    return _workspace(capi.lib().dlb_embed_rank_plan_bytes(vocab, tokens_per_rank, d), device).zero_()


def embed_rank_plan(global_plan, global_tokens, tokens_per_rank, n_ranks, my_rank, vocab, d, rank_plan=None, stream=None):
    """Numbers the table rows any rank uses and finds this rank's tokens of each, from the plan of the
    gathered ids; rank_plan[:4].view(int32)[0] is the number of used rows (device)."""
    if rank_plan is None:
        rank_plan = embed_rank_plan_workspace(vocab, tokens_per_rank, d, global_plan.device)
    check(capi.lib().dlb_embed_rank_plan(ptr(global_plan), global_tokens, tokens_per_rank, n_ranks, my_rank,
                                         ptr(rank_plan), rank_plan.numel(), vocab, d,
                                         current_stream() if stream is None else stream))
    return rank_plan


def embed_scatter_bwd_compact(dy, global_plan, global_tokens, rank_plan, tokens_per_rank, my_rank, compact_rows, vocab,
                              stream=None):
    """compact_rows [max_rows, d]: the first `used` rows receive this rank's sums."""
    _need_cuda(dy, global_plan, rank_plan, compact_rows)
    d = dy.shape[1]
    check(capi.lib().dlb_embed_scatter_bwd_compact(ptr(dy), ptr(global_plan), global_tokens, ptr(rank_plan),
                                                   tokens_per_rank, my_rank, ptr(compact_rows), compact_rows.shape[0],
                                                   vocab, d, dtype_of(dy), current_stream() if stream is None else stream))
    return compact_rows


def embed_expand_rows(compact_rows, rank_plan, tokens_per_rank, grad, what=3, stream=None):
    vocab, d = grad.shape
    check(capi.lib().dlb_embed_expand_rows(ptr(compact_rows), ptr(rank_plan), tokens_per_rank, ptr(grad), vocab, d, what,
                                           current_stream() if stream is None else stream))
    return grad


def act_cache(kind, x):
    return _workspace(capi.lib().dlb_act_cache_bytes(kind, x.numel(), dtype_of(x)), x.device)


def act_fwd(kind, x, bias=None, y=None, cache=None, want_cache=True):
    """Returns (y, cache)."""
    _need_cuda(x, bias, y, cache)
    rows, cols = (x.shape[0], x.shape[1]) if x.dim() == 2 else (1, x.numel())
    y = torch.empty_like(x) if y is None else y
    if want_cache and cache is None:
        cache = act_cache(kind, x)
    check(capi.lib().dlb_act_fwd(kind, ptr(x), ptr(bias), ptr(y), ptr(cache) if want_cache else None,
                                 rows, cols, dtype_of(x), current_stream()))
    return y, cache


def act_bwd_workspace(kind, rows, cols, device):
    return _workspace(capi.lib().dlb_act_bwd_workspace_bytes(kind, rows, cols), device)


def act_bwd(kind, dy, cache, dx=None, dbias=None, want_dbias=False, workspace=None):
    """Returns (dx, dbias)."""
    _need_cuda(dy, cache, dx, dbias)
    rows, cols = (dy.shape[0], dy.shape[1]) if dy.dim() == 2 else (1, dy.numel())
    dx = torch.empty_like(dy) if dx is None else dx
    if want_dbias:
        dbias = torch.empty(cols, dtype=torch.float32, device=dy.device) if dbias is None else dbias
        workspace = act_bwd_workspace(kind, rows, cols, dy.device) if workspace is None else workspace
    else:
        dbias = None
    check(capi.lib().dlb_act_bwd(kind, ptr(dy), ptr(cache), ptr(dx), ptr(dbias), ptr(workspace),
                                 workspace.numel() if workspace is not None else 0, rows, cols,
                                 dtype_of(dy), current_stream()))
    return dx, dbias


def bias_grad(dy, dbias=None, workspace=None):
    _need_cuda(dy, dbias)
    rows, cols = dy.shape
    dbias = torch.empty(cols, dtype=torch.float32, device=dy.device) if dbias is None else dbias
    if workspace is None:
        workspace = _workspace(capi.lib().dlb_bias_grad_workspace_bytes(rows, cols), dy.device)
    check(capi.lib().dlb_bias_grad(ptr(dy), ptr(dbias), ptr(workspace), workspace.numel(), rows, cols,
                                   dtype_of(dy), current_stream()))
    return dbias


def sgd_update(params, grads, lr):
    _need_cuda(params, grads)
    check(capi.lib().dlb_sgd_update(ptr(params), ptr(grads), lr, params.numel(), current_stream()))
    return params


def _ptr_array(tensors):
    import ctypes
    arr = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() if t is not None else None for t in tensors])
    return arr


def optim_step(kind, params, grads, m=None, v=None, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01,
               step=1):
    """One optimizer step over lists of fp32 tensors (parameter groups), in place."""
    import ctypes
    n = len(params)
    sizes = (ctypes.c_int * n)(*[p.numel() for p in params])
    inv1 = 1.0 / (1.0 - beta1 ** step) if kind in (capi.OPT_ADAM, capi.OPT_ADAMW) else 1.0
    inv2 = 1.0 / (1.0 - beta2 ** step) if kind in (capi.OPT_ADAM, capi.OPT_ADAMW) else 1.0
    check(capi.lib().dlb_optim_step(kind, n, _ptr_array(params), _ptr_array(grads),
                                    _ptr_array(m) if m is not None else None,
                                    _ptr_array(v) if v is not None else None, sizes, lr, beta1, beta2, eps,
                                    weight_decay, inv1, inv2, current_stream()))


def grad_norm_clip(grads, max_norm=0.0, result=None, workspace=None):
    """Returns the device tensor {sum of squares, norm, applied scale}; clips in place when max_norm > 0."""
    import ctypes
    n = len(grads)
    device = grads[0].device if n else torch.device("cuda")
    sizes = (ctypes.c_int * n)(*[g.numel() for g in grads])
    result = torch.empty(3, dtype=torch.float32, device=device) if result is None else result
    workspace = _workspace(capi.lib().dlb_grad_norm_workspace_bytes(), device) if workspace is None else workspace
    check(capi.lib().dlb_grad_norm_clip(n, _ptr_array(grads), sizes, max_norm, ptr(workspace), workspace.numel(),
                                        ptr(result), current_stream()))
    return result


# --- pass-through dense ops (fp32) --------------------------------------------------
def gemm(a, b, bias=None, out=None, alpha=1.0, accumulate=False):
    """out (+)= alpha * a @ b + bias for fp32 tensors [M,K]·[K,N] or batched [Z,M,K]·[Z,K,N].

    ``a`` and ``b`` may be any strided views (transposes included); ``out`` is
    made contiguous if not given.
    """
    batched = a.dim() == 3
    a3 = a if batched else a.unsqueeze(0)
    b3 = b if batched else b.unsqueeze(0)
    z, m, k = a3.shape
    n = b3.shape[2]
    assert b3.shape[0] == z and b3.shape[1] == k and a.dtype == torch.float32 and b.dtype == torch.float32
    if out is None:
        assert not accumulate
        out = torch.empty((z, m, n) if batched else (m, n), dtype=torch.float32, device=a.device)
    o3 = out if batched else out.unsqueeze(0)
    assert o3.stride(2) == 1 or n == 1
    check(capi.lib().dlb_gemm_f32(ptr(a3), ptr(b3), ptr(bias) if bias is not None else None, ptr(o3), m, n, k,
                                  a3.stride(1), a3.stride(2), b3.stride(1), b3.stride(2), o3.stride(1), z, 1,
                                  a3.stride(0), 0, b3.stride(0), 0, o3.stride(0), 0, alpha, int(accumulate),
                                  current_stream()))
    return out


def softmax_fwd(x, out=None, causal_period=0):
    """Row softmax over the last dimension of a contiguous fp32 tensor."""
    out = torch.empty_like(x) if out is None else out
    width = x.shape[-1]
    check(capi.lib().dlb_softmax_fwd(ptr(x), ptr(out), x.numel() // width, width, causal_period, current_stream()))
    return out


def softmax_bwd(dy, s, dx=None, scale=1.0):
    dx = torch.empty_like(dy) if dx is None else dx
    width = dy.shape[-1]
    check(capi.lib().dlb_softmax_bwd(ptr(dy), ptr(s), ptr(dx), dy.numel() // width, width, scale, current_stream()))
    return dx


def loss_fwd(kind, y, y_pred, classes=1):
    n = y.numel() // classes if kind == capi.LOSS_CCE else y.numel()
    err = torch.empty(n, dtype=torch.float32, device=y.device)
    check(capi.lib().dlb_loss_fwd(kind, ptr(y), ptr(y_pred), ptr(err), n, classes, current_stream()))
    return err


def loss_bwd(kind, y, y_pred, classes=1):
    n = y.numel() // classes if kind == capi.LOSS_CCE else y.numel()
    grad = torch.empty_like(y_pred)
    check(capi.lib().dlb_loss_bwd(kind, ptr(y), ptr(y_pred), ptr(grad), n, classes, current_stream()))
    return grad


def ce_from_ids_fwd(target_ids, y_pred, eps=1e-10):
    n, classes = y_pred.shape
    err = torch.empty(n, dtype=torch.float32, device=y_pred.device)
    check(capi.lib().dlb_ce_from_ids_fwd(ptr(target_ids), ptr(y_pred), ptr(err), n, classes, eps, current_stream()))
    return err


def ce_from_ids_bwd(target_ids, y_pred, eps=1e-10):
    n, classes = y_pred.shape
    grad = torch.empty_like(y_pred)
    check(capi.lib().dlb_ce_from_ids_bwd(ptr(target_ids), ptr(y_pred), ptr(grad), n, classes, eps, current_stream()))
    return grad


# --- multi-GPU: table gradient over peer memory ---------------------------------------------
def _addr_array(addresses):
    """HOST array of device addresses (ints) for the h_* arguments of the peer entry points."""
    import ctypes
    return (ctypes.c_void_p * len(addresses))(*addresses)


def peer_group(n_ranks, my_rank, cap_rows, flags, recv, grad, status, small=None, small_n=0, timeout_ms=2000,
               stage=None):
    """A capi.PeerGroup from lists of device addresses (ints), one per rank, as mapped on this GPU."""
    import ctypes
    g = capi.PeerGroup()
    g.n_ranks, g.my_rank, g.cap_rows, g.small_n, g.timeout_ms = n_ranks, my_rank, cap_rows, small_n, timeout_ms
    for q in range(n_ranks):
        g.flags[q], g.recv[q], g.grad[q] = flags[q], recv[q], grad[q]
        g.small[q] = small[q] if small is not None else None
        g.stage[q] = stage[q] if stage is not None else None
    g.status = ptr(status)
    g._keepalive = status
    return g


def embed_scatter_bwd_peer(dy, global_plan, global_tokens, rank_plan, tokens_per_rank, group, small, max_rows, vocab,
                           channel, epoch, clear_unused=1, part=0, stream=None):
    """part: 0 everything in stream order; 1 the sums, 2 the first push, 3 the second push (see the header)."""
    import ctypes
    d = dy.shape[1]
    check(capi.lib().dlb_embed_scatter_bwd_peer(ptr(dy), ptr(global_plan), global_tokens, ptr(rank_plan), tokens_per_rank,
                                                ctypes.byref(group), ptr(small), max_rows, int(clear_unused), part, vocab,
                                                d, dtype_of(dy), channel, epoch,
                                                current_stream() if stream is None else stream))


def embed_reduce_broadcast_peer(rank_plan, tokens_per_rank, group, small_out, vocab, d, dtype, wait_channel, wait_epoch,
                                signal_channel, signal_epoch, stream=None):
    """dtype: the storage type of the gradients the scatter was given (capi.F32 / capi.BF16)."""
    import ctypes
    check(capi.lib().dlb_embed_reduce_broadcast_peer(ptr(rank_plan), tokens_per_rank, ctypes.byref(group), ptr(small_out),
                                                     vocab, d, dtype, wait_channel, wait_epoch, signal_channel,
                                                     signal_epoch, current_stream() if stream is None else stream))


def peer_barrier(peer_flags, my_rank, channel, epoch, status, timeout_ms=2000, stream=None):
    """peer_flags: device addresses (ints) of every rank's flag words; status: uint32/int32 device tensor [1]."""
    check(capi.lib().dlb_peer_barrier(_addr_array(peer_flags), len(peer_flags), my_rank, channel, epoch, timeout_ms,
                                      ptr(status), current_stream() if stream is None else stream))


def peer_wait(peer_flags, my_rank, channel, epoch, status, timeout_ms=2000, stream=None):
    check(capi.lib().dlb_peer_wait(_addr_array(peer_flags), len(peer_flags), my_rank, channel, epoch, timeout_ms,
                                   ptr(status), current_stream() if stream is None else stream))


def peer_put(src, peer_dst, peer_flags, my_rank, channel, epoch, status, wait=True, timeout_ms=2000, stream=None):
    """Copies `src` into slot my_rank of every rank's buffer (peer_dst: device addresses), announces, waits."""
    nbytes = src.numel() * src.element_size()
    check(capi.lib().dlb_peer_put(ptr(src), nbytes, _addr_array(peer_dst), _addr_array(peer_flags), len(peer_flags),
                                  my_rank, channel, epoch, int(wait), timeout_ms, ptr(status),
                                  current_stream() if stream is None else stream))


# --- checkpoint staging ---------------------------------------------------------------------
def checkpoint_pack(params):
    """The DLCU file body (per group: int32 size, then the floats) of a list of fp32 tensors, as a uint8 device tensor."""
    import ctypes
    n = len(params)
    sizes = (ctypes.c_int * n)(*[p.numel() for p in params])
    nbytes = capi.lib().dlb_checkpoint_body_bytes(n, sizes)
    body = torch.empty(nbytes, dtype=torch.uint8, device=params[0].device if n else "cuda")
    check(capi.lib().dlb_checkpoint_pack(n, _ptr_array(params), sizes, ptr(body), nbytes, current_stream()))
    return body


def checkpoint_unpack(body, params):
    """Scatters a DLCU file body (uint8 device tensor) into the fp32 tensors of `params`, in place."""
    import ctypes
    n = len(params)
    sizes = (ctypes.c_int * n)(*[p.numel() for p in params])
    check(capi.lib().dlb_checkpoint_unpack(n, _ptr_array(params), sizes, ptr(body), body.numel(), current_stream()))
