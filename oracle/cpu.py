"""TEST INFRASTRUCTURE: numpy front end of oracle/host_ref.cpp (liboracle.so).

Every function takes and returns C-contiguous numpy arrays (float32 unless
said otherwise) and runs single-threaded on the host.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "_build" / "liboracle.so"
SUB_LEN = 32  # tokens per sub-segment of the CUDA scatter-add (kSubLen in csrc/embedding.cu)
SLICES = 8    # groups of sub-segments added separately (kCombineSlices in csrc/embedding.cu)

_lib = None


def build() -> Path:
    subprocess.run(["make", "-s", "-C", str(HERE), "oracle"], check=True)
    return LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            build()
        _lib = C.CDLL(str(LIB_PATH))
    return _lib


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a


def _p(a):
    return None if a is None else C.c_void_p(a.ctypes.data)


def residual_add(a, b):
    a, b = _f(a), _f(b)
    out = np.empty_like(a)
    lib().orc_residual_add(_p(a), _p(b), _p(out), C.c_int64(a.size))
    return out


def ln_residual_fwd(a, b, gamma, beta, eps=1e-5):
    """Returns (y, xhat, inv_std)."""
    a, gamma, beta = _f(a), _f(gamma), _f(beta)
    b = None if b is None else _f(b)
    rows, d = a.shape
    y, xhat = np.empty_like(a), np.empty_like(a)
    inv_std = np.empty(rows, np.float32)
    lib().orc_ln_residual_fwd(_p(a), _p(b), _p(gamma), _p(beta), _p(y), _p(xhat), _p(inv_std),
                              rows, d, C.c_float(eps))
    return y, xhat, inv_std


def ln_bwd(dy_a, dy_b, xhat, inv_std, gamma):
    """Returns (dx, dgamma, dbeta) in the reference's fp32 order."""
    dy_a, xhat, inv_std, gamma = _f(dy_a), _f(xhat), _f(inv_std), _f(gamma)
    dy_b = None if dy_b is None else _f(dy_b)
    rows, d = dy_a.shape
    dx = np.empty_like(dy_a)
    dgamma, dbeta = np.empty(d, np.float32), np.empty(d, np.float32)
    lib().orc_ln_bwd_dx(_p(dy_a), _p(dy_b), _p(xhat), _p(inv_std), _p(gamma), _p(dx), rows, d)
    lib().orc_ln_param_grad(_p(dy_a), _p(dy_b), _p(xhat), _p(dgamma), _p(dbeta), rows, d)
    return dx, dgamma, dbeta


def ln_param_grad_f64(dy_a, dy_b, xhat):
    dy_a, xhat = _f(dy_a), _f(xhat)
    dy_b = None if dy_b is None else _f(dy_b)
    rows, d = dy_a.shape
    dgamma, dbeta = np.empty(d, np.float64), np.empty(d, np.float64)
    lib().orc_ln_param_grad_f64(_p(dy_a), _p(dy_b), _p(xhat), _p(dgamma), _p(dbeta), rows, d)
    return dgamma, dbeta


def pe_table(seq_len, d):
    t = np.empty((seq_len, d), np.float32)
    lib().orc_pe_table(_p(t), seq_len, d)
    return t


def pe_add(x, pe):
    x, pe = _f(x), _f(pe)
    batch, seq_len, d = x.shape
    out = np.empty_like(x)
    lib().orc_pe_add(_p(x), _p(pe), _p(out), batch, seq_len, d)
    return out


def embed_gather(table, ids, pe=None, seq_len=0):
    table = _f(table)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    pe = None if pe is None else _f(pe)
    out = np.empty((ids.size, table.shape[1]), np.float32)
    lib().orc_embed_gather(_p(table), _p(ids), _p(pe), seq_len, _p(out), ids.size, table.shape[1])
    return out


def embed_scatter(dy, ids, vocab, mode="sequential"):
    """mode: 'sequential' (ascending tokens), 'segmented' (the CUDA kernel's association), 'f64'."""
    dy = _f(dy)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    n, d = dy.shape
    if mode == "f64":
        grad = np.empty((vocab, d), np.float64)
        lib().orc_embed_scatter_f64(_p(dy), _p(ids), _p(grad), n, vocab, d)
    elif mode == "segmented":
        grad = np.empty((vocab, d), np.float32)
        lib().orc_embed_scatter_segmented(_p(dy), _p(ids), _p(grad), n, vocab, d, SUB_LEN, SLICES)
    else:
        grad = np.empty((vocab, d), np.float32)
        lib().orc_embed_scatter(_p(dy), _p(ids), _p(grad), n, vocab, d)
    return grad


def act_fwd(kind, x, bias=None):
    """Returns (y, pre) with pre = x + bias."""
    x = _f(x)
    bias = None if bias is None else _f(bias)
    rows, cols = (x.shape[0], x.shape[1]) if x.ndim == 2 else (1, x.size)
    y, pre = np.empty_like(x), np.empty_like(x)
    lib().orc_act_fwd(kind, _p(x), _p(bias), _p(y), _p(pre), C.c_int64(rows), C.c_int64(cols))
    return y, pre


def act_bwd(kind, dy, cache):
    """cache: forward input (pre) for relu/gelu, forward output for sigmoid/tanh."""
    dy, cache = _f(dy), _f(cache)
    dx = np.empty_like(dy)
    lib().orc_act_bwd(kind, _p(dy), _p(cache), _p(dx), C.c_int64(dy.size))
    return dx


def bias_grad(dy, f64=False):
    dy = _f(dy)
    rows, cols = dy.shape
    if f64:
        out = np.empty(cols, np.float64)
        lib().orc_bias_grad_f64(_p(dy), _p(out), C.c_int64(rows), C.c_int64(cols))
    else:
        out = np.empty(cols, np.float32)
        lib().orc_bias_grad(_p(dy), _p(out), C.c_int64(rows), C.c_int64(cols))
    return out


def sgd_update(p, g, lr):
    p = _f(p).copy()
    g = _f(g)
    lib().orc_sgd_update(_p(p), _p(g), C.c_float(lr), C.c_int64(p.size))
    return p


def optim_step(kind, p, g, m, v, lr, beta1, beta2, eps, weight_decay, step):
    """kind: 1 adam, 2 adamw, 3 rmsprop.  Returns updated copies (p, m, v)."""
    p, g, m = _f(p).copy(), _f(g), _f(m).copy()
    v = _f(v).copy() if v is not None else np.zeros_like(p)
    inv1 = np.float32(1.0 / (1.0 - beta1 ** step)) if kind != 3 else np.float32(1)
    inv2 = np.float32(1.0 / (1.0 - beta2 ** step)) if kind != 3 else np.float32(1)
    lib().orc_optim_step(kind, _p(p), _p(g), _p(m), _p(v), C.c_int64(p.size), C.c_float(lr), C.c_float(beta1),
                         C.c_float(beta2), C.c_float(eps), C.c_float(weight_decay), C.c_float(inv1), C.c_float(inv2))
    return p, m, v


def sq_norm(g):
    g = _f(g)
    fn = lib().orc_sq_norm_f64
    fn.restype = C.c_double
    return float(fn(_p(g), C.c_int64(g.size)))


# --- pass-through dense ops ------------------------------------------------------------
def gemm(a, b, bias=None, alpha=1.0, c=None):
    """alpha * a @ b + bias (+ c) for 2-D fp32 arrays of any strides, in the reference's summation order."""
    assert a.dtype == np.float32 and b.dtype == np.float32
    m, k = a.shape
    n = b.shape[1]
    out = np.zeros((m, n), np.float32) if c is None else _f(c).copy()
    es = 4
    bias = None if bias is None else _f(bias)
    lib().orc_gemm(C.c_void_p(a.ctypes.data), C.c_void_p(b.ctypes.data), _p(bias), _p(out), m, n, k,
                   C.c_int64(a.strides[0] // es), C.c_int64(a.strides[1] // es), C.c_int64(b.strides[0] // es),
                   C.c_int64(b.strides[1] // es), C.c_int64(n), C.c_float(alpha), int(c is not None))
    return out


def softmax_fwd(x, causal_period=0):
    x = _f(x)
    out = np.empty_like(x)
    lib().orc_softmax_fwd(_p(x), _p(out), C.c_int64(x.size // x.shape[-1]), x.shape[-1], causal_period)
    return out


def softmax_bwd(dy, s, scale=1.0):
    dy, s = _f(dy), _f(s)
    dx = np.empty_like(dy)
    lib().orc_softmax_bwd(_p(dy), _p(s), _p(dx), C.c_int64(dy.size // dy.shape[-1]), dy.shape[-1], C.c_float(scale))
    return dx


def loss(kind, y, y_pred, classes=1):
    """Returns (error[n], grad) for kind 0 squared, 1 absolute, 2 binary CE, 3 categorical CE."""
    y, y_pred = _f(y), _f(y_pred)
    n = y.size // classes if kind == 3 else y.size
    err, grad = np.empty(n, np.float32), np.empty_like(y_pred)
    lib().orc_loss(kind, _p(y), _p(y_pred), _p(err), _p(grad), C.c_int64(n), classes)
    return err, grad


def ce_from_ids(target, y_pred, eps=1e-10):
    y_pred = _f(y_pred)
    target = np.ascontiguousarray(target, np.int32)
    n, classes = y_pred.shape
    err, grad = np.empty(n, np.float32), np.empty_like(y_pred)
    lib().orc_ce_from_ids(_p(target), _p(y_pred), _p(err), _p(grad), n, classes, C.c_float(eps))
    return err, grad
