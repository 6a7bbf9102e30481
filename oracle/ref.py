"""TEST INFRASTRUCTURE: torch front end of oracle/ref_shim.cu (libref_shim.so).

Runs the reference's own, unmodified CUDA kernels (fp32 only, default stream)
on device tensors.  The library is built from the reference checkout by
``make -C oracle ref`` where that checkout exists; elsewhere only the prebuilt
file is used, and ``available()`` says whether it is there.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "_ref" / "libref_shim.so"

_lib = None
# Reference layers with weights built in this process so far: the reference seeds the n-th one
# with global_seed + 9973*n (src/layers.cuh:15-19) and the counter cannot be reset.
layers_built = 0


def available() -> bool:
    return LIB_PATH.exists()


_P, _I, _F = C.c_void_p, C.c_int, C.c_float
_SIGNATURES = {
    "ref_residual_add": [_P, _P, _P, _I],
    "ref_ln_fwd": [_P, _P, _P, _P, _P, _P, _I, _I, _F],
    "ref_ln_bwd": [_P, _P, _P, _P, _P, _P, _P, _I, _I],
    "ref_embed_fwd": [_P, _P, _P, _I, _I],
    "ref_embed_bwd": [_P, _P, _P, _I, _I, _I],
    "ref_pe_add": [_P, _P, _P, _I, _I, _I],
    "ref_pe_bwd": [_P, _P, _I],
    "ref_pe_table": [_P, _I, _I],
    "ref_act_fwd": [_I, _P, _P, _P, _I],
    "ref_act_bwd": [_I, _P, _P, _P, _I],
    "ref_tanh_bwd_element": [_P, _P, _P, _I],
    "ref_bias_grad": [_P, _P, _I, _I],
    "ref_bias_add": [_P, _P, _P, _I, _I],
    "ref_sgd": [_P, _P, _F, _I],
    "ref_optim_step": [_I, _P, _P, _P, _P, _I, _F, _F, _F, _F, _F, _F, _F],
    "ref_clip_grad_norm": [_P, _I, _F, _P],
    "ref_embedding_init": [C.c_uint64, _I, _I, _I, _P, C.c_char_p],
    "ref_embedding_layer_run": [_P, _P, _P, _I, _I, _I, _P, _P],
}


def lib() -> C.CDLL:
    """The shim with argument types set, so that 64-bit device addresses are never truncated."""
    global _lib
    if _lib is None:
        handle = C.CDLL(str(LIB_PATH))
        for name, args in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = C.c_int, args
        _lib = handle
    return _lib


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _ok(code, what):
    torch.cuda.synchronize()
    if code != 0:
        raise RuntimeError(f"reference shim {what}: CUDA error {code}")


def _i32(n):
    if n >= 2 ** 31:
        raise ValueError("the reference indexes with int: tensor too large")
    return int(n)


def residual_add(a, b, out=None):
    out = torch.empty_like(a) if out is None else out
    _ok(lib().ref_residual_add(_p(a), _p(b), _p(out), _i32(a.numel())), "residual_add")
    return out


def ln_fwd(x, gamma, beta, eps=1e-5, y=None, xhat=None, inv_std=None):
    rows, d = x.shape
    y = torch.empty_like(x) if y is None else y
    xhat = torch.empty_like(x) if xhat is None else xhat
    inv_std = torch.empty(rows, dtype=torch.float32, device=x.device) if inv_std is None else inv_std
    _ok(lib().ref_ln_fwd(_p(x), _p(gamma), _p(beta), _p(y), _p(xhat), _p(inv_std), rows, d,
                         C.c_float(eps)), "ln_fwd")
    return y, xhat, inv_std


def ln_bwd(dy, xhat, inv_std, gamma, dx=None, dgamma=None, dbeta=None):
    rows, d = dy.shape
    dx = torch.empty_like(dy) if dx is None else dx
    dgamma = torch.empty(d, dtype=torch.float32, device=dy.device) if dgamma is None else dgamma
    dbeta = torch.empty(d, dtype=torch.float32, device=dy.device) if dbeta is None else dbeta
    _ok(lib().ref_ln_bwd(_p(dy), _p(xhat), _p(inv_std), _p(gamma), _p(dx), _p(dgamma), _p(dbeta),
                         rows, d), "ln_bwd")
    return dx, dgamma, dbeta


def embed_fwd(table, ids, out=None):
    n, d = ids.numel(), table.shape[1]
    out = torch.empty(n, d, dtype=torch.float32, device=table.device) if out is None else out
    _ok(lib().ref_embed_fwd(_p(table), _p(ids), _p(out), n, d), "embed_fwd")
    return out


def embed_bwd(dy, ids, vocab, grad=None):
    n, d = dy.shape
    grad = torch.empty(vocab, d, dtype=torch.float32, device=dy.device) if grad is None else grad
    _ok(lib().ref_embed_bwd(_p(dy), _p(ids), _p(grad), n, vocab, d), "embed_bwd")
    return grad


def pe_table(seq_len, d):
    t = np.empty((seq_len, d), np.float32)
    code = lib().ref_pe_table(C.c_void_p(t.ctypes.data), seq_len, d)
    _ok(code, "pe_table")
    return torch.from_numpy(t)


def pe_add(x, pe, out=None):
    batch, seq_len, d = x.shape
    out = torch.empty_like(x) if out is None else out
    _ok(lib().ref_pe_add(_p(x), _p(pe), _p(out), batch, seq_len, d), "pe_add")
    return out


def pe_bwd(dy, dx=None):
    dx = torch.empty_like(dy) if dx is None else dx
    _ok(lib().ref_pe_bwd(_p(dy), _p(dx), _i32(dy.numel())), "pe_bwd")
    return dx


def bias_add(x, bias, out=None):
    rows, cols = x.shape
    out = torch.empty_like(x) if out is None else out
    _ok(lib().ref_bias_add(_p(x), _p(bias), _p(out), rows, cols), "bias_add")
    return out


def act_fwd(kind, x, y=None, cache=None, want_cache=True):
    y = torch.empty_like(x) if y is None else y
    if want_cache and cache is None:
        cache = torch.empty_like(x)
    _ok(lib().ref_act_fwd(kind, _p(x), _p(y), _p(cache) if want_cache else None, _i32(x.numel())), "act_fwd")
    return y, cache


def act_bwd(kind, dy, cache, dx=None):
    dx = torch.empty_like(dy) if dx is None else dx
    _ok(lib().ref_act_bwd(kind, _p(dy), _p(cache), _p(dx), _i32(dy.numel())), "act_bwd")
    return dx


def tanh_bwd_element(dh, h, out=None):
    out = torch.empty_like(dh) if out is None else out
    _ok(lib().ref_tanh_bwd_element(_p(dh), _p(h), _p(out), _i32(dh.numel())), "tanh_bwd_element")
    return out


def bias_grad(dy, dbias=None):
    rows, cols = dy.shape
    dbias = torch.empty(cols, dtype=torch.float32, device=dy.device) if dbias is None else dbias
    _ok(lib().ref_bias_grad(_p(dy), _p(dbias), rows, cols), "bias_grad")
    return dbias


def sgd(p, g, lr):
    _ok(lib().ref_sgd(_p(p), _p(g), C.c_float(lr), _i32(p.numel())), "sgd")
    return p


def embedding_init(seed, vocab, d, num_tokens, checkpoint_path=None):
    """cuRAND-initialised table of a reference EmbeddingLayer built after set_global_init_seed(seed)."""
    global layers_built
    layers_built += 1
    t = np.empty((vocab, d), np.float32)
    path = None if checkpoint_path is None else str(checkpoint_path).encode()
    code = lib().ref_embedding_init(C.c_uint64(seed), vocab, d, num_tokens, C.c_void_p(t.ctypes.data), path)
    _ok(code, "embedding_init")
    return t


def embedding_layer_run(table, ids, dout):
    """The reference EmbeddingLayer class end to end on host arrays: (out, grad)."""
    global layers_built
    layers_built += 1
    table = np.ascontiguousarray(table, np.float32)
    ids = np.ascontiguousarray(ids, np.int32)
    dout = np.ascontiguousarray(dout, np.float32)
    vocab, d = table.shape
    out = np.empty((ids.size, d), np.float32)
    grad = np.empty_like(table)
    code = lib().ref_embedding_layer_run(C.c_void_p(table.ctypes.data), C.c_void_p(ids.ctypes.data),
                                         C.c_void_p(dout.ctypes.data), vocab, d, ids.size,
                                         C.c_void_p(out.ctypes.data), C.c_void_p(grad.ctypes.data))
    _ok(code, "embedding_layer_run")
    return out, grad


def optim_step(kind, p, g, m, v, lr, beta1, beta2, eps, weight_decay, step):
    """In place on device tensors; kind 1 adam, 2 adamw, 3 rmsprop."""
    inv1 = 1.0 / (1.0 - beta1 ** step) if kind != 3 else 1.0
    inv2 = 1.0 / (1.0 - beta2 ** step) if kind != 3 else 1.0
    _ok(lib().ref_optim_step(kind, _p(p), _p(g), _p(m), _p(v), _i32(p.numel()), lr, beta1, beta2, eps, weight_decay,
                             inv1, inv2), "optim_step")


def clip_grad_norm(g, max_norm):
    out = C.c_float(0)
    _ok(lib().ref_clip_grad_norm(_p(g), _i32(g.numel()), max_norm, C.byref(out)), "clip_grad_norm")
    return float(out.value)
