"""ctypes binding of the C ABI declared in include/dlcuda_b200.h.

The library is the product; this module only gives Python (tests, bench) a way
to call it with raw device pointers.  Loading fails loudly when the shared
library has not been built: there is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libdlcuda_b200.so"

F32, BF16 = 0, 1
RELU, SIGMOID, TANH, GELU = 0, 1, 2, 3
OPT_SGD, OPT_ADAM, OPT_ADAMW, OPT_RMSPROP = 0, 1, 2, 3
LOSS_SQUARED, LOSS_ABSOLUTE, LOSS_BCE, LOSS_CCE = 0, 1, 2, 3
OK, ERR_INVALID_ARG, ERR_WORKSPACE, ERR_UNSUPPORTED, ERR_CUDA, ERR_NO_DEVICE = range(6)

_p, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes); mirrors include/dlcuda_b200.h one to one.
SIGNATURES = {
    "dlb_version": (_i, []),
    "dlb_status_string": (C.c_char_p, [_i]),
    "dlb_last_error": (C.c_char_p, []),
    "dlb_launch_count": (C.c_uint64, []),
    "dlb_pipeline_timeouts": (_i, [_p]),
    "dlb_set_option": (_i, [C.c_char_p, _i]),
    "dlb_residual_add": (_i, [_p, _p, _p, _i64, _i, _p]),
    "dlb_ln_residual_fwd": (_i, [_p, _p, _p, _p, _p, _p, _p, _i, _i, _f, _i, _p]),
    "dlb_ln_bwd_workspace_bytes": (_sz, [_i, _i]),
    "dlb_ln_bwd": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _sz, _i, _i, _i, _p]),
    "dlb_ln_bwd_noalloc_max_bytes": (_sz, []),
    "dlb_ln_bwd_noalloc": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _p]),
    "dlb_pe_build_table_host": (_i, [_p, _i, _i]),
    "dlb_pe_add_fwd": (_i, [_p, _p, _p, _i, _i, _i, _i, _p]),
    "dlb_pe_add_bwd": (_i, [_p, _p, _i64, _i, _p]),
    "dlb_embed_gather_fwd": (_i, [_p, _p, _p, _i, _p, _i, _i, _i, _i, _p]),
    "dlb_embed_workspace_bytes": (_sz, [_i, _i, _i]),
    "dlb_embed_sort_tokens": (_i, [_p, _p, _sz, _i, _i, _i, _p]),
    "dlb_embed_scatter_bwd": (_i, [_p, _p, _p, _p, _sz, _i, _i, _i, _i, _p]),
    "dlb_embed_rank_plan_bytes": (_sz, [_i, _i, _i]),
    "dlb_embed_rank_plan": (_i, [_p, _i, _i, _i, _i, _p, _sz, _i, _i, _p]),
    "dlb_embed_scatter_bwd_compact": (_i, [_p, _p, _i, _p, _i, _i, _p, _i, _i, _i, _i, _p]),
    "dlb_embed_expand_rows": (_i, [_p, _p, _i, _p, _i, _i, _i, _p]),
    "dlb_act_cache_bytes": (_sz, [_i, _i64, _i]),
    "dlb_act_fwd": (_i, [_i, _p, _p, _p, _p, _i64, _i64, _i, _p]),
    "dlb_act_bwd_workspace_bytes": (_sz, [_i, _i64, _i64]),
    "dlb_act_bwd": (_i, [_i, _p, _p, _p, _p, _p, _sz, _i64, _i64, _i, _p]),
    "dlb_bias_grad_workspace_bytes": (_sz, [_i64, _i64]),
    "dlb_bias_grad": (_i, [_p, _p, _p, _sz, _i64, _i64, _i, _p]),
    "dlb_sgd_update": (_i, [_p, _p, _f, _i64, _p]),
    "dlb_optim_step": (_i, [_i, _i, _p, _p, _p, _p, _p, _f, _f, _f, _f, _f, _f, _f, _p]),
    "dlb_grad_norm_workspace_bytes": (_sz, []),
    "dlb_grad_norm_clip": (_i, [_i, _p, _p, _f, _p, _sz, _p, _p]),
    "dlb_checkpoint_body_bytes": (_sz, [_i, _p]),
    "dlb_checkpoint_pack": (_i, [_i, _p, _p, _p, _sz, _p]),
    "dlb_checkpoint_unpack": (_i, [_i, _p, _p, _p, _sz, _p]),
    "dlb_embed_scatter_bwd_peer": (_i, [_p, _p, _i, _p, _i, _p, _p, _i, _i, _i, _i, _i, _i, _i, C.c_uint32, _p]),
    "dlb_embed_reduce_broadcast_peer": (_i, [_p, _i, _p, _p, _i, _i, _i, _i, C.c_uint32, _i, C.c_uint32, _p]),
    "dlb_peer_flags_bytes": (_sz, []),
    "dlb_peer_barrier": (_i, [_p, _i, _i, _i, C.c_uint32, _i, _p, _p]),
    "dlb_peer_wait": (_i, [_p, _i, _i, _i, C.c_uint32, _i, _p, _p]),
    "dlb_peer_put": (_i, [_p, _sz, _p, _p, _i, _i, _i, C.c_uint32, _i, _i, _p, _p]),
    "dlb_gemm_f32": (_i, [_p, _p, _p, _p, _i, _i, _i, _i64, _i64, _i64, _i64, _i64, _i, _i,
                          _i64, _i64, _i64, _i64, _i64, _i64, _f, _i, _p]),
    "dlb_softmax_fwd": (_i, [_p, _p, _i64, _i, _i, _p]),
    "dlb_softmax_bwd": (_i, [_p, _p, _p, _i64, _i, _f, _p]),
    "dlb_loss_fwd": (_i, [_i, _p, _p, _p, _i64, _i, _p]),
    "dlb_loss_bwd": (_i, [_i, _p, _p, _p, _i64, _i, _p]),
    "dlb_ce_from_ids_fwd": (_i, [_p, _p, _p, _i, _i, _f, _p]),
    "dlb_ce_from_ids_bwd": (_i, [_p, _p, _p, _i, _i, _f, _p]),
}


MAX_PEERS = 16


class PeerGroup(C.Structure):
    """dlb_peer_group of include/dlcuda_b200.h: the buffers of every rank as mapped on this GPU."""
    _fields_ = [("n_ranks", _i), ("my_rank", _i), ("cap_rows", _i), ("small_n", _i), ("timeout_ms", _i),
                ("reserved", _i), ("flags", _p * MAX_PEERS), ("recv", _p * MAX_PEERS), ("grad", _p * MAX_PEERS),
                ("small", _p * MAX_PEERS), ("stage", _p * MAX_PEERS), ("status", _p)]


class DlbError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"dlcuda_b200 status {status}: {message}")
        self.status = status


_lib = None


def lib() -> C.CDLL:
    """The loaded library with argument types set; raises if it is not built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m dl_cuda_b200.build` "
                "(the kernels have no CPU fallback)")
        handle = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != OK:
        raise DlbError(status, lib().dlb_last_error().decode() or lib().dlb_status_string(status).decode())


def set_option(name: str, value: int) -> None:
    """Kernel-variant override for measurements (0 = heuristic); see dlb_set_option in the header."""
    check(lib().dlb_set_option(name.encode(), int(value)))


def pipeline_timeouts() -> int:
    """Waits that gave up inside pipelined kernels on the current device (0 = all good)."""
    out = C.c_uint(0)
    check(lib().dlb_pipeline_timeouts(C.byref(out)))
    return int(out.value)


def ptr(t) -> int | None:
    """Device (or host) address of a torch tensor / numpy array, None for None."""
    if t is None:
        return None
    if hasattr(t, "data_ptr"):
        return t.data_ptr()
    return t.ctypes.data


def dtype_of(t) -> int:
    import torch
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"unsupported storage type {t.dtype}")


def current_stream() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream
