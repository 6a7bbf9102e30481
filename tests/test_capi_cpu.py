"""CPU-side checks of the boundary: the library loads, exports every symbol the
header declares, and rejects bad arguments before touching a device."""
import ctypes
import re
from pathlib import Path

import numpy as np

from dl_cuda_b200 import capi

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "dlcuda_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dlb_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    names = declared_symbols()
    assert len(names) >= 20
    handle = ctypes.CDLL(str(capi.LIB_PATH))
    for name in names:
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"


def test_binding_table_matches_header():
    assert sorted(capi.SIGNATURES) == declared_symbols()


def test_status_strings_and_version():
    lib = capi.lib()
    assert lib.dlb_version() >= 100
    assert lib.dlb_status_string(capi.OK) == b"ok"
    assert b"fallback" in lib.dlb_status_string(capi.ERR_NO_DEVICE)


def test_bad_arguments_are_rejected_without_a_device():
    lib = capi.lib()
    assert lib.dlb_ln_residual_fwd(None, None, None, None, None, None, None, -1, 8, 1e-5, 0, None) == capi.ERR_INVALID_ARG
    assert b"rows=-1" in lib.dlb_last_error()
    assert lib.dlb_ln_residual_fwd(None, None, None, None, None, None, None, 4, 8, 1e-5, 0, None) == capi.ERR_INVALID_ARG
    assert lib.dlb_act_fwd(0, None, None, None, None, 4, 0, 0, None) == capi.ERR_INVALID_ARG
    assert lib.dlb_embed_gather_fwd(None, None, None, 0, None, 4, 0, 8, 0, None) == capi.ERR_INVALID_ARG
    assert lib.dlb_embed_sort_tokens(None, None, 0, 4, 10, 8, None) == capi.ERR_WORKSPACE
    assert lib.dlb_ln_bwd_workspace_bytes(0, 8) == 0
    assert lib.dlb_ln_bwd_workspace_bytes(16, 8) > 0
    assert lib.dlb_act_cache_bytes(capi.RELU, 1000, capi.F32) == 125
    assert lib.dlb_act_cache_bytes(capi.TANH, 1000, capi.BF16) == 2000
    # zero-sized work is a no-op that needs no device
    assert lib.dlb_residual_add(None, None, None, 0, 0, None) == capi.OK


def test_pe_table_host_matches_formula():
    seq_len, d = 9, 10
    t = np.empty((seq_len, d), np.float32)
    capi.check(capi.lib().dlb_pe_build_table_host(t.ctypes.data, seq_len, d))
    pos = np.arange(seq_len, dtype=np.float64)[:, None]
    i = np.arange(d)[None, :]
    angle = pos / np.power(10000.0, (2 * (i // 2)) / d)
    want = np.where(i % 2 == 0, np.sin(angle), np.cos(angle))
    assert np.abs(t - want).max() < 1e-5
    assert t[0, 0] == 0.0 and t[0, 1] == 1.0
