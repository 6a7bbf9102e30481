"""Host-only pieces of the layer API (learning-rate schedules, token sampling) in the C++ headers of
dl_cuda_b200/src, against the reference's own headers.  Both come from tests/cpp/layer_models.cu compiled
against each header set; the functions used here never touch a GPU, so this runs in the CPU suite.  The
reference build exists only where the reference checkout was present at build time: without it the
comparisons are skipped and the stand-alone properties still run."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

from conftest import rng_for

ROOT = Path(__file__).resolve().parent.parent
PATHS = {"native": ROOT / "tests" / "cpp" / "libnative_models.so", "ref": ROOT / "oracle" / "_ref" / "libref_models.so"}
_fp, _ip = C.POINTER(C.c_float), C.POINTER(C.c_int)
_libs = {}


def load(which):
    if which not in _libs:
        path = PATHS[which]
        if which == "native" and not path.exists():
            from dl_cuda_b200 import build
            build.build_cpp_tests()
        if not path.exists():
            pytest.skip(f"{path.name} not built")
        lib = C.CDLL(str(path))
        if not hasattr(lib, "lm_sample"):
            pytest.skip(f"{path.name} predates lm_sample: rebuild")
        lib.lm_schedule.argtypes = [C.c_float, C.c_float, C.c_int, C.c_int, _fp]
        lib.lm_schedule.restype = None
        lib.lm_sample.argtypes = [_fp, C.c_int, C.c_float, C.c_int, C.c_float, C.c_uint, C.c_int, _ip, _fp]
        lib.lm_sample.restype = None
        _libs[which] = lib
    return _libs[which]


def sample(which, probs, temperature, top_k, top_p, seed, draws):
    tokens, filtered = np.empty(draws, np.int32), np.empty_like(probs)
    load(which).lm_sample(probs.ctypes.data_as(_fp), probs.size, temperature, top_k, top_p, seed, draws,
                          tokens.ctypes.data_as(_ip), filtered.ctypes.data_as(_fp))
    return tokens, filtered


def probs_row(n, seed):
    p = rng_for(seed).random(n).astype(np.float32) ** 3
    return (p / p.sum()).astype(np.float32)


@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 0, 1.0), (0.8, 0, 0.9), (0.5, 5, 1.0), (1.3, 10, 0.7),
                                                    (1.0, 100, 0.5)])
def test_sampling_matches_reference(temperature, top_k, top_p):
    probs = probs_row(30, 3)
    tokens, filtered = sample("native", probs, temperature, top_k, top_p, 123, 400)
    ref_tokens, ref_filtered = sample("ref", probs, temperature, top_k, top_p, 123, 400)
    assert np.array_equal(filtered.view(np.uint32), ref_filtered.view(np.uint32))
    assert np.array_equal(tokens, ref_tokens)


def test_sampling_properties():
    probs = probs_row(50, 4)
    tokens, filtered = sample("native", probs, 1.0, 7, 1.0, 9, 2000)
    kept = np.flatnonzero(filtered)
    assert kept.size == 7 and set(kept) == set(np.argsort(-probs)[:7])         # top-k keeps the k largest
    assert set(np.unique(tokens)) <= set(kept)
    tokens, filtered = sample("native", probs, 1.0, 0, 0.6, 9, 2000)
    order = np.argsort(-probs)
    mass = np.cumsum(probs[order])
    cutoff = int(np.argmax(mass >= np.float32(0.6))) + 1
    assert set(np.flatnonzero(filtered)) == set(order[:cutoff])                # shortest prefix reaching p
    peaked = probs.copy()
    peaked[17] = 2.0
    peaked /= peaked.sum()
    tokens, _ = sample("native", peaked, 0.2, 0, 1.0, 9, 500)
    assert np.mean(tokens == 17) > 0.99                                        # cold temperature sharpens the row
    tokens, _ = sample("native", probs, 1.0, 0, 1.0, 9, 20000)
    freq = np.bincount(tokens, minlength=50) / 20000
    assert np.abs(freq - probs).max() < 0.02                                   # plain sampling follows the row
    again, _ = sample("native", probs, 1.0, 0, 1.0, 9, 20000)
    assert np.array_equal(tokens, again)                                       # same seed, same draws


def test_schedules():
    def schedule(which, lr_max, lr_min, warmup, epochs):
        lr = np.empty(epochs, np.float32)
        load(which).lm_schedule(lr_max, lr_min, warmup, epochs, lr.ctypes.data_as(_fp))
        return lr

    lr = schedule("native", 3e-3, 1e-5, 50, 800)
    assert lr[0] == np.float32(3e-3) * (np.float32(1) / np.float32(50)) and lr[49] == np.float32(3e-3)
    assert np.all(np.diff(lr[:50]) > 0) and np.all(np.diff(lr[50:]) <= 0) and lr[-1] > 1e-5
    want = 1e-5 + 0.5 * (3e-3 - 1e-5) * (1 + np.cos(np.pi * (np.arange(800) - 50) / 800))
    assert np.allclose(lr[50:], want[50:], rtol=1e-5)
    for args in ((3e-3, 1e-5, 50, 800), (1e-2, 0.0, 0, 10), (1.0, 0.5, 3, 4)):
        assert np.array_equal(schedule("native", *args).view(np.uint32), schedule("ref", *args).view(np.uint32))
