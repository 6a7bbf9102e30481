"""Shared test plumbing: the gpu marker, seeded inputs, error measures."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def rng_for(seed: int, tensor_index: int = 0) -> np.random.Generator:
    """Counter-based generator: base seed + tensor index, same bytes on every machine."""
    return np.random.Generator(np.random.Philox(key=seed + tensor_index))


def rel_err(got, want) -> float:
    """max |got-want| / max(|got|, |want|, rms(want)): near-zero sums do not dominate."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    if want.size == 0:
        return 0.0
    rms = float(np.sqrt(np.mean(want * want)))
    denom = np.maximum(np.maximum(np.abs(got), np.abs(want)), max(rms, 1e-30))
    return float(np.max(np.abs(got - want) / denom))


def ulp_diff(got, want) -> int:
    """Largest distance in units in the last place between two float32 arrays (NaN==NaN)."""
    g = np.asarray(got, dtype=np.float32).ravel()
    w = np.asarray(want, dtype=np.float32).ravel()
    both_nan = np.isnan(g) & np.isnan(w)
    gi = g.view(np.int32).astype(np.int64)
    wi = w.view(np.int32).astype(np.int64)
    gi = np.where(gi < 0, np.int64(-2 ** 31) - gi, gi)
    wi = np.where(wi < 0, np.int64(-2 ** 31) - wi, wi)
    diff = np.abs(gi - wi)
    diff[both_nan] = 0
    return int(diff.max()) if diff.size else 0


def bits_identical(got, want) -> bool:
    """Same 32-bit patterns everywhere (used GPU against GPU)."""
    g = np.ascontiguousarray(got, dtype=np.float32)
    w = np.ascontiguousarray(want, dtype=np.float32)
    return g.shape == w.shape and bool(np.array_equal(g.view(np.uint32), w.view(np.uint32)))


def bits_equal(got, want) -> bool:
    """Same 32-bit patterns, except that a NaN matches a NaN: x86 and the GPU produce
    different default-NaN payloads for inf*0, which is not a difference of value."""
    g = np.ascontiguousarray(got, dtype=np.float32)
    w = np.ascontiguousarray(want, dtype=np.float32)
    if g.shape != w.shape:
        return False
    same = (g.view(np.uint32) == w.view(np.uint32)) | (np.isnan(g) & np.isnan(w))
    return bool(same.all())


def zipf_ids(rng: np.random.Generator, n: int, vocab: int, s: float = 1.1, permute: bool = True):
    """Bounded Zipf over [0, vocab): p(k) ~ (k+1)^-s, hot ids optionally spread over the table."""
    p = (np.arange(1, vocab + 1, dtype=np.float64)) ** (-s)
    p /= p.sum()
    ids = rng.choice(vocab, size=n, p=p)
    if permute:
        ids = rng.permutation(vocab)[ids]
    return ids.astype(np.int32)
