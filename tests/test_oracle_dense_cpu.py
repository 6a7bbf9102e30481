"""CPU checks of the oracle's restatement of the dense pass-through ops against float64 numpy."""
import numpy as np

from conftest import rel_err, rng_for
from oracle import cpu as oracle


def test_gemm_restatement_matches_float64_for_every_layout():
    g = rng_for(900)
    a = g.standard_normal((13, 29)).astype(np.float32)
    b = g.standard_normal((29, 17)).astype(np.float32)
    bias = g.standard_normal(17).astype(np.float32)
    c0 = g.standard_normal((13, 17)).astype(np.float32)
    want = 0.5 * (a.astype(np.float64) @ b.astype(np.float64)) + bias
    for av in (a, np.ascontiguousarray(a.T).T):
        for bv in (b, np.ascontiguousarray(b.T).T):
            assert rel_err(oracle.gemm(av, bv, bias=bias, alpha=0.5), want) < 1e-6
    assert rel_err(oracle.gemm(a, b, c=c0), c0 + a.astype(np.float64) @ b.astype(np.float64)) < 1e-6
    # ascending-k fused multiply-add, spelled out for one element
    acc = np.float32(0)
    for kk in range(29):
        acc = np.float32(np.float64(a[3, kk]) * np.float64(b[kk, 5]) + np.float64(acc))
    assert oracle.gemm(a, b)[3, 5] == acc


def test_softmax_restatement():
    g = rng_for(901)
    x = (4 * g.standard_normal((9, 12))).astype(np.float32)
    e = np.exp(x.astype(np.float64) - x.max(axis=1, keepdims=True))
    want = e / e.sum(axis=1, keepdims=True)
    got = oracle.softmax_fwd(x)
    assert rel_err(got, want) < 1e-6
    causal = oracle.softmax_fwd(np.tile(x[:, :9], (1, 1)).copy(), causal_period=9)
    assert np.all(np.triu(causal, 1) == 0.0) and np.allclose(causal.sum(axis=1), 1.0, atol=1e-6)
    dy = g.standard_normal((9, 12)).astype(np.float32)
    dot = (dy.astype(np.float64) * got).sum(axis=1, keepdims=True)
    assert rel_err(oracle.softmax_bwd(dy, got, 0.25), got * (dy - dot) * 0.25) < 1e-5


def test_loss_restatements():
    g = rng_for(902)
    n = 11
    y, p = g.standard_normal(n).astype(np.float32), g.standard_normal(n).astype(np.float32)
    err, grad = oracle.loss(0, y, p)
    assert rel_err(err, (y - p) ** 2) < 1e-6 and rel_err(grad, 2 * (p - y) / n) < 1e-6
    err, grad = oracle.loss(1, y, p)
    assert rel_err(err, np.abs(y - p)) < 1e-6 and rel_err(grad, np.sign(p - y) / n) < 1e-6
    yb, pb = g.integers(0, 2, n).astype(np.float32), g.random(n).astype(np.float32)
    err, grad = oracle.loss(2, yb, pb)
    pb64 = np.clip(pb.astype(np.float64), 1e-10, 1 - 1e-10)
    assert rel_err(err, -yb * np.log(pb64) - (1 - yb) * np.log(1 - pb64)) < 1e-5
    pred = g.random((n, 4)).astype(np.float32)
    target = g.integers(0, 4, n).astype(np.int32)
    err, grad = oracle.ce_from_ids(target, pred)
    picked = pred[np.arange(n), target].astype(np.float64)
    assert rel_err(err, -np.log(picked)) < 1e-6
    assert rel_err(grad[np.arange(n), target], -1 / (picked * n)) < 1e-6 and np.count_nonzero(grad) == n
    onehot = np.eye(4, dtype=np.float32)[target]
    err2, grad2 = oracle.loss(3, onehot, pred, 4)
    assert rel_err(err2, err) < 1e-5
