"""Pins the CPU oracle (oracle/host_ref.cpp) to the reference: its own known-answer vectors and
fixtures written by the reference's unmodified CUDA kernels (tests/golden/make_golden.py).
Runs without a GPU."""
from pathlib import Path

import numpy as np
import pytest

from conftest import bits_equal, rel_err, ulp_diff
from oracle import cpu as oracle

GOLDEN = Path(__file__).resolve().parent / "golden"


def load(name):
    return dict(np.load(GOLDEN / name))


def test_reference_embedding_known_answer():
    # tests/gpu_correctness_tests.cu:196-252 of the reference, and what its EmbeddingLayer returned
    g = load("embedding_layer_known_answer.npz")
    out = oracle.embed_gather(g["table"], g["ids"])
    grad = oracle.embed_scatter(g["dout"], g["ids"], 5)
    assert np.array_equal(out, np.array([[3, 4, 5], [9, 10, 11], [3, 4, 5], [12, 13, 14]], np.float32))
    want = np.zeros((5, 3), np.float32)
    want[1], want[3], want[4] = 4.0, 2.0, 4.0
    assert np.array_equal(grad, want)
    assert np.array_equal(out, g["out"]) and np.array_equal(grad, g["grad"])
    assert np.array_equal(grad, oracle.embed_scatter(g["dout"], g["ids"], 5, "segmented"))


@pytest.mark.parametrize("name", ["layernorm_37x100.npz", "layernorm_16x1024.npz", "layernorm_5x3.npz"])
def test_layernorm_matches_reference_kernels(name):
    g = load(name)
    y, xhat, inv_std = oracle.ln_residual_fwd(g["a"], g["b"], g["gamma"], g["beta"], float(g["eps"]))
    # same sequential order and the same fused multiply-adds as the GPU code: a few ulp at most
    assert ulp_diff(inv_std, g["inv_std"]) <= 2
    assert rel_err(y, g["y"]) <= 1e-6 and rel_err(xhat, g["xhat"]) <= 1e-6
    dx, dgamma, dbeta = oracle.ln_bwd(g["dy_a"], g["dy_b"], g["xhat"], g["inv_std"], g["gamma"])
    assert rel_err(dx, g["dx"]) <= 1e-6
    assert rel_err(dgamma, g["dgamma"]) <= 1e-6 and rel_err(dbeta, g["dbeta"]) <= 1e-6


def test_activations_match_reference_kernels():
    g = load("activation_9x40.npz")
    for kind, name in ((0, "relu"), (1, "sigmoid"), (2, "tanh"), (3, "gelu")):
        y, pre = oracle.act_fwd(kind, g["x"], g["bias"])
        assert bits_equal(pre, g["pre"])
        if kind == 0:
            assert bits_equal(y, g["relu_y"])
        else:
            assert rel_err(y, g[f"{name}_y"]) <= 1e-6  # host libm vs CUDA expf/tanhf
        # backward from the reference's own cache: bit-for-bit (GELU: its tanhf differs by ulps)
        cache = g["pre"] if kind in (0, 3) else g[f"{name}_y"]
        dx = oracle.act_bwd(kind, g["dy"], cache)
        if kind == 3:
            assert rel_err(dx, g["gelu_dx"]) <= 1e-6
        else:
            assert bits_equal(dx, g[f"{name}_dx"]), name
    assert rel_err(oracle.bias_grad(g["dy"]), g["dbias_of_dy"]) <= 1e-6


def test_embedding_matches_reference_kernels():
    g = load("embedding_v50_d12.npz")
    seq = int(g["seq"])
    assert bits_equal(oracle.pe_table(seq, 12), g["pe"])
    assert bits_equal(oracle.embed_gather(g["table"], g["ids"]), g["gathered"])
    assert bits_equal(oracle.embed_gather(g["table"], g["ids"], g["pe"], seq), g["out"])
    for mode in ("sequential", "segmented"):
        assert bits_equal(oracle.embed_scatter(g["dy"], g["ids"], 50, mode), g["grad"])


def test_sgd_matches_reference_kernel():
    g = load("sgd_257.npz")
    assert bits_equal(oracle.sgd_update(g["p"], g["g"], float(g["lr"])), g["out"])


def test_residual_add_and_bias_grad_orders():
    rng = np.random.default_rng(0)
    a, b = rng.standard_normal(1000).astype(np.float32), rng.standard_normal(1000).astype(np.float32)
    assert bits_equal(oracle.residual_add(a, b), a + b)
    dy = rng.standard_normal((300, 7)).astype(np.float32)
    want = np.zeros(7, np.float32)
    for r in range(300):
        want += dy[r]
    assert bits_equal(oracle.bias_grad(dy), want)
    assert rel_err(oracle.bias_grad(dy, f64=True), dy.astype(np.float64).sum(0)) <= 1e-12
