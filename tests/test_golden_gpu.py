"""The CUDA kernels (through the C ABI) against fixtures written by the reference's own kernels."""
from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import bits_equal, rel_err
from dl_cuda_b200 import capi, ops

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def load(name):
    return dict(np.load(GOLDEN / name))


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("name", ["layernorm_37x100.npz", "layernorm_16x1024.npz", "layernorm_5x3.npz"])
def test_layernorm_fixture(name):
    g = load(name)
    y, xhat, inv_std = ops.ln_residual_fwd(dev(g["a"]), dev(g["b"]), dev(g["gamma"]), dev(g["beta"]), float(g["eps"]))
    assert rel_err(y.cpu().numpy(), g["y"]) <= 1e-5
    assert rel_err(xhat.cpu().numpy(), g["xhat"]) <= 1e-5
    assert rel_err(inv_std.cpu().numpy(), g["inv_std"]) <= 1e-5
    dx, dgamma, dbeta = ops.ln_bwd(dev(g["dy_a"]), dev(g["dy_b"]), dev(g["xhat"]), dev(g["inv_std"]), dev(g["gamma"]))
    assert rel_err(dx.cpu().numpy(), g["dx"]) <= 1e-5
    assert rel_err(dgamma.cpu().numpy(), g["dgamma"]) <= 1e-5
    assert rel_err(dbeta.cpu().numpy(), g["dbeta"]) <= 1e-5


def test_activation_fixture_bit_exact():
    g = load("activation_9x40.npz")
    for kind, name in ((capi.RELU, "relu"), (capi.SIGMOID, "sigmoid"), (capi.TANH, "tanh")):
        y, cache = ops.act_fwd(kind, dev(g["x"]), dev(g["bias"]))
        assert bits_equal(y.cpu().numpy(), g[f"{name}_y"]), name
        dx, _ = ops.act_bwd(kind, dev(g["dy"]), cache)
        assert bits_equal(dx.cpu().numpy(), g[f"{name}_dx"]), name
    y, cache = ops.act_fwd(capi.GELU, dev(g["x"]), dev(g["bias"]))
    assert rel_err(y.cpu().numpy(), g["gelu_y"]) <= 1e-6
    dx, _ = ops.act_bwd(capi.GELU, dev(g["dy"]), cache)
    assert rel_err(dx.cpu().numpy(), g["gelu_dx"]) <= 1e-6
    assert rel_err(ops.bias_grad(dev(g["dy"])).cpu().numpy(), g["dbias_of_dy"]) <= 1e-5


def test_embedding_fixture_bit_exact():
    g = load("embedding_v50_d12.npz")
    seq = int(g["seq"])
    ids = dev(g["ids"])
    assert bits_equal(ops.pe_table(seq, 12).numpy(), g["pe"])
    assert bits_equal(ops.embed_gather_fwd(dev(g["table"]), ids).cpu().numpy(), g["gathered"])
    assert bits_equal(ops.embed_gather_fwd(dev(g["table"]), ids, dev(g["pe"]), seq).cpu().numpy(), g["out"])
    ws = ops.embed_sort_tokens(ids, 50, 12)
    assert bits_equal(ops.embed_scatter_bwd(dev(g["dy"]), ids, 50, ws).cpu().numpy(), g["grad"])
    k = load("embedding_layer_known_answer.npz")
    ids = dev(k["ids"])
    assert np.array_equal(ops.embed_gather_fwd(dev(k["table"]), ids).cpu().numpy(), k["out"])
    ws = ops.embed_sort_tokens(ids, 5, 3)
    assert np.array_equal(ops.embed_scatter_bwd(dev(k["dout"]), ids, 5, ws).cpu().numpy(), k["grad"])


def test_sgd_fixture_bit_exact():
    g = load("sgd_257.npz")
    assert bits_equal(ops.sgd_update(dev(g["p"]), dev(g["g"]), float(g["lr"])).cpu().numpy(), g["out"])
