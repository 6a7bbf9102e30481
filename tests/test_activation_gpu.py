"""Bias + ReLU/Sigmoid/Tanh/GELU epilogues through the C ABI.

fp32 ReLU/Sigmoid/Tanh must carry the same bits as the reference's kernels
(checked against the shim where it is present and against fixtures written by
it); against the CPU oracle ReLU and every backward are bit-exact and
Sigmoid/Tanh/GELU forward are within a few ulp (host libm vs CUDA's expf/tanhf)."""
import numpy as np
import pytest
import torch

from conftest import bits_equal, bits_identical, rel_err, rng_for, ulp_diff
from dl_cuda_b200 import capi, ops
from oracle import cpu as oracle
from oracle import ref as refshim

pytestmark = pytest.mark.gpu

KINDS = [capi.RELU, capi.SIGMOID, capi.TANH, capi.GELU]
NAMES = {capi.RELU: "relu", capi.SIGMOID: "sigmoid", capi.TANH: "tanh", capi.GELU: "gelu"}
LIBM_ULP = 4  # host expf/tanhf vs CUDA expf/tanhf


def dev(x, dtype=None):
    if x is None:
        return None
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t if dtype is None else t.to(dtype)


def special_values():
    return np.array([0.0, -0.0, 1.0, -1.0, np.inf, -np.inf, np.nan, 1e-38, -1e-38, 1e-45, 88.0, -88.0,
                     100.0, -100.0, 3.4e38, -3.4e38, 0.5, -0.5, 9.0, -9.0, 20.0, -20.0, 1e-8, -1e-8],
                    dtype=np.float32)


def make(rows, cols, seed, with_special=True):
    x = (2.0 * rng_for(seed, 0).standard_normal((rows, cols))).astype(np.float32)
    if with_special and x.size >= 24:
        x.ravel()[:24] = special_values()
    bias = (0.1 * rng_for(seed, 1).standard_normal(cols)).astype(np.float32)
    dy = rng_for(seed, 2).standard_normal((rows, cols)).astype(np.float32)
    if with_special and dy.size >= 48:
        dy.ravel()[24:27] = [np.inf, -np.inf, np.nan]
        dy.ravel()[3] = -2.0  # negative upstream on a masked-off element: -0.0 must survive
    return x, bias, dy


SHAPES = [(1, 1), (1, 7), (3, 5), (1, 8), (2, 64), (64, 256), (2048, 256), (33, 1000), (17, 1024),
          (5, 4096), (1000, 24), (7, 16384), (257, 520)]


def cache_for_oracle(kind, y, pre):
    return pre if kind in (capi.RELU, capi.GELU) else y


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("rows,cols", SHAPES)
@pytest.mark.parametrize("with_bias", [False, True])
def test_act_fp32_vs_oracle(kind, rows, cols, with_bias):
    x, bias, dy = make(rows, cols, 4321 + rows * 7 + cols)
    tb = dev(bias) if with_bias else None
    y, cache = ops.act_fwd(kind, dev(x), tb)
    y0, pre0 = oracle.act_fwd(kind, x, bias if with_bias else None)
    yh = y.cpu().numpy()
    if kind == capi.RELU:
        assert bits_equal(yh, y0)
    else:
        finite = np.isfinite(y0)
        assert np.array_equal(np.isnan(yh), np.isnan(y0))
        if kind == capi.GELU:  # 1 + tanh(..) cancels for negative x: compare values, not ulps
            assert rel_err(yh[finite], y0[finite]) <= 1e-6
        else:
            assert ulp_diff(yh[finite], y0[finite]) <= LIBM_ULP

    # backward from what the GPU forward cached, against the oracle on the GPU's own y
    dx, dbias = ops.act_bwd(kind, dev(dy), cache, want_dbias=with_bias)
    dx0 = oracle.act_bwd(kind, dy, cache_for_oracle(kind, yh, pre0))
    dxh = dx.cpu().numpy()
    if kind == capi.GELU:
        ok = np.isfinite(dx0)
        assert rel_err(dxh[ok], dx0[ok]) <= 1e-5
    else:
        assert bits_equal(dxh, dx0), f"{NAMES[kind]} backward differs from the oracle"
    if with_bias:
        clean = np.where(np.isfinite(dxh), dxh, 0.0).astype(np.float32)
        if not np.isfinite(dxh).all():
            return  # the column sums of non-finite columns are non-finite too; nothing to compare
        want = oracle.bias_grad(clean, f64=True)
        assert rel_err(dbias.cpu().numpy(), want) <= 1e-5


@pytest.mark.parametrize("kind", [capi.RELU, capi.SIGMOID, capi.TANH])
@pytest.mark.parametrize("rows,cols", [(3, 5), (64, 256), (33, 1000), (2048, 256), (7, 16384)])
def test_act_bit_exact_vs_reference_kernels(kind, rows, cols):
    if not refshim.available():
        pytest.skip("reference shim not built")
    x, bias, dy = make(rows, cols, 97 + cols)
    tx, tbias, tdy = dev(x), dev(bias), dev(dy)
    # reference: bias add, then the activation layer's forward with its cache copy, then backward
    pre_r = refshim.bias_add(tx, tbias)
    y_r, cache_r = refshim.act_fwd(kind, pre_r)
    dx_r = refshim.act_bwd(kind, tdy, cache_r)
    y, cache = ops.act_fwd(kind, tx, tbias)
    dx, dbias = ops.act_bwd(kind, tdy, cache, want_dbias=True)
    assert bits_identical(y.cpu().numpy(), y_r.cpu().numpy()), f"{NAMES[kind]} forward bits differ"
    assert bits_identical(dx.cpu().numpy(), dx_r.cpu().numpy()), f"{NAMES[kind]} backward bits differ"
    if kind == capi.TANH:
        twin = refshim.tanh_bwd_element(tdy, cache_r)
        assert bits_identical(dx.cpu().numpy(), twin.cpu().numpy())
    # no-bias path too
    y2, cache2 = ops.act_fwd(kind, tx)
    y2_r, cache2_r = refshim.act_fwd(kind, tx)
    assert bits_identical(y2.cpu().numpy(), y2_r.cpu().numpy())
    dx2, _ = ops.act_bwd(kind, tdy, cache2)
    assert bits_identical(dx2.cpu().numpy(), refshim.act_bwd(kind, tdy, cache2_r).cpu().numpy())


def test_gelu_vs_reference_kernels():
    if not refshim.available():
        pytest.skip("reference shim not built")
    x, bias, dy = make(64, 256, 31, with_special=False)
    tx, tdy = dev(x), dev(dy)
    y, cache = ops.act_fwd(capi.GELU, tx)
    y_r, cache_r = refshim.act_fwd(capi.GELU, tx)
    assert ulp_diff(y.cpu().numpy(), y_r.cpu().numpy()) <= 2
    dx, _ = ops.act_bwd(capi.GELU, tdy, cache)
    assert rel_err(dx.cpu().numpy(), refshim.act_bwd(capi.GELU, tdy, cache_r).cpu().numpy()) <= 1e-6


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("rows,cols", [(3, 5), (64, 256), (33, 1000), (9, 4096)])
def test_act_bf16_storage(kind, rows, cols):
    x, bias, dy = make(rows, cols, 11 + cols, with_special=False)
    bf = torch.bfloat16
    tx, tdy = dev(x, bf), dev(dy, bf)
    y, cache = ops.act_fwd(kind, tx, dev(bias))
    y0, pre0 = oracle.act_fwd(kind, tx.float().cpu().numpy(), bias)
    assert y.dtype == bf
    assert rel_err(y.float().cpu().numpy(), y0) <= 1e-2
    dx, dbias = ops.act_bwd(kind, tdy, cache, want_dbias=True)
    # the oracle consumes the cache backward actually read: bf16-rounded y (or pre for GELU)
    n = rows * cols
    cache32 = pre0 if kind == capi.RELU else cache.view(bf)[:n].float().cpu().numpy().reshape(rows, cols)
    dx0 = oracle.act_bwd(kind, tdy.float().cpu().numpy(), cache32)
    assert rel_err(dx.float().cpu().numpy(), dx0) <= 1e-2
    assert rel_err(dbias.cpu().numpy(), oracle.bias_grad(dx0, f64=True)) <= 1e-2


def test_relu_cache_is_one_bit_per_element():
    x, _, _ = make(64, 256, 3)
    n = x.size
    assert capi.lib().dlb_act_cache_bytes(capi.RELU, n, capi.F32) == n // 8
    y, cache = ops.act_fwd(capi.RELU, dev(x))
    bits = np.unpackbits(cache.cpu().numpy()[: n // 8], bitorder="little")
    assert np.array_equal(bits.astype(bool), (x.ravel() > 0))


def test_act_inplace_and_inference():
    x, bias, dy = make(128, 512, 19, with_special=False)
    tx = dev(x)
    y_ref, cache = ops.act_fwd(capi.TANH, tx, dev(bias))
    alias = tx.clone()
    ops.act_fwd(capi.TANH, alias, dev(bias), y=alias, want_cache=False)
    assert torch.equal(alias, y_ref)
    tdy = dev(dy)
    dx_ref, _ = ops.act_bwd(capi.TANH, tdy, cache)
    alias = tdy.clone()
    ops.act_bwd(capi.TANH, alias, cache, dx=alias)
    assert torch.equal(alias, dx_ref)


def test_bias_grad_standalone_and_reproducible():
    rows, cols = 4099, 1032
    dy = rng_for(5, 0).standard_normal((rows, cols)).astype(np.float32)
    tdy = dev(dy)
    got = [ops.bias_grad(tdy) for _ in range(3)]
    assert torch.equal(got[0], got[1]) and torch.equal(got[0], got[2])
    assert rel_err(got[0].cpu().numpy(), oracle.bias_grad(dy, f64=True)) <= 1e-5
    if refshim.available():
        assert rel_err(got[0].cpu().numpy(), refshim.bias_grad(tdy).cpu().numpy()) <= 4 * np.sqrt(rows) * 2.0 ** -24
    odd = dev(dy[:37, :13].copy())
    assert rel_err(ops.bias_grad(odd).cpu().numpy(), oracle.bias_grad(dy[:37, :13], f64=True)) <= 1e-5
