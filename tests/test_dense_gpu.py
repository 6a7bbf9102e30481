"""Pass-through dense ops of the C ABI (fp32 products, row softmax, losses) against the CPU oracle.

The products keep the reference's per-element arithmetic (one fused multiply-add per k in ascending
order), so they are compared bit for bit; softmax and the losses go through expf/logf and a
warp-parallel row sum and are compared within 1e-5 relative."""
import numpy as np
import pytest
import torch

from conftest import bits_equal, rel_err, rng_for
from dl_cuda_b200 import capi, ops
from oracle import cpu as oracle

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (4, 8, 2), (64, 64, 16), (65, 63, 17), (130, 30, 64), (7, 200, 129),
                                   (256, 64, 64), (33, 1, 5)])
@pytest.mark.parametrize("layout", ["nn", "nt", "tn"])
def test_gemm_bit_exact_against_oracle(m, n, k, layout):
    g = rng_for(700, m * 31 + n * 7 + k)
    a = g.standard_normal((m, k)).astype(np.float32)
    b = g.standard_normal((k, n)).astype(np.float32)
    bias = g.standard_normal(n).astype(np.float32)
    # the transposed layouts hold the same values in memory transposed and are passed as strided views
    a_dev = dev(a.T).t() if layout == "tn" else dev(a)
    b_dev = dev(b.T).t() if layout == "nt" else dev(b)
    a_host = np.ascontiguousarray(a.T).T if layout == "tn" else a
    b_host = np.ascontiguousarray(b.T).T if layout == "nt" else b
    got = ops.gemm(a_dev, b_dev, bias=dev(bias), alpha=0.125).cpu().numpy()
    want = oracle.gemm(a_host, b_host, bias=bias, alpha=0.125)
    assert bits_equal(got, want)
    # against float64 as well, to catch an oracle that is wrong in the same way
    ref64 = 0.125 * (a.astype(np.float64) @ b.astype(np.float64)) + bias
    assert rel_err(got, ref64) < 1e-5


def test_gemm_accumulate_and_no_bias():
    g = rng_for(701)
    a = g.standard_normal((70, 40)).astype(np.float32)
    b = g.standard_normal((40, 50)).astype(np.float32)
    c0 = g.standard_normal((70, 50)).astype(np.float32)
    out = dev(c0)
    ops.gemm(dev(a), dev(b), out=out, accumulate=True)
    assert bits_equal(out.cpu().numpy(), oracle.gemm(a, b, c=c0))
    plain = ops.gemm(dev(a), dev(b)).cpu().numpy()
    assert bits_equal(plain, oracle.gemm(a, b))


def test_gemm_batched_heads_by_stride():
    """All (batch, head) products of attention in one launch, heads addressed inside [tokens, d_model]."""
    B, H, S, hd = 3, 4, 20, 8
    D = H * hd
    g = rng_for(702)
    q = g.standard_normal((B * S, D)).astype(np.float32)
    k = g.standard_normal((B * S, D)).astype(np.float32)
    scores = torch.empty(B * H, S, S, device="cuda")
    tq, tk = dev(q), dev(k)
    capi.check(capi.lib().dlb_gemm_f32(tq.data_ptr(), tk.data_ptr(), None, scores.data_ptr(), S, S, hd, D, 1, 1, D, S,
                                       B * H, H, S * D, hd, S * D, hd, H * S * S, S * S, 0.25, 0,
                                       capi.current_stream()))
    got = scores.cpu().numpy()
    for b in range(B):
        for h in range(H):
            qh = q[b * S:(b + 1) * S, h * hd:(h + 1) * hd]
            kh = k[b * S:(b + 1) * S, h * hd:(h + 1) * hd]
            assert bits_equal(got[b * H + h], oracle.gemm(qh, kh.T, alpha=0.25))


def test_gemm_rejects_bad_arguments():
    lib = capi.lib()
    t = torch.zeros(16, device="cuda")
    p = t.data_ptr()
    assert lib.dlb_gemm_f32(p, p, None, p, -1, 4, 4, 4, 1, 4, 1, 4, 1, 1, 0, 0, 0, 0, 0, 0, 1.0, 0, None) \
        == capi.ERR_INVALID_ARG
    assert lib.dlb_gemm_f32(p, p, None, p, 4, 4, 4, 4, 1, 4, 1, 2, 1, 1, 0, 0, 0, 0, 0, 0, 1.0, 0, None) \
        == capi.ERR_INVALID_ARG
    assert lib.dlb_gemm_f32(p, p, None, p, 4, 4, 4, 4, 1, 4, 1, 4, 6, 4, 0, 0, 0, 0, 0, 0, 1.0, 0, None) \
        == capi.ERR_INVALID_ARG
    assert lib.dlb_gemm_f32(None, p, None, p, 4, 4, 4, 4, 1, 4, 1, 4, 1, 1, 0, 0, 0, 0, 0, 0, 1.0, 0, None) \
        == capi.ERR_INVALID_ARG
    assert lib.dlb_gemm_f32(p, p, None, p, 0, 4, 4, 4, 1, 4, 1, 4, 1, 1, 0, 0, 0, 0, 0, 0, 1.0, 0, None) == capi.OK


@pytest.mark.parametrize("rows,width", [(1, 1), (5, 30), (64, 64), (200, 33), (7, 1000)])
def test_softmax_forward_backward(rows, width):
    g = rng_for(710, rows + width)
    x = (3 * g.standard_normal((rows, width))).astype(np.float32)
    dy = g.standard_normal((rows, width)).astype(np.float32)
    y = ops.softmax_fwd(dev(x))
    want = oracle.softmax_fwd(x)
    # the oracle adds the row's exponentials one after another in fp32, the kernel in a lane-strided tree
    assert rel_err(y.cpu().numpy(), want) < 1e-5
    assert np.allclose(y.cpu().numpy().sum(axis=1), 1.0, atol=1e-5)
    dx = ops.softmax_bwd(dev(dy), y, scale=0.5).cpu().numpy()
    assert rel_err(dx, oracle.softmax_bwd(dy, y.cpu().numpy(), 0.5)) < 1e-5


def test_softmax_causal_mask_and_in_place():
    S, BH = 24, 6
    g = rng_for(711)
    x = g.standard_normal((BH * S, S)).astype(np.float32)
    t = dev(x)
    ops.softmax_fwd(t, out=t, causal_period=S)
    got = t.cpu().numpy()
    want = oracle.softmax_fwd(x, causal_period=S)
    assert rel_err(got, want) < 1e-6
    rows = np.arange(BH * S) % S
    cols = np.arange(S)
    assert np.all(got[cols[None, :] > rows[:, None]] == 0.0)  # exact zeros above the diagonal
    assert np.all(want[cols[None, :] > rows[:, None]] == 0.0)


@pytest.mark.parametrize("kind", [capi.LOSS_SQUARED, capi.LOSS_ABSOLUTE, capi.LOSS_BCE, capi.LOSS_CCE])
def test_losses(kind):
    g = rng_for(720, kind)
    n, classes = 37, 5
    if kind == capi.LOSS_CCE:
        y = np.eye(classes, dtype=np.float32)[g.integers(0, classes, n)]
        pred = g.random((n, classes)).astype(np.float32)
        pred /= pred.sum(axis=1, keepdims=True)
    elif kind == capi.LOSS_BCE:
        y = g.integers(0, 2, n).astype(np.float32)
        pred = g.random(n).astype(np.float32)
        pred[:3] = [0.0, 0.999999, 1e-12]  # the clamp from below; p = 1 gives inf - inf in the reference too
    else:
        y = g.standard_normal(n).astype(np.float32)
        pred = g.standard_normal(n).astype(np.float32)
        pred[0] = y[0]  # sign(0) = 0 for the absolute error
    err = ops.loss_fwd(kind, dev(y), dev(pred), classes).cpu().numpy()
    grad = ops.loss_bwd(kind, dev(y), dev(pred), classes).cpu().numpy()
    want_err, want_grad = oracle.loss(kind, y, pred, classes)
    assert rel_err(err, want_err) < 1e-6
    assert rel_err(grad, want_grad) < 1e-6


def test_cross_entropy_from_ids():
    g = rng_for(730)
    n, classes = 64, 30
    pred = g.random((n, classes)).astype(np.float32)
    pred /= pred.sum(axis=1, keepdims=True)
    target = g.integers(0, classes, n).astype(np.int32)
    pred[0, target[0]] = 0.0  # clamped to epsilon
    err = ops.ce_from_ids_fwd(dev(target), dev(pred)).cpu().numpy()
    grad = ops.ce_from_ids_bwd(dev(target), dev(pred)).cpu().numpy()
    want_err, want_grad = oracle.ce_from_ids(target, pred)
    assert rel_err(err, want_err) < 1e-6
    assert rel_err(grad, want_grad) < 1e-6
    assert np.count_nonzero(grad) == n
