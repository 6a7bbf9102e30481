"""Layer norm with the residual folded in: CUDA path (through the C ABI) against
the CPU oracle and, where the shim library is present, against the reference's
own kernels.  Tolerances: <= 1e-5 relative in fp32,
<= 1e-2 with bf16 storage (relative to max(|a|,|b|,rms))."""
import numpy as np
import pytest
import torch

from conftest import rel_err, rng_for
from dl_cuda_b200 import capi, ops
from oracle import cpu as oracle
from oracle import ref as refshim

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5
BF16_TOL = 1e-2
# Column sums over R rows: the reference adds R fp32 terms top to bottom, the GPU
# adds them as a tree; each is within ~sqrt(R)*2^-24 of the exact sum, so against
# the reference's own order the bound is widened for tall inputs.
def colsum_tol(rows):
    return max(FP32_TOL, 4.0 * np.sqrt(rows) * 2.0 ** -24)


def make_inputs(rows, d, seed, two_inputs=True):
    a = rng_for(seed, 0).standard_normal((rows, d)).astype(np.float32)
    b = rng_for(seed, 1).standard_normal((rows, d)).astype(np.float32) if two_inputs else None
    gamma = rng_for(seed, 2).uniform(0.5, 1.5, d).astype(np.float32)
    beta = (0.1 * rng_for(seed, 3).standard_normal(d)).astype(np.float32)
    dy_a = rng_for(seed, 4).standard_normal((rows, d)).astype(np.float32)
    dy_b = rng_for(seed, 5).standard_normal((rows, d)).astype(np.float32) if two_inputs else None
    return a, b, gamma, beta, dy_a, dy_b


def dev(x, dtype=None):
    if x is None:
        return None
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t if dtype is None else t.to(dtype)


SHAPES = [
    (1, 1), (5, 3), (7, 4), (33, 8), (37, 100), (64, 64), (2048, 64), (130, 256), (19, 260),
    (257, 1024), (64, 1000), (50, 2048), (40, 4096), (9, 8192), (3, 16384), (2, 40000), (11, 1023),
]


@pytest.mark.parametrize("rows,d", SHAPES)
@pytest.mark.parametrize("two_inputs", [True, False])
def test_ln_fwd_bwd_fp32_vs_oracle(rows, d, two_inputs):
    a, b, gamma, beta, dy_a, dy_b = make_inputs(rows, d, 1234 + rows + d, two_inputs)
    y, xhat, inv_std = ops.ln_residual_fwd(dev(a), dev(b), dev(gamma), dev(beta), 1e-5)
    y0, xhat0, inv0 = oracle.ln_residual_fwd(a, b, gamma, beta, 1e-5)
    assert rel_err(y.cpu().numpy(), y0) <= FP32_TOL
    assert rel_err(xhat.cpu().numpy(), xhat0) <= FP32_TOL
    assert rel_err(inv_std.cpu().numpy(), inv0) <= FP32_TOL

    # backward from the oracle's caches so that forward differences do not leak in
    dx, dg, db = ops.ln_bwd(dev(dy_a), dev(dy_b), dev(xhat0), dev(inv0), dev(gamma))
    dx0, dg0, db0 = oracle.ln_bwd(dy_a, dy_b, xhat0, inv0, gamma)
    if d == 1:  # dx is exactly zero in exact arithmetic; only rounding residue of dy*gamma remains
        assert np.abs(dx.cpu().numpy()).max() <= 1e-4 * np.abs(dy_a).max() * 4
    else:
        assert rel_err(dx.cpu().numpy(), dx0) <= FP32_TOL
    dg64, db64 = oracle.ln_param_grad_f64(dy_a, dy_b, xhat0)
    assert rel_err(dg.cpu().numpy(), dg64) <= FP32_TOL
    assert rel_err(db.cpu().numpy(), db64) <= FP32_TOL
    assert rel_err(dg.cpu().numpy(), dg0) <= colsum_tol(rows)
    assert rel_err(db.cpu().numpy(), db0) <= colsum_tol(rows)


@pytest.mark.parametrize("rows,d", [(37, 100), (257, 1024), (2048, 64), (40, 4096), (5, 3), (11, 1023)])
def test_ln_vs_reference_kernels(rows, d):
    if not refshim.available():
        pytest.skip("reference shim not built")
    a, b, gamma, beta, dy_a, dy_b = make_inputs(rows, d, 99 + rows, True)
    ta, tb, tg, tbeta = dev(a), dev(b), dev(gamma), dev(beta)
    y, xhat, inv_std = ops.ln_residual_fwd(ta, tb, tg, tbeta, 1e-5)
    s = refshim.residual_add(ta, tb)
    y_r, xhat_r, inv_r = refshim.ln_fwd(s, tg, tbeta, 1e-5)
    assert rel_err(y.cpu().numpy(), y_r.cpu().numpy()) <= FP32_TOL
    assert rel_err(xhat.cpu().numpy(), xhat_r.cpu().numpy()) <= FP32_TOL
    assert rel_err(inv_std.cpu().numpy(), inv_r.cpu().numpy()) <= FP32_TOL

    tdy_a, tdy_b = dev(dy_a), dev(dy_b)
    dx, dg, db = ops.ln_bwd(tdy_a, tdy_b, xhat_r, inv_r, tg)
    dy_sum = refshim.residual_add(tdy_a, tdy_b)
    dx_r, dg_r, db_r = refshim.ln_bwd(dy_sum, xhat_r, inv_r, tg)
    assert rel_err(dx.cpu().numpy(), dx_r.cpu().numpy()) <= FP32_TOL
    assert rel_err(dg.cpu().numpy(), dg_r.cpu().numpy()) <= colsum_tol(rows)
    assert rel_err(db.cpu().numpy(), db_r.cpu().numpy()) <= colsum_tol(rows)


@pytest.mark.parametrize("rows,d", [(33, 8), (37, 104), (300, 1024), (64, 4096), (40, 1000), (7, 9), (6, 16384)])
def test_ln_bf16_storage(rows, d):
    a, b, gamma, beta, dy_a, dy_b = make_inputs(rows, d, 777 + d, True)
    bf = torch.bfloat16
    ta, tb, tdy_a, tdy_b = dev(a, bf), dev(b, bf), dev(dy_a, bf), dev(dy_b, bf)
    # the oracle sees the bf16-rounded inputs, accumulates in fp32
    a32, b32 = ta.float().cpu().numpy(), tb.float().cpu().numpy()
    y, xhat, inv_std = ops.ln_residual_fwd(ta, tb, dev(gamma), dev(beta), 1e-5)
    assert y.dtype == bf and xhat.dtype == bf and inv_std.dtype == torch.float32
    y0, xhat0, inv0 = oracle.ln_residual_fwd(a32, b32, gamma, beta, 1e-5)
    assert rel_err(y.float().cpu().numpy(), y0) <= BF16_TOL
    assert rel_err(xhat.float().cpu().numpy(), xhat0) <= BF16_TOL
    assert rel_err(inv_std.cpu().numpy(), inv0) <= FP32_TOL

    xh_bf = xhat  # backward consumes the bf16 cache forward wrote
    dx, dg, db = ops.ln_bwd(tdy_a, tdy_b, xh_bf, inv_std, dev(gamma))
    dx0, dg0, db0 = oracle.ln_bwd(tdy_a.float().cpu().numpy(), tdy_b.float().cpu().numpy(),
                                  xh_bf.float().cpu().numpy(), inv_std.cpu().numpy(), gamma)
    assert rel_err(dx.float().cpu().numpy(), dx0) <= BF16_TOL
    assert rel_err(dg.cpu().numpy(), dg0) <= BF16_TOL
    assert rel_err(db.cpu().numpy(), db0) <= BF16_TOL


PIPE_SHAPES = [(1301, 1024, "fp32"), (700, 4096, "fp32"), (1301, 4096, "bf16"), (2500, 2048, "bf16"),
               (2400, 1000, "fp32"), (1250, 8192, "bf16"), (1300, 512, "fp32")]


@pytest.mark.parametrize("rows,d,storage", PIPE_SHAPES)
@pytest.mark.parametrize("two_inputs", [True, False])
def test_ln_bwd_pipelined_kernel(rows, d, storage, two_inputs):
    """Tall inputs take the bulk-copy pipeline; the row count is not a multiple of the tile."""
    a, b, gamma, beta, dy_a, dy_b = make_inputs(rows, d, 31 + rows, two_inputs)
    dt = torch.bfloat16 if storage == "bf16" else torch.float32
    tol = BF16_TOL if storage == "bf16" else FP32_TOL
    ta, tb = dev(a, dt), dev(b, dt)
    _, xhat, inv_std = ops.ln_residual_fwd(ta, tb, dev(gamma), dev(beta))
    tdy_a, tdy_b = dev(dy_a, dt), dev(dy_b, dt)
    dx, dg, db = ops.ln_bwd(tdy_a, tdy_b, xhat, inv_std, dev(gamma))
    f = lambda t: None if t is None else t.float().cpu().numpy()
    dx0, dg0, db0 = oracle.ln_bwd(f(tdy_a), f(tdy_b), f(xhat), f(inv_std), gamma)
    dg64, db64 = oracle.ln_param_grad_f64(f(tdy_a), f(tdy_b), f(xhat))
    assert rel_err(f(dx), dx0) <= tol
    assert rel_err(f(dg), dg64) <= FP32_TOL
    assert rel_err(f(db), db64) <= FP32_TOL
    assert rel_err(f(dg), dg0) <= colsum_tol(rows)
    # dx may alias dy_a here too, and the result is reproducible bit for bit
    alias = tdy_a.clone()
    _, dg2, db2 = ops.ln_bwd(alias, tdy_b, xhat, inv_std, dev(gamma), dx=alias)
    assert torch.equal(alias, dx) and torch.equal(dg2, dg) and torch.equal(db2, db)
    assert capi.pipeline_timeouts() == 0


def test_ln_inference_mode_and_aliasing():
    rows, d = 100, 512
    a, b, gamma, beta, dy_a, _ = make_inputs(rows, d, 5, True)
    ta, tb = dev(a), dev(b)
    y_ref, _, _ = ops.ln_residual_fwd(ta, tb, dev(gamma), dev(beta))
    y_inf, xh, inv = ops.ln_residual_fwd(ta, tb, dev(gamma), dev(beta), cache=False)
    assert xh is None and inv is None
    assert torch.equal(y_ref, y_inf)
    # y may alias a; dx may alias dy
    alias = ta.clone()
    ops.ln_residual_fwd(alias, tb, dev(gamma), dev(beta), y=alias)
    assert torch.equal(alias, y_ref)
    _, xhat, inv_std = ops.ln_residual_fwd(ta, tb, dev(gamma), dev(beta))
    tdy = dev(dy_a)
    dx_ref, dg_ref, db_ref = ops.ln_bwd(tdy, None, xhat, inv_std, dev(gamma))
    alias = tdy.clone()
    _, dg2, db2 = ops.ln_bwd(alias, None, xhat, inv_std, dev(gamma), dx=alias)
    assert torch.equal(alias, dx_ref) and torch.equal(dg2, dg_ref) and torch.equal(db2, db_ref)


def test_ln_bwd_is_bitwise_reproducible():
    rows, d = 5000, 1024
    a, b, gamma, beta, dy_a, dy_b = make_inputs(rows, d, 42, True)
    _, xhat, inv_std = ops.ln_residual_fwd(dev(a), dev(b), dev(gamma), dev(beta))
    outs = [ops.ln_bwd(dev(dy_a), dev(dy_b), xhat, inv_std, dev(gamma)) for _ in range(3)]
    for o in outs[1:]:
        for t0, t1 in zip(outs[0], o):
            assert torch.equal(t0, t1)


def test_ln_unaligned_pointers_take_the_generic_path():
    rows, d = 9, 64
    a, b, gamma, beta, _, _ = make_inputs(rows, d, 8, True)
    big = torch.empty(rows * d + 1, dtype=torch.float32, device="cuda")
    off = big[1:].view(rows, d)  # 4-byte aligned only
    off.copy_(dev(a))
    y, _, _ = ops.ln_residual_fwd(off, dev(b), dev(gamma), dev(beta))
    y0, _, _ = oracle.ln_residual_fwd(a, b, gamma, beta)
    assert rel_err(y.cpu().numpy(), y0) <= FP32_TOL


def test_ln_errors():
    lib = capi.lib()
    x = torch.zeros(4, 8, device="cuda")
    g = torch.ones(8, device="cuda")
    # xhat without inv_std
    st = lib.dlb_ln_residual_fwd(x.data_ptr(), None, g.data_ptr(), g.data_ptr(), x.data_ptr(), x.data_ptr(),
                                 None, 4, 8, 1e-5, 0, None)
    assert st == capi.ERR_INVALID_ARG
    # workspace too small
    st = lib.dlb_ln_bwd(x.data_ptr(), None, x.data_ptr(), g.data_ptr(), g.data_ptr(), x.data_ptr(),
                        g.data_ptr(), g.data_ptr(), x.data_ptr(), 16, 4, 8, 0, None)
    assert st == capi.ERR_WORKSPACE
    # zero rows: gradients of the parameters are zeroed
    dg = torch.full((8,), 3.0, device="cuda")
    db = torch.full((8,), 3.0, device="cuda")
    st = lib.dlb_ln_bwd(None, None, None, None, None, None, dg.data_ptr(), db.data_ptr(), None, 0, 0, 8, 0, None)
    assert st == capi.OK
    torch.cuda.synchronize()
    assert float(dg.abs().sum()) == 0.0 and float(db.abs().sum()) == 0.0
