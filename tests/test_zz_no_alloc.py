"""dlb_ln_bwd_noalloc: the layer-norm backward for callers that cannot allocate device memory
(its scratch is an array inside the library).  Called through the C ABI twice in a row and
compared with dlb_ln_bwd, which takes a caller-provided workspace (both run the same kernels, so
the results must carry the same bits) and with the CPU oracle (<= 1e-5 relative for fp32 storage,
<= 1e-2 for bf16).  Collected last on purpose."""
import numpy as np
import pytest
import torch

from conftest import rel_err, rng_for
from dl_cuda_b200 import capi, ops
from oracle import cpu as oracle

pytestmark = pytest.mark.gpu


def dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t if dtype is None else t.to(dtype)


def call_noalloc(dy_a, dy_b, xhat, inv_std, gamma):
    rows, d = dy_a.shape
    dx = torch.empty_like(dy_a)
    dgamma = torch.empty(d, dtype=torch.float32, device="cuda")
    dbeta = torch.empty(d, dtype=torch.float32, device="cuda")
    p = capi.ptr
    capi.check(capi.lib().dlb_ln_bwd_noalloc(p(dy_a), p(dy_b), p(xhat), p(inv_std), p(gamma), p(dx), p(dgamma),
                                             p(dbeta), rows, d, capi.dtype_of(dy_a), capi.current_stream()))
    return dx, dgamma, dbeta


@pytest.mark.parametrize("rows,d,storage,two", [(700, 1024, "fp32", True), (3000, 2048, "bf16", False),
                                                (33, 100, "fp32", True), (5, 3, "fp32", False)])
def test_noalloc_matches_the_workspace_entry_point_twice(rows, d, storage, two):
    dt = torch.bfloat16 if storage == "bf16" else torch.float32
    g = rng_for(900 + rows, 0)
    dy_a = dev(g.standard_normal((rows, d)).astype(np.float32), dt)
    dy_b = dev(g.standard_normal((rows, d)).astype(np.float32), dt) if two else None
    xhat = dev(g.standard_normal((rows, d)).astype(np.float32), dt)
    inv_std = dev(g.uniform(0.5, 2.0, rows).astype(np.float32))
    gamma = dev(g.uniform(0.5, 1.5, d).astype(np.float32))
    want = ops.ln_bwd(dy_a, dy_b, xhat, inv_std, gamma)
    # the oracle on exactly the values the kernels see (bf16 storage rounded first)
    host = lambda t: None if t is None else t.float().cpu().numpy()
    dx0, _, _ = oracle.ln_bwd(host(dy_a), host(dy_b), host(xhat), host(inv_std), host(gamma))
    dg64, db64 = oracle.ln_param_grad_f64(host(dy_a), host(dy_b), host(xhat))
    tol = 1e-2 if storage == "bf16" else 1e-5
    for _ in range(2):  # the built-in scratch keeps the previous call's contents: the second call must not care
        got = call_noalloc(dy_a, dy_b, xhat, inv_std, gamma)
        torch.cuda.synchronize()
        for a, b in zip(got, want):
            assert torch.equal(a, b)
        if d > 1:
            assert rel_err(host(got[0]), dx0) <= tol
        assert rel_err(host(got[1]), dg64) <= 1e-5
        assert rel_err(host(got[2]), db64) <= 1e-5
    # a different shape in between, then the first one again
    other = call_noalloc(xhat[: max(1, rows // 2)].contiguous(), None, xhat[: max(1, rows // 2)].contiguous(),
                         inv_std[: max(1, rows // 2)].contiguous(), gamma)
    assert torch.isfinite(other[1].float()).all()
    again = call_noalloc(dy_a, dy_b, xhat, inv_std, gamma)
    for a, b in zip(again, want):
        assert torch.equal(a, b)


def test_noalloc_refuses_what_does_not_fit():
    lib = capi.lib()
    limit = lib.dlb_ln_bwd_noalloc_max_bytes()
    assert limit == 16 << 20
    rows, d = 64, 4096
    assert lib.dlb_ln_bwd_workspace_bytes(rows, d) > limit
    x = torch.zeros(rows, d, device="cuda")
    v = torch.ones(d, device="cuda")
    r = torch.ones(rows, device="cuda")
    st = lib.dlb_ln_bwd_noalloc(x.data_ptr(), None, x.data_ptr(), r.data_ptr(), v.data_ptr(), x.data_ptr(),
                                v.data_ptr(), v.data_ptr(), rows, d, capi.F32, None)
    assert st == capi.ERR_UNSUPPORTED
    assert b"built-in array" in lib.dlb_last_error()
