"""Multi-group optimizer steps and gradient-norm clipping through the C ABI, against the CPU oracle
and (where the shim is present) against the reference's own kernels."""
import numpy as np
import pytest
import torch

from conftest import bits_identical, rel_err, rng_for
from dl_cuda_b200 import capi, ops
from oracle import cpu as oracle
from oracle import ref as refshim

pytestmark = pytest.mark.gpu

SIZES = [1, 5, 4096, 4097, 64 * 64, 64, 12345, 3, 100000]
HYP = dict(lr=3e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)


def make_groups(seed, unaligned=False):
    groups = []
    for i, n in enumerate(SIZES):
        g = rng_for(seed, i)
        arrs = [g.standard_normal(n).astype(np.float32), g.standard_normal(n).astype(np.float32),
                (0.1 * g.standard_normal(n)).astype(np.float32), np.abs(0.01 * g.standard_normal(n)).astype(np.float32)]
        groups.append(arrs)  # p, g, m, v
    return groups


def to_dev(a, unaligned):
    if not unaligned:
        return torch.from_numpy(a.copy()).cuda()
    big = torch.empty(a.size + 1, device="cuda")
    view = big[1:]
    view.copy_(torch.from_numpy(a))
    return view


@pytest.mark.parametrize("kind", [capi.OPT_SGD, capi.OPT_ADAM, capi.OPT_ADAMW, capi.OPT_RMSPROP])
@pytest.mark.parametrize("unaligned", [False, True])
def test_optimizer_step_matches_oracle_and_reference(kind, unaligned):
    groups = make_groups(100 + kind)
    if kind == capi.OPT_RMSPROP:  # its state is a running mean of squares: never negative
        groups = [[p, g, np.abs(m), v] for p, g, m, v in groups]
    step = 3
    dev = [[to_dev(a, unaligned) for a in grp] for grp in groups]
    ops.optim_step(kind, [d[0] for d in dev], [d[1] for d in dev], [d[2] for d in dev], [d[3] for d in dev],
                   step=step, **HYP)
    for (p, g, m, v), d in zip(groups, dev):
        if kind == capi.OPT_SGD:
            want_p, want_m, want_v = oracle.sgd_update(p, g, HYP["lr"]), m, v
        else:
            want_p, want_m, want_v = oracle.optim_step(kind, p, g, m, v, HYP["lr"], HYP["beta1"], HYP["beta2"],
                                                       HYP["eps"], HYP["weight_decay"], step)
        assert rel_err(d[0].cpu().numpy(), want_p) <= 1e-6
        assert rel_err(d[2].cpu().numpy(), want_m) <= 1e-6
        if kind in (capi.OPT_ADAM, capi.OPT_ADAMW):
            assert rel_err(d[3].cpu().numpy(), want_v) <= 1e-6
        if refshim.available() and kind != capi.OPT_SGD:
            rp, rg, rm, rv = (torch.from_numpy(a.copy()).cuda() for a in (p, g, m, v))
            refshim.optim_step(kind, rp, rg, rm, rv, HYP["lr"], HYP["beta1"], HYP["beta2"], HYP["eps"],
                               HYP["weight_decay"], step)
            # same formulas; the compiler may fuse a different product of b*m + (1-b)*g: a few ulp
            assert rel_err(d[0].cpu().numpy(), rp.cpu().numpy()) <= 1e-6
            assert rel_err(d[2].cpu().numpy(), rm.cpu().numpy()) <= 1e-6
            if kind != capi.OPT_RMSPROP:
                assert rel_err(d[3].cpu().numpy(), rv.cpu().numpy()) <= 1e-6


def test_more_groups_than_one_launch_holds():
    n_groups = 150
    ps = [torch.full((7 + i,), 1.0, device="cuda") for i in range(n_groups)]
    gs = [torch.full((7 + i,), float(i), device="cuda") for i in range(n_groups)]
    ops.optim_step(capi.OPT_SGD, ps, gs, lr=0.5)
    for i, p in enumerate(ps):
        assert torch.all(p == 1.0 - 0.5 * i)
    res = ops.grad_norm_clip(gs).cpu().numpy()
    want = sum(float(i) ** 2 * (7 + i) for i in range(n_groups))
    assert abs(res[0] - want) / want <= 1e-6 and res[2] == 1.0


@pytest.mark.parametrize("max_norm", [0.0, 1.0, 1e9])
def test_grad_norm_and_clip(max_norm):
    groups = make_groups(7)
    gs = [torch.from_numpy(grp[1].copy()).cuda() for grp in groups]
    want_sq = sum(oracle.sq_norm(grp[1]) for grp in groups)
    res = ops.grad_norm_clip(gs, max_norm)
    again = ops.grad_norm_clip([torch.from_numpy(grp[1].copy()).cuda() for grp in groups], max_norm)
    assert torch.equal(res[:2], again[:2])  # fixed summation order
    r = res.cpu().numpy()
    norm = np.sqrt(want_sq)
    assert abs(r[0] - want_sq) / want_sq <= 1e-5 and abs(r[1] - norm) / norm <= 1e-5
    clipped = max_norm > 0 and norm > max_norm
    coeff = np.float32(max_norm) / (np.float32(r[1]) + np.float32(1e-6)) if clipped else np.float32(1)
    assert r[2] == coeff
    for grp, g in zip(groups, gs):
        want = grp[1] * coeff if clipped else grp[1]
        assert bits_identical(g.cpu().numpy(), want.astype(np.float32))
    if refshim.available() and max_norm > 0:
        one = torch.from_numpy(groups[-1][1].copy()).cuda()
        mine = torch.from_numpy(groups[-1][1].copy()).cuda()
        ref_norm = refshim.clip_grad_norm(one, max_norm)
        my = ops.grad_norm_clip([mine], max_norm).cpu().numpy()
        assert abs(my[1] - ref_norm) / ref_norm <= 1e-5
        assert rel_err(mine.cpu().numpy(), one.cpu().numpy()) <= 1e-5


def test_clip_reads_this_calls_norm_when_calls_follow_each_other_without_a_sync():
    """Back-to-back clip calls that reuse the result and workspace buffers: each scale kernel must see the
    coefficient its own call computed, not the one left in the buffer by the call before (the kernels overlap
    their launch with the previous kernel's tail, so a load that is not ordered by the grid dependency would
    return the old value)."""
    g = rng_for(950)
    base = g.standard_normal(1 << 20).astype(np.float32)
    result = torch.empty(3, dtype=torch.float32, device="cuda")
    workspace = torch.empty(capi.lib().dlb_grad_norm_workspace_bytes(), dtype=torch.uint8, device="cuda")
    filler_a = torch.ones(32 << 20, device="cuda")
    filler_b = torch.ones(32 << 20, device="cuda")
    filler_out = torch.empty_like(filler_a)
    scales = [1.0, 7.0, 0.5, 19.0, 3.0, 0.25, 11.0, 2.0]
    grads = [torch.from_numpy(base * s).cuda() for s in scales]
    for t in grads:
        ops.residual_add(filler_a, filler_b, out=filler_out)  # a longer kernel in front, so the next launches arrive early
        ops.grad_norm_clip([t], 1.0, result=result, workspace=workspace)
    torch.cuda.synchronize()
    norm0 = float(np.sqrt(np.sum(base.astype(np.float64) ** 2)))
    for t, s in zip(grads, scales):
        got = t.cpu().numpy()
        got_norm = float(np.sqrt(np.sum(got.astype(np.float64) ** 2)))
        assert abs(got_norm - 1.0) < 1e-4, (s, got_norm, norm0 * s)


def test_checkpoint_body_pack_and_unpack():
    """One launch lays the parameter groups out as the body of a DLCU weights file (int32 size, floats, per group);
    one launch scatters such a body back.  More than 64 groups, an empty group and odd sizes included."""
    g = rng_for(960)
    sizes = [5, 4096, 0, 4097, 1, 12345] + [7 + i for i in range(70)]
    params = [torch.from_numpy(g.standard_normal(n).astype(np.float32)).cuda() for n in sizes]
    body = ops.checkpoint_pack(params).cpu().numpy()
    want = b"".join(np.int32(n).tobytes() + p.cpu().numpy().tobytes() for n, p in zip(sizes, params))
    assert body.tobytes() == want
    fresh = [torch.full((n,), 3.0, device="cuda") for n in sizes]
    ops.checkpoint_unpack(torch.from_numpy(body).cuda(), fresh)
    for a, b in zip(params, fresh):
        assert torch.equal(a, b)
    small = torch.empty(8, dtype=torch.uint8, device="cuda")
    import ctypes
    arr = (ctypes.c_int * 1)(100)
    assert capi.lib().dlb_checkpoint_pack(1, ops._ptr_array(params[1:2]), arr, small.data_ptr(), 8, None) \
        == capi.ERR_WORKSPACE
