"""Every kernel that exists in more than one form (dlb_set_option) gives the results of the default
form: the same bits where the order of the additions is the same, within the op's tolerance where the
option changes how partial sums are grouped (layer-norm and bias gradients reduced over rows)."""
import contextlib

import numpy as np
import pytest
import torch

from conftest import rel_err, rng_for, zipf_ids
from dl_cuda_b200 import capi, ops

pytestmark = pytest.mark.gpu


@contextlib.contextmanager
def options(**kv):
    try:
        for name, value in kv.items():
            capi.set_option(name, value)
        yield
    finally:
        for name in kv:
            capi.set_option(name, 0)
        assert capi.pipeline_timeouts() == 0


def dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t if dtype is None else t.to(dtype)


def scatter(dy_t, ids_t, vocab):
    ws = ops.embed_sort_tokens(ids_t, vocab, dy_t.shape[1])
    return ops.embed_scatter_bwd(dy_t, ids_t, vocab, ws)


SCATTER_CASES = [  # vocab, d, tokens, storage
    (30, 2048, 20000, "bf16"), (3, 4096, 9000, "fp32"),  # nearly every token in a long row
    (2000, 4096, 6000, "bf16"), (2000, 4096, 3000, "fp32"), (500, 512, 9000, "bf16"), (40000, 256, 5000, "fp32"),
    (300, 64, 70000, "fp32"), (65, 64, 2048, "bf16"), (17, 8, 40, "fp32"), (3000, 1024, 100, "bf16"),
    (129, 100, 700, "fp32"), (64, 8192, 300, "bf16"),
]


@pytest.mark.parametrize("form", [dict(scatter_variant=1), dict(scatter_variant=2),
                                  dict(scatter_variant=2, scatter_bulk_ctas_per_sm=1),
                                  dict(scatter_variant=2, scatter_bulk_ctas_per_sm=5), dict(scatter_zero_kernel=1),
                                  dict(scatter_variant=2, scatter_zero_kernel=1)])
@pytest.mark.parametrize("vocab,d,n,storage", SCATTER_CASES)
def test_scatter_forms_give_the_same_bits(vocab, d, n, storage, form):
    ids = dev(zipf_ids(rng_for(70, 0), n, vocab))
    dy = dev(rng_for(70, 1).standard_normal((n, d)).astype(np.float32),
             torch.bfloat16 if storage == "bf16" else None)
    want = scatter(dy, ids, vocab)
    with options(**form):
        got = scatter(dy, ids, vocab)
        again = scatter(dy, ids, vocab)
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))
    assert torch.equal(again.view(torch.int32), want.view(torch.int32))


@pytest.mark.parametrize("pattern", ["all_same", "one_each", "none_in_half"])
def test_scatter_bulk_form_edge_patterns(pattern):
    vocab, d, n = 700, 2048, 4000
    if pattern == "all_same":
        ids = np.full(n, 5, np.int32)
    elif pattern == "one_each":
        n = vocab
        ids = rng_for(71, 0).permutation(vocab).astype(np.int32)
    else:
        ids = (rng_for(71, 1).integers(0, vocab // 2, n)).astype(np.int32)
    dy = dev(rng_for(71, 2).standard_normal((n, d)).astype(np.float32), torch.bfloat16)
    with options(scatter_variant=1):
        want = scatter(dy, dev(ids), vocab)
    with options(scatter_variant=2):
        got = scatter(dy, dev(ids), vocab)
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))


@pytest.mark.parametrize("form", [dict(gather_variant=1), dict(gather_variant=2),
                                  dict(gather_variant=2, gather_bulk_ctas_per_sm=1),
                                  dict(gather_variant=2, gather_bulk_waves=1), dict(gather_variant=2, gather_bulk_waves=7),
                                  dict(gather_rows_in_flight=8)])
@pytest.mark.parametrize("vocab,d,batch,seq,storage", [(2000, 4096, 5, 300, "bf16"), (2000, 4096, 3, 200, "fp32"),
                                                        (65, 64, 32, 64, "fp32"), (500, 1024, 9, 77, "bf16"),
                                                        (40000, 256, 16, 50, "fp32"), (300, 104, 2, 33, "bf16")])
def test_gather_forms_give_the_same_bits(vocab, d, batch, seq, storage, form):
    dt = torch.bfloat16 if storage == "bf16" else None
    table = dev((0.02 * rng_for(72, 0).standard_normal((vocab, d))).astype(np.float32), dt)
    ids = dev(zipf_ids(rng_for(72, 1), batch * seq, vocab))
    pe = ops.pe_table(seq, d).cuda()
    with options(gather_variant=1, gather_rows_in_flight=4):
        want = ops.embed_gather_fwd(table, ids, pe, seq)
    with options(**form):
        got = ops.embed_gather_fwd(table, ids, pe, seq)
    assert torch.equal(got.view(torch.int16 if storage == "bf16" else torch.int32),
                       want.view(torch.int16 if storage == "bf16" else torch.int32))


LN_FORMS = [dict(ln_bwd_pipe=1), dict(ln_bwd_pipe=2), dict(ln_bwd_pipe=2, ln_bwd_pipe_threads=128),
            dict(ln_bwd_pipe=2, ln_bwd_pipe_threads=512, ln_bwd_pipe_ctas_per_sm=1),
            dict(ln_bwd_pipe=2, ln_bwd_pipe_rows_per_tile=1), dict(ln_bwd_pipe=2, ln_bwd_pipe_rows_per_tile=8),
            dict(ln_bwd_pipe=2, ln_bwd_pipe_ctas_per_sm=2, ln_bwd_pipe_rows_per_tile=2)]


@pytest.mark.parametrize("form", LN_FORMS)
@pytest.mark.parametrize("rows,d,storage,two", [(3000, 1024, "fp32", False), (2500, 4096, "bf16", False),
                                                (2500, 4096, "bf16", True), (1000, 2048, "fp32", True),
                                                (777, 512, "bf16", False)])
def test_layer_norm_backward_forms_agree(rows, d, storage, two, form):
    dt = torch.bfloat16 if storage == "bf16" else torch.float32
    g = rng_for(73, rows)
    a = dev(g.standard_normal((rows, d)).astype(np.float32), dt)
    b = dev(g.standard_normal((rows, d)).astype(np.float32), dt)
    gamma = dev(g.uniform(0.5, 1.5, d).astype(np.float32))
    beta = dev((0.1 * g.standard_normal(d)).astype(np.float32))
    dy_a = dev(g.standard_normal((rows, d)).astype(np.float32), dt)
    dy_b = dev(g.standard_normal((rows, d)).astype(np.float32), dt) if two else None
    _, xhat, inv_std = ops.ln_residual_fwd(a, b, gamma, beta)
    want = ops.ln_bwd(dy_a, dy_b, xhat, inv_std, gamma)
    with options(**form):
        got = ops.ln_bwd(dy_a, dy_b, xhat, inv_std, gamma)
    # dx: the same per-row arithmetic whatever the tiling; dgamma/dbeta: other groups of partial sums
    tol_dx = 1e-2 if storage == "bf16" else 1e-5
    assert rel_err(got[0].float().cpu().numpy(), want[0].float().cpu().numpy()) <= tol_dx
    for i in (1, 2):
        assert rel_err(got[i].cpu().numpy(), want[i].cpu().numpy()) <= 1e-5


@pytest.mark.parametrize("kind", [capi.RELU, capi.SIGMOID, capi.TANH])
@pytest.mark.parametrize("cap", [1, 32, 4096])
def test_activation_backward_partial_row_cap(kind, cap):
    rows, cols = 5000, 768
    g = rng_for(74, cap)
    x = dev(g.standard_normal((rows, cols)).astype(np.float32) * 2)
    bias = dev((0.1 * g.standard_normal(cols)).astype(np.float32))
    dy = dev(g.standard_normal((rows, cols)).astype(np.float32))
    _, cache = ops.act_fwd(kind, x, bias)
    dx0, db0 = ops.act_bwd(kind, dy, cache, want_dbias=True)
    with options(act_bwd_partial_rows=cap):
        dx1, db1 = ops.act_bwd(kind, dy, cache, want_dbias=True)
    assert torch.equal(dx0.view(torch.int32), dx1.view(torch.int32))
    assert rel_err(db1.cpu().numpy(), db0.cpu().numpy()) <= 1e-5
