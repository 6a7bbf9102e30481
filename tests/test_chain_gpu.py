"""The whole chain queued back to back on one stream (as bench.py does), many steps without a host
synchronisation: every step must reproduce the first step's bits."""
import numpy as np
import pytest
import torch

from conftest import rng_for, zipf_ids
from dl_cuda_b200 import capi, ops

pytestmark = pytest.mark.gpu


def test_chain_steps_are_reproducible_without_host_syncs():
    T, S, D, F, V = 2048, 256, 1024, 4096, 5000
    bf = torch.bfloat16
    g = lambda i, *s: torch.from_numpy(rng_for(5, i).standard_normal(s).astype(np.float32)).cuda()
    table = (g(0, V, D) * 0.02).to(bf)
    ids = torch.from_numpy(zipf_ids(rng_for(5, 1), T, V)).cuda()
    pe = ops.pe_table(S, D).cuda()
    attn, ffo, dy, dffi = g(2, T, D).to(bf), g(3, T, D).to(bf), g(4, T, D).to(bf), g(5, T, D).to(bf)
    ffpre, dact = g(6, T, F).to(bf), g(7, T, F).to(bf)
    gamma, beta, bias = torch.rand(D, device="cuda") + 0.5, g(8, D) * 0.1, g(9, F) * 0.1

    def step():
        ws = ops.embed_sort_tokens(ids, V, D)
        x0 = ops.embed_gather_fwd(table, ids, pe, S)
        y1, xh1, is1 = ops.ln_residual_fwd(x0, attn, gamma, beta)
        act, mask = ops.act_fwd(capi.RELU, ffpre, bias)
        y2, xh2, is2 = ops.ln_residual_fwd(y1, ffo, gamma, beta)
        dx2, dg2, db2 = ops.ln_bwd(dy, None, xh2, is2, gamma)
        dpre, dbias = ops.act_bwd(capi.RELU, dact, mask, want_dbias=True)
        dx1, dg1, db1 = ops.ln_bwd(dx2, dffi, xh1, is1, gamma)
        grad = ops.embed_scatter_bwd(dx1, ids, V, ws)
        return [y2, act, dx1, dpre, dg1, db1, dg2, db2, dbias, grad]

    first = [t.clone() for t in step()]
    torch.cuda.synchronize()
    for _ in range(25):
        outs = step()
    torch.cuda.synchronize()
    for a, b in zip(outs, first):
        assert torch.equal(a, b)
    assert capi.pipeline_timeouts() == 0


def test_chain_is_capturable_as_one_cuda_graph():
    """Every entry point of the chain (the cluster plan kernel and the PDL launches included) is captured into
    one CUDA graph; a replay must give the eager result bit for bit."""
    T, S, D, F, V = 2048, 64, 64, 256, 65
    g = lambda i, *s: torch.from_numpy(rng_for(6, i).standard_normal(s).astype(np.float32)).cuda()
    table, res, dy, pre, dact = g(0, V, D) * 0.02, g(1, T, D), g(2, T, D), g(3, T, F), g(4, T, F)
    ids = torch.from_numpy(rng_for(6, 5).integers(0, V, T).astype(np.int32)).cuda()
    pe = ops.pe_table(S, D).cuda()
    gamma, beta = torch.ones(D, device="cuda"), torch.zeros(D, device="cuda")
    x0, y, xh, dx = (torch.empty(T, D, device="cuda") for _ in range(4))
    inv, dg, db = torch.empty(T, device="cuda"), torch.empty(D, device="cuda"), torch.empty(D, device="cuda")
    act, dpre, mask = torch.empty(T, F, device="cuda"), torch.empty(T, F, device="cuda"), ops.act_cache(capi.RELU, pre)
    grad = torch.empty(V, D, device="cuda")
    ws_ln, ws_embed = ops.ln_bwd_workspace(T, D, grad.device), ops.embed_workspace(T, V, D, grad.device)

    def chain():
        ops.embed_sort_tokens(ids, V, D, workspace=ws_embed)
        ops.embed_gather_fwd(table, ids, pe, S, out=x0)
        ops.ln_residual_fwd(x0, res, gamma, beta, 1e-5, y=y, xhat=xh, inv_std=inv)
        ops.act_fwd(capi.RELU, pre, None, y=act, cache=mask)
        ops.act_bwd(capi.RELU, dact, mask, dx=dpre)
        ops.ln_bwd(dy, None, xh, inv, gamma, dx=dx, dgamma=dg, dbeta=db, workspace=ws_ln)
        ops.embed_scatter_bwd(dx, ids, V, ws_embed, grad=grad)

    chain()
    torch.cuda.synchronize()
    want = [t.clone() for t in (y, dx, dg, db, dpre, grad)]
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        chain()
    for t in (y, dx, dg, db, dpre, grad):
        t.fill_(7.0)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    for got, ref in zip((y, dx, dg, db, dpre, grad), want):
        assert torch.equal(got, ref)
    assert capi.pipeline_timeouts() == 0
