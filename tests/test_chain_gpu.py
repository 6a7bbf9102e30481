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
