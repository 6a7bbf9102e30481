"""Host logic of the multi-GPU path on CPU: two gloo ranks each run their token shard through the
oracle and all-reduce the parameter gradients; the result must match the unsharded run."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import rel_err, rng_for
from dl_cuda_b200.sharding import allreduce_param_grads, shard_positions, shard_rows


def test_shard_rows_covers_everything_once():
    for total, world, mult in [(32768, 8, 4096), (32768, 4, 4096), (10, 3, 1), (12, 5, 2), (0, 2, 1), (7, 8, 1)]:
        spans = [shard_rows(total, world, r, mult) for r in range(world)]
        assert spans[0][0] == 0
        for (a, n), (b, _) in zip(spans, spans[1:]):
            assert a + n == b and n % mult == 0
        assert spans[-1][0] + spans[-1][1] == total
    with pytest.raises(ValueError):
        shard_rows(10, 2, 2)
    with pytest.raises(ValueError):
        shard_rows(10, 2, 0, 4)


def _problem():
    rows, d, vocab, seq = 64, 24, 17, 16
    g = rng_for(77, 0)
    return dict(rows=rows, d=d, vocab=vocab, seq=seq,
                dy=g.standard_normal((rows, d)).astype(np.float32),
                xhat=g.standard_normal((rows, d)).astype(np.float32),
                ids=g.integers(0, vocab, rows).astype(np.int32),
                dx=g.standard_normal((rows, d)).astype(np.float32))


def _rank_main(rank, world, port, out):
    from oracle import cpu as oracle
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    p = _problem()
    first, n = shard_rows(p["rows"], world, rank, p["seq"])
    sl = slice(first, first + n)
    dgamma, dbeta = np.zeros(p["d"], np.float32), np.zeros(p["d"], np.float32)
    grad = np.zeros((p["vocab"], p["d"]), np.float32)
    if n:
        inv = np.ones(n, np.float32)
        _, dgamma, dbeta = oracle.ln_bwd(p["dy"][sl], None, p["xhat"][sl], inv, np.ones(p["d"], np.float32))
        grad = oracle.embed_scatter(p["dx"][sl], p["ids"][sl], p["vocab"])
    small = torch.from_numpy(np.concatenate([dgamma, dbeta]))
    table = torch.from_numpy(grad)
    allreduce_param_grads(dist, small, table)
    if rank == 0:
        out.put((small.numpy().copy(), table.numpy().copy()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_match_the_unsharded_result():
    from oracle import cpu as oracle
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, out)) for r in range(2)]
    for pr in procs:
        pr.start()
    small, table = out.get(timeout=120)
    for pr in procs:
        pr.join(timeout=120)
        assert pr.exitcode == 0
    p = _problem()
    _, dgamma, dbeta = oracle.ln_bwd(p["dy"], None, p["xhat"], np.ones(p["rows"], np.float32), np.ones(p["d"], np.float32))
    grad = oracle.embed_scatter(p["dx"], p["ids"], p["vocab"])
    assert rel_err(small[: p["d"]], dgamma) <= 1e-5 and rel_err(small[p["d"]:], dbeta) <= 1e-5
    assert rel_err(table, grad) <= 1e-5


def test_shard_positions_covers_every_token_once():
    batch, seq = 8, 4096
    for world in (1, 2, 4, 8):
        seen = np.zeros((batch, seq), np.int32)
        for r in range(world):
            first, positions, rows = shard_positions(batch, seq, world, r)
            assert rows == batch * positions
            local = np.arange(rows)
            seen[local // positions, first + local % positions] += 1
        assert (seen == 1).all()
    with pytest.raises(ValueError):
        shard_positions(8, 4096, 3, 0)
    with pytest.raises(ValueError):
        shard_positions(8, 4096, 4, 4)


def test_position_shards_reproduce_the_unsharded_forward():
    """A rank that takes positions [first, first + n) of every sequence, with its n rows of the PE table and
    seq_len = n, computes exactly the rows b * seq + first + p of the unsharded gather + PE output."""
    from oracle import cpu as oracle
    batch, seq, d, vocab = 3, 8, 12, 11
    g = rng_for(78, 0)
    table = (0.02 * g.standard_normal((vocab, d))).astype(np.float32)
    ids = g.integers(0, vocab, batch * seq).astype(np.int32)
    pe = oracle.pe_table(seq, d)
    whole = oracle.embed_gather(table, ids, pe, seq).reshape(batch, seq, d)
    for world in (1, 2, 4, 8):
        for r in range(world):
            first, n, rows = shard_positions(batch, seq, world, r)
            local_ids = ids.reshape(batch, seq)[:, first:first + n].reshape(-1).copy()
            out = oracle.embed_gather(table, local_ids, np.ascontiguousarray(pe[first:first + n]), n)
            assert rows == local_ids.size
            assert np.array_equal(out.reshape(batch, n, d), whole[:, first:first + n])
