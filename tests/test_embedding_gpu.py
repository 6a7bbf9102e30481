"""Token embedding: gather (+ sinusoidal PE) and the deterministic scatter-add of
the table gradient, through the C ABI, against the oracle, the reference's
known-answer vectors and (where present) the reference's own kernels."""
import numpy as np
import pytest
import torch

from conftest import bits_equal, rel_err, rng_for, zipf_ids
from dl_cuda_b200 import capi, ops
from oracle import cpu as oracle
from oracle import ref as refshim

pytestmark = pytest.mark.gpu


def dev(x, dtype=None):
    if x is None:
        return None
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t if dtype is None else t.to(dtype)


def scatter(dy_t, ids_t, vocab):
    ws = ops.embed_sort_tokens(ids_t, vocab, dy_t.shape[1])
    return ops.embed_scatter_bwd(dy_t, ids_t, vocab, ws)


def test_reference_known_answer():
    # tests/gpu_correctness_tests.cu:196-252 of the reference
    table = np.arange(15, dtype=np.float32).reshape(5, 3)
    ids = np.array([1, 3, 1, 4], np.int32)
    dout = np.repeat(np.arange(1, 5, dtype=np.float32)[:, None], 3, axis=1)
    out = ops.embed_gather_fwd(dev(table), dev(ids)).cpu().numpy()
    assert np.array_equal(out, np.array([[3, 4, 5], [9, 10, 11], [3, 4, 5], [12, 13, 14]], np.float32))
    grad = scatter(dev(dout), dev(ids), 5).cpu().numpy()
    want = np.zeros((5, 3), np.float32)
    want[1], want[3], want[4] = 4.0, 2.0, 4.0
    assert np.array_equal(grad, want)
    if refshim.available():
        out_r, grad_r = refshim.embedding_layer_run(table, ids, dout)
        assert np.array_equal(out, out_r) and np.array_equal(grad, grad_r)


CASES = [  # vocab, d, batch, seq
    (65, 64, 32, 64), (5, 3, 1, 4), (30, 64, 1, 64), (1000, 256, 4, 128), (50, 12, 3, 21), (7, 1024, 2, 9),
    (300, 4096, 2, 50), (129, 100, 5, 33), (17, 8200, 1, 6), (40000, 8, 8, 512), (2, 16, 1, 1),
]


@pytest.mark.parametrize("vocab,d,batch,seq", CASES)
def test_gather_pe_bit_exact(vocab, d, batch, seq):
    n = batch * seq
    table = (0.02 * rng_for(10, 0).standard_normal((vocab, d))).astype(np.float32)
    ids = rng_for(10, 1).integers(0, vocab, n).astype(np.int32)
    ids[0], ids[-1] = 0, vocab - 1
    pe = ops.pe_table(seq, d)
    assert bits_equal(pe.numpy(), oracle.pe_table(seq, d))
    ttable, tids, tpe = dev(table), dev(ids), pe.cuda()
    fused = ops.embed_gather_fwd(ttable, tids, tpe, seq).cpu().numpy()
    assert bits_equal(fused, oracle.embed_gather(table, ids, pe.numpy(), seq))
    plain = ops.embed_gather_fwd(ttable, tids)
    assert bits_equal(plain.cpu().numpy(), oracle.embed_gather(table, ids))
    # the unfused PE layer gives the same bits as the fused gather
    added = ops.pe_add_fwd(plain.view(batch, seq, d), tpe)
    assert bits_equal(added.cpu().numpy().reshape(n, d), fused)
    assert bits_equal(added.cpu().numpy(), oracle.pe_add(plain.cpu().numpy().reshape(batch, seq, d), pe.numpy()))
    if refshim.available():
        g_r = refshim.embed_fwd(ttable, tids)
        assert bits_equal(plain.cpu().numpy(), g_r.cpu().numpy())
        assert bits_equal(added.cpu().numpy(), refshim.pe_add(g_r.view(batch, seq, d), tpe).cpu().numpy())
        assert bits_equal(pe.numpy(), refshim.pe_table(seq, d).numpy())
    # backward of PE is the identity
    assert torch.equal(ops.pe_add_bwd(added), added)


@pytest.mark.parametrize("vocab,d,batch,seq", CASES)
def test_scatter_add_vs_oracle(vocab, d, batch, seq):
    n = batch * seq
    ids = zipf_ids(rng_for(20, 0), n, vocab)
    dy = rng_for(20, 1).standard_normal((n, d)).astype(np.float32)
    grad = scatter(dev(dy), dev(ids), vocab).cpu().numpy()
    # the kernel's association is restated exactly by the segmented oracle: bit-equal
    assert bits_equal(grad, oracle.embed_scatter(dy, ids, vocab, "segmented"))
    assert rel_err(grad, oracle.embed_scatter(dy, ids, vocab, "f64")) <= 1e-5
    assert rel_err(grad, oracle.embed_scatter(dy, ids, vocab, "sequential")) <= 1e-5
    if refshim.available():
        assert rel_err(grad, refshim.embed_bwd(dev(dy), dev(ids), vocab).cpu().numpy()) <= 1e-5


@pytest.mark.parametrize("pattern", ["all_same", "two_hot", "ascending", "descending", "ends"])
def test_scatter_add_edge_patterns(pattern):
    vocab, d, n = 300, 128, 5000
    if pattern == "all_same":
        ids = np.full(n, 123, np.int32)
    elif pattern == "two_hot":
        ids = np.where(np.arange(n) % 3 == 0, 7, 290).astype(np.int32)
    elif pattern == "ascending":
        ids = (np.arange(n) % vocab).astype(np.int32)
    elif pattern == "descending":
        ids = (vocab - 1 - np.arange(n) % vocab).astype(np.int32)
    else:
        ids = np.where(np.arange(n) % 2 == 0, 0, vocab - 1).astype(np.int32)
    dy = rng_for(30, 0).standard_normal((n, d)).astype(np.float32)
    grad = scatter(dev(dy), dev(ids), vocab).cpu().numpy()
    assert bits_equal(grad, oracle.embed_scatter(dy, ids, vocab, "segmented"))
    assert rel_err(grad, oracle.embed_scatter(dy, ids, vocab, "f64")) <= 1e-5


@pytest.mark.parametrize("vocab,d,n", [(500, 8, 70000), (70000, 16, 66000), (300, 64, 65536), (300, 64, 65537)])
def test_scatter_add_many_tokens(vocab, d, n):
    """Above 65536 tokens the plan is built by the multi-kernel radix sort instead of the
    single cluster launch; both sides of the switch must agree with the oracle."""
    ids = zipf_ids(rng_for(21, 0), n, vocab)
    dy = rng_for(21, 1).standard_normal((n, d)).astype(np.float32)
    grad = scatter(dev(dy), dev(ids), vocab).cpu().numpy()
    assert bits_equal(grad, oracle.embed_scatter(dy, ids, vocab, "segmented"))
    assert rel_err(grad, oracle.embed_scatter(dy, ids, vocab, "f64")) <= 1e-5


def test_scatter_add_is_deterministic_and_overwrites():
    vocab, d, n = 2000, 512, 16384
    ids = zipf_ids(rng_for(40, 0), n, vocab)
    dy = rng_for(40, 1).standard_normal((n, d)).astype(np.float32)
    tdy, tids = dev(dy), dev(ids)
    ws = ops.embed_sort_tokens(tids, vocab, d)
    grad = torch.full((vocab, d), 7.0, device="cuda")  # stale contents must vanish
    ops.embed_scatter_bwd(tdy, tids, vocab, ws, grad=grad)
    first = grad.clone()
    for _ in range(3):
        ws2 = ops.embed_sort_tokens(tids, vocab, d)
        again = ops.embed_scatter_bwd(tdy, tids, vocab, ws2)
        assert torch.equal(first, again)
    untouched = np.setdiff1d(np.arange(vocab), ids)
    assert float(first[torch.from_numpy(untouched).cuda()].abs().sum()) == 0.0


@pytest.mark.parametrize("vocab,d,n", [(1000, 256, 512), (65, 64, 2048), (300, 4096, 100)])
def test_embedding_bf16_storage(vocab, d, n):
    bf = torch.bfloat16
    table = dev((0.02 * rng_for(50, 0).standard_normal((vocab, d))).astype(np.float32), bf)
    ids = zipf_ids(rng_for(50, 1), n, vocab)
    seq = n // 4
    pe = ops.pe_table(seq, d)
    out = ops.embed_gather_fwd(table, dev(ids), pe.cuda(), seq)
    want = oracle.embed_gather(table.float().cpu().numpy(), ids, pe.numpy(), seq)
    assert out.dtype == bf
    assert rel_err(out.float().cpu().numpy(), want) <= 1e-2
    dy = dev(rng_for(50, 2).standard_normal((n, d)).astype(np.float32), bf)
    grad = scatter(dy, dev(ids), vocab)
    assert grad.dtype == torch.float32
    # fp32 accumulation of bf16 inputs in the same association: bit-equal to the oracle
    assert bits_equal(grad.cpu().numpy(), oracle.embed_scatter(dy.float().cpu().numpy(), ids, vocab, "segmented"))


def test_out_of_range_ids_stay_inside_the_table():
    table = np.arange(12, dtype=np.float32).reshape(4, 3)
    ids = np.array([0, 3, 99, -5], np.int32)
    out = ops.embed_gather_fwd(dev(table), dev(ids)).cpu().numpy()
    assert np.array_equal(out[2], table[3]) and np.array_equal(out[3], table[0])


def test_sgd_update_matches_reference_formula():
    p = rng_for(60, 0).standard_normal(10007).astype(np.float32)
    g = rng_for(60, 1).standard_normal(10007).astype(np.float32)
    got = ops.sgd_update(dev(p), dev(g), 0.05).cpu().numpy()
    assert bits_equal(got, oracle.sgd_update(p, g, 0.05))
    if refshim.available():
        assert bits_equal(got, refshim.sgd(dev(p), dev(g), 0.05).cpu().numpy())


def test_residual_add_bit_exact():
    for n in (1, 7, 1024, 100003):
        a = rng_for(70, 0).standard_normal(n).astype(np.float32)
        b = rng_for(70, 1).standard_normal(n).astype(np.float32)
        got = ops.residual_add(dev(a), dev(b)).cpu().numpy()
        assert bits_equal(got, oracle.residual_add(a, b))
        if refshim.available():
            assert bits_equal(got, refshim.residual_add(dev(a), dev(b)).cpu().numpy())


def test_plan_and_scatter_back_to_back_without_host_syncs():
    """Plan build, scatter-add and the next batch's upload queued back to back on one stream,
    several batches in a row, with nothing but stream order between them."""
    vocab, d, n = 300, 64, 65536
    want = None
    for rep in range(6):
        ids = zipf_ids(rng_for(21, 0), n, vocab)
        dy = rng_for(21, 1).standard_normal((n, d)).astype(np.float32)
        tids, tdy = dev(ids), dev(dy)
        ws = ops.embed_sort_tokens(tids, vocab, d)
        grad = ops.embed_scatter_bwd(tdy, tids, vocab, ws)
        got = grad.cpu().numpy()
        if want is None:
            want = oracle.embed_scatter(dy, ids, vocab, "segmented")
        assert bits_equal(got, want), f"batch {rep}"


def shard(n, ranks, r):
    """Token range of rank r when n tokens are dealt ceil(n / ranks) per rank (the last may get fewer)."""
    per = (n + ranks - 1) // ranks
    return per, min(n, r * per), min(n, (r + 1) * per)


@pytest.mark.parametrize("vocab,d,n,ranks,storage", [(2000, 256, 4096, 2, "fp32"), (32000, 512, 8192, 4, "bf16"),
                                                     (50, 64, 3000, 3, "fp32"), (300, 4096, 640, 8, "bf16"),
                                                     (97, 128, 4001, 5, "fp32")])
def test_compacted_multi_rank_gradient(vocab, d, n, ranks, storage):
    """The multi-GPU form of the table gradient with the ranks emulated on one GPU: from ONE sort of all
    ranks' ids each rank finds its own tokens, scatter-adds them into the compact [used, d] buffer, the
    buffers are summed (the all-reduce), and the expansion must equal the single-rank dense gradient."""
    dt = torch.bfloat16 if storage == "bf16" else torch.float32
    ids = zipf_ids(rng_for(61, 0), n, vocab)
    dy = dev(rng_for(61, 1).standard_normal((n, d)).astype(np.float32), dt)
    tids = dev(ids)
    dense = scatter(dy, tids, vocab)
    global_plan = ops.embed_sort_tokens(tids, vocab, d)
    used_host = int(np.unique(ids).size)
    total = None
    rank_plan = None
    for r in range(ranks):
        per, lo, hi = shard(n, ranks, r)
        dy_r = dy[lo:hi].contiguous() if hi > lo else dy[:1].contiguous()
        rank_plan = ops.embed_rank_plan(global_plan, n, per, ranks, r, vocab, d)
        used = int(rank_plan[:4].view(torch.int32)[0].item())
        assert used == used_host
        rows = torch.full((min(vocab, n), d), 9.0, device="cuda")  # stale contents must vanish
        ops.embed_scatter_bwd_compact(dy_r, global_plan, n, rank_plan, per, r, rows, vocab)
        assert float(rows[used:].min()) == 9.0 if used < rows.shape[0] else True  # nothing beyond the used rows
        total = rows[:used].clone() if total is None else total + rows[:used]
    grad = torch.full((vocab, d), 5.0, device="cuda")
    ops.embed_expand_rows(total, rank_plan, per, grad, what=1)   # zero the unused rows (can overlap the all-reduce)
    ops.embed_expand_rows(total, rank_plan, per, grad, what=2)   # then copy the reduced rows
    assert rel_err(grad.cpu().numpy(), dense.cpu().numpy()) <= 1e-5
    unused = np.setdiff1d(np.arange(vocab), ids)
    if unused.size:
        assert float(grad[torch.from_numpy(unused).cuda()].abs().sum()) == 0.0
    both = torch.full((vocab, d), 5.0, device="cuda")
    ops.embed_expand_rows(total, rank_plan, per, both, what=3)
    assert torch.equal(both, grad)


def test_rank_plan_against_numpy():
    """Slots, local ranges and source masks of the rank plan, restated with numpy."""
    vocab, d, n, ranks = 500, 64, 6000, 4
    ids = zipf_ids(rng_for(63, 0), n, vocab)
    ids[17] = vocab + 3  # an id outside the table belongs to no row
    tids = dev(ids)
    global_plan = ops.embed_sort_tokens(tids, vocab, d)
    order = np.argsort(ids, kind="stable")
    inside = ids[order] < vocab
    used_rows = np.unique(ids[ids < vocab])
    for r in range(ranks):
        per, lo, hi = shard(n, ranks, r)
        plan = ops.embed_rank_plan(global_plan, n, per, ranks, r, vocab, d)
        ints = plan.view(torch.int32).cpu().numpy()
        used = int(ints[0])
        assert used == used_rows.size
        stride = ((vocab * 4 + 255) // 256) * 64  # int32 words per [V] array (256-byte aligned)
        base = 64                                 # the header takes 256 bytes
        slot_map, used_list = ints[base:base + vocab], ints[base + stride:base + stride + used]
        row_begin = ints[base + 2 * stride:base + 2 * stride + used]
        row_end = ints[base + 3 * stride:base + 3 * stride + used]
        src_mask = ints[base + 4 * stride:base + 4 * stride + used]
        assert np.array_equal(used_list, used_rows)
        mine_rows = np.unique(ids[lo:hi][ids[lo:hi] < vocab])
        assert int(ints[3]) == mine_rows.size  # rows this rank has tokens for
        local_counts = np.bincount(ids[lo:hi][ids[lo:hi] < vocab], minlength=vocab)
        assert int(ints[6]) == int((local_counts > 1).sum())  # of those, rows with several tokens
        mine_stride = (min(vocab, per) * 4 + 255) // 256 * 64  # int32 words per [my rows] array
        my_route = ints[base + 8 * stride:base + 8 * stride + mine_rows.size]
        my_src = ints[base + 8 * stride + mine_stride:base + 8 * stride + mine_stride + mine_rows.size]
        my_slot = ints[base + 8 * stride + 2 * mine_stride:base + 8 * stride + 2 * mine_stride + mine_rows.size]
        slot_of = {int(v): i for i, v in enumerate(used_rows)}
        assert np.array_equal(used_rows[my_slot], mine_rows)
        global_counts = np.bincount(ids[ids < vocab], minlength=vocab)
        sources = np.array([bin(int(m)).count("1") for m in src_mask])
        assert int(ints[7]) == int(((sources >= 2) & (np.arange(used) % ranks == r)).sum())
        assert int(ints[8]) == int(((sources == 1) & (src_mask != (1 << r)) & (global_counts[used_rows] == 1)).sum())
        multi_seen = 0
        for k, v in enumerate(mine_rows):
            sole = src_mask[slot_of[int(v)]] == (1 << r)
            want_route = (int(v) | 0x80000000) - (1 << 32) if sole else slot_of[int(v)]
            assert int(my_route[k]) == want_route
            if local_counts[v] == 1:
                assert lo + int(my_src[k]) == int(np.flatnonzero(ids[lo:hi] == v)[0]) + lo
            else:
                multi_seen += 1
                assert int(my_src[k]) == -multi_seen
        for slot in range(0, used, 7):
            v = used_rows[slot]
            toks = order[inside & (ids[order] == v)]
            assert src_mask[slot] == sum(1 << int(q) for q in np.unique(toks // per))
            mine = toks[(toks >= lo) & (toks < hi)]
            assert row_end[slot] - row_begin[slot] == mine.size
            if mine.size:
                pos = np.flatnonzero(order == mine[0])[0]
                assert row_begin[slot] == pos
                assert np.array_equal(order[row_begin[slot]:row_end[slot]], mine)


class EmulatedRanks:
    """Every rank's peer buffers on this one GPU (the "mappings" are the plain addresses)."""

    def __init__(self, ranks, vocab, d, cap, small_n, narrow=True):
        z = lambda k: torch.zeros(k, device="cuda")
        self.recv = [torch.full((ranks * cap * d,), 3.0, device="cuda") for _ in range(ranks)]  # needs no zeroing
        self.tables = [torch.full((vocab, d), 5.0, device="cuda") for _ in range(ranks)]
        self.flags = [torch.zeros(capi.lib().dlb_peer_flags_bytes() // 4, dtype=torch.int32, device="cuda") for _ in range(ranks)]
        self.small = [z(max(ranks * small_n, 4)) for _ in range(ranks)]
        self.status = [torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(ranks)]
        # rows whose one token lies on another rank arrive here as bf16 and are widened by the receiver
        self.stage = [torch.full((ranks * cap * d,), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(ranks)] \
            if narrow else None
        addr = lambda ts: [t.data_ptr() for t in ts]
        self.groups = [ops.peer_group(ranks, r, cap, addr(self.flags), addr(self.recv), addr(self.tables), self.status[r],
                                      addr(self.small) if small_n else None, small_n, timeout_ms=1000,
                                      stage=addr(self.stage) if narrow else None)
                       for r in range(ranks)]


@pytest.mark.parametrize("storage", ["fp32", "bf16", "bf16-wide"])
@pytest.mark.parametrize("vocab,d,n,ranks", [(50, 64, 300, 2), (1000, 256, 5000, 4), (32000, 512, 16384, 8),
                                             (97, 128, 4000, 3), (50, 64, 300, 1), (300, 4096, 2000, 16)])
def test_peer_exchange_with_the_ranks_emulated_on_one_gpu(vocab, d, n, ranks, storage):
    """The peer-memory form of the table-gradient exchange, every rank's buffers on this one GPU and the
    phases run rank after rank (all pushes, then all owner sums: every flag is set before it is waited
    for, so no kernel waits for a later launch).  A row one rank alone has tokens for is stored into every
    table by that rank; a shared row goes to its owner, which adds the partial rows in rank order and
    stores the sum into every table; every rank zeroes the rows nobody uses in its own table; the small
    gradients of all ranks are summed in rank order.  Every table must equal the single-rank dense
    gradient, twice in a row with stale tables and receive areas.  With bf16 storage a row whose one
    token lies on another rank travels as bf16 through a staging area and is widened by the receiver
    ("bf16-wide": without staging areas every row travels as fp32); the second round lets every rank
    clear its unused rows with dlb_embed_expand_rows instead of inside the push kernel."""
    dt = torch.float32 if storage == "fp32" else torch.bfloat16
    ids = zipf_ids(rng_for(71, 0), n, vocab)
    dy = dev(rng_for(71, 1).standard_normal((n, d)).astype(np.float32), dt)
    tids = dev(ids)
    dense = scatter(dy, tids, vocab).cpu().numpy()
    # The sums in double.  Hot rows add thousands of N(0,1) terms in fp32 and the error measure divides by the
    # rms of a table that is mostly zero rows, so the single-rank gradient itself sits at 1.1e-5 from them at
    # the largest case; every grouping is held to 3e-5 here.
    exact = np.zeros((vocab, d), np.float64)
    np.add.at(exact, ids, dy.float().cpu().numpy().astype(np.float64))
    assert rel_err(dense, exact) <= 3e-5
    global_plan = ops.embed_sort_tokens(tids, vocab, d)
    max_rows = min(vocab, n)
    cap = (max_rows + ranks - 1) // ranks
    small_n = 24
    em = EmulatedRanks(ranks, vocab, d, cap, small_n, narrow=storage != "bf16-wide")
    code = capi.F32 if storage == "fp32" else capi.BF16
    small_in = [dev(rng_for(73, r).standard_normal(small_n).astype(np.float32)) for r in range(ranks)]
    small_want = small_in[0].clone()
    for r in range(1, ranks):
        small_want = small_want + small_in[r]
    for attempt in range(2):
        epoch = attempt + 1
        plans, small_out = [], [torch.full((small_n,), 9.0, device="cuda") for _ in range(ranks)]
        for r in range(ranks):
            per, lo, hi = shard(n, ranks, r)
            plans.append(ops.embed_rank_plan(global_plan, n, per, ranks, r, vocab, d))
        for r in range(ranks):
            per, lo, hi = shard(n, ranks, r)
            dy_r = dy[lo:hi].contiguous() if hi > lo else dy[:1].contiguous()
            if attempt == 1:
                ops.embed_expand_rows(None, plans[r], per, em.tables[r], what=1)
            # first round in one call; second round in the three parts a caller overlaps on two streams
            for part in ((0,) if attempt == 0 else (1, 2, 3)):
                ops.embed_scatter_bwd_peer(dy_r, global_plan, n, plans[r], per, em.groups[r], small_in[r], max_rows, vocab,
                                           0, epoch, clear_unused=int(attempt == 0), part=part)
        for r in range(ranks):
            ops.embed_reduce_broadcast_peer(plans[r], per, em.groups[r], small_out[r], vocab, d, code, 0, epoch, 1, epoch)
        for r in range(ranks):
            ops.peer_wait([f.data_ptr() for f in em.flags], r, 1, epoch, em.status[r], timeout_ms=1000)
        torch.cuda.synchronize()
        for r in range(ranks):
            assert int(em.status[r].item()) == 0, (attempt, r)
            got = em.tables[r].cpu().numpy()
            assert rel_err(got, exact) <= 3e-5, (attempt, r)
            assert rel_err(got, dense) <= 3e-5, (attempt, r)  # two fp32 groupings of the same terms
            assert torch.equal(small_out[r], small_want), (attempt, r)
            if r:
                assert torch.equal(em.tables[r], em.tables[0])  # every rank holds the same bits
        for t in em.tables:
            t.fill_(7.0)


@pytest.mark.parametrize("storage", ["fp32", "bf16"])
def test_peer_exchange_clears_only_what_the_last_step_wrote(storage):
    """clear_unused = 2 with the ranks emulated: three steps with different ids, nothing else touching the
    tables in between.  Step 0 finds no record (the rank plan workspaces start zero-filled) and garbage in
    the tables, so it clears everything; steps 1 and 2 clear only the rows of the step before them that
    they do not write.  After every step every table equals the single-rank dense gradient."""
    vocab, d, n, ranks, small_n = 3000, 256, 6000, 4, 0
    dt = torch.float32 if storage == "fp32" else torch.bfloat16
    code = capi.F32 if storage == "fp32" else capi.BF16
    max_rows = min(vocab, n)
    cap = (max_rows + ranks - 1) // ranks
    em = EmulatedRanks(ranks, vocab, d, cap, small_n)
    per = shard(n, ranks, 0)[0]
    plans = [ops.embed_rank_plan_workspace(vocab, per, d, "cuda") for _ in range(ranks)]
    for step in range(3):
        ids = zipf_ids(rng_for(81 + step, 0), n, vocab)
        dy = dev(rng_for(81 + step, 1).standard_normal((n, d)).astype(np.float32), dt)
        tids = dev(ids)
        dense = scatter(dy, tids, vocab)
        global_plan = ops.embed_sort_tokens(tids, vocab, d)
        for r in range(ranks):
            ops.embed_rank_plan(global_plan, n, per, ranks, r, vocab, d, rank_plan=plans[r])
        for r in range(ranks):
            _, lo, hi = shard(n, ranks, r)
            ops.embed_scatter_bwd_peer(dy[lo:hi].contiguous(), global_plan, n, plans[r], per, em.groups[r], None, max_rows,
                                       vocab, 0, step + 1, clear_unused=2)
        for r in range(ranks):
            ops.embed_reduce_broadcast_peer(plans[r], per, em.groups[r], None, vocab, d, code, 0, step + 1, 1, step + 1)
        torch.cuda.synchronize()
        for r in range(ranks):
            assert int(em.status[r].item()) == 0
            assert rel_err(em.tables[r].cpu().numpy(), dense.cpu().numpy()) <= 3e-5, (step, r)
            assert torch.equal(em.tables[r], em.tables[0])
        used_now = np.unique(ids)
        assert float(em.tables[0][torch.from_numpy(np.setdiff1d(np.arange(vocab), used_now)).cuda()].abs().sum()) == 0.0


def test_peer_reduce_reports_a_receive_area_that_is_too_small():
    """cap_rows smaller than the rows an owner holds: the kernel drops those rows, raises bit 31 of the
    status word and touches nothing outside the receive area."""
    vocab, d, n, ranks = 400, 64, 3000, 2
    ids = rng_for(75, 0).integers(0, vocab, n).astype(np.int32)  # every row used by both ranks
    tids = dev(ids)
    global_plan = ops.embed_sort_tokens(tids, vocab, d)
    cap = 20  # 2 * 20 = 40 slots, far fewer than the ~400 used rows
    em = EmulatedRanks(ranks, vocab, d, cap, 0)
    per, lo, hi = shard(n, ranks, 0)
    plan = ops.embed_rank_plan(global_plan, n, per, ranks, 0, vocab, d)
    guard = em.recv[0].clone()
    ops.embed_reduce_broadcast_peer(plan, per, em.groups[0], None, vocab, d, capi.F32, 3, 0, 1, 1)  # epoch 0: no wait
    torch.cuda.synchronize()
    assert (int(em.status[0].item()) & 0xffffffff) == 1 << 31
    assert torch.equal(em.recv[0], guard)


def test_peer_put_gathers_and_waits():
    """dlb_peer_put with the ranks emulated: all pushes first (no wait), then the waits pass at once."""
    ranks, k = 4, 1024
    flags = [torch.zeros(capi.lib().dlb_peer_flags_bytes() // 4, dtype=torch.int32, device="cuda") for _ in range(ranks)]
    gathered = [torch.zeros(ranks * k, dtype=torch.int32, device="cuda") for _ in range(ranks)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    mine = [torch.arange(k, dtype=torch.int32, device="cuda") + 1000 * r for r in range(ranks)]
    fl, dst = [f.data_ptr() for f in flags], [g.data_ptr() for g in gathered]
    for r in range(ranks):
        ops.peer_put(mine[r], dst, fl, r, 2, 1, status, wait=False, timeout_ms=1000)
    for r in range(ranks):
        ops.peer_wait(fl, r, 2, 1, status, timeout_ms=1000)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for r in range(ranks):
        assert torch.equal(gathered[r], torch.cat(mine))
    # alone in its group a rank gathers from itself and passes its own wait
    solo = torch.zeros(k, dtype=torch.int32, device="cuda")
    ops.peer_put(mine[1], [solo.data_ptr()], [flags[0].data_ptr()], 0, 3, 1, status, wait=True, timeout_ms=1000)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and torch.equal(solo, mine[1])


def test_peer_barrier_single_rank_and_timeout():
    """n = 1: the rank signals itself and passes.  A flag nobody sets: the wait runs out after the given time,
    the status bit of the channel is set and the stream keeps working."""
    flags = torch.zeros(capi.lib().dlb_peer_flags_bytes() // 4, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for epoch in (1, 2, 3):
        ops.peer_barrier([flags.data_ptr()], 0, 1, epoch, status, timeout_ms=1000)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert int(flags[16].item()) == 3  # channel 1, source rank 0
    # two ranks, but the other one never arrives (its flag array is a second buffer that nothing writes)
    other = torch.zeros_like(flags)
    ops.peer_barrier([flags.data_ptr(), other.data_ptr()], 0, 2, 1, status, timeout_ms=50)
    probe = ops.residual_add(torch.ones(8, device="cuda"), torch.ones(8, device="cuda"))
    torch.cuda.synchronize()
    assert int(status.item()) == 1 << 2
    assert int(other[2 * 16].item()) == 1      # the announcement to the absent rank was made
    assert float(probe.sum()) == 16.0          # the context is alive


def test_peer_entry_points_reject_bad_arguments():
    import ctypes
    lib = capi.lib()
    vocab, d, n = 50, 64, 100
    ids = dev(zipf_ids(rng_for(72, 0), n, vocab))
    dy = dev(rng_for(72, 1).standard_normal((n, d)).astype(np.float32))
    plan = ops.embed_sort_tokens(ids, vocab, d)
    rank_plan = ops.embed_rank_plan(plan, n, 50, 2, 0, vocab, d)
    em = EmulatedRanks(2, vocab, d, 25, 0)
    recv_before = em.recv[0].clone()

    def scatter_status(group, max_rows=50, channel=0):
        return lib.dlb_embed_scatter_bwd_peer(dy.data_ptr(), plan.data_ptr(), n, rank_plan.data_ptr(), 50,
                                              ctypes.byref(group), None, max_rows, 1, 0, vocab, d, capi.F32, channel, 1, None)

    def group(**changes):
        g = ops.peer_group(2, 0, 25, [f.data_ptr() for f in em.flags], [t.data_ptr() for t in em.recv],
                           [t.data_ptr() for t in em.tables], em.status[0], None, 0, 1000)
        for k, v in changes.items():
            setattr(g, k, v)
        return g

    assert scatter_status(group(n_ranks=0)) == capi.ERR_INVALID_ARG       # no ranks
    assert scatter_status(group(n_ranks=17)) == capi.ERR_INVALID_ARG      # more than 16 ranks
    assert scatter_status(group(my_rank=2)) == capi.ERR_INVALID_ARG       # rank out of range
    assert scatter_status(group(cap_rows=10)) == capi.ERR_INVALID_ARG     # receive areas too small for max_rows
    assert scatter_status(group(timeout_ms=0)) == capi.ERR_INVALID_ARG
    assert scatter_status(group(small_n=6)) == capi.ERR_INVALID_ARG       # not a multiple of 4
    assert scatter_status(group(), channel=4) == capi.ERR_INVALID_ARG
    broken = group()
    broken.recv[1] = None
    assert scatter_status(broken) == capi.ERR_INVALID_ARG                 # a null receive area
    assert lib.dlb_embed_reduce_broadcast_peer(rank_plan.data_ptr(), 50, ctypes.byref(group(my_rank=5)), None, vocab, d,
                                               capi.F32, 0, 1, 1, 1, None) == capi.ERR_INVALID_ARG
    assert lib.dlb_embed_reduce_broadcast_peer(None, 50, ctypes.byref(group()), None, vocab, d, capi.F32, 0, 1, 1, 1, None) \
        == capi.ERR_WORKSPACE
    assert lib.dlb_embed_reduce_broadcast_peer(rank_plan.data_ptr(), 50, ctypes.byref(group()), None, vocab, d, 7, 0, 1, 1,
                                               1, None) == capi.ERR_INVALID_ARG      # unknown dtype
    assert lib.dlb_embed_rank_plan(plan.data_ptr(), n, 10, 2, 0, rank_plan.data_ptr(), rank_plan.numel(), vocab, d, None) \
        == capi.ERR_INVALID_ARG                                           # 2 ranks of 10 tokens do not cover 100
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    one = ops._addr_array([flags.data_ptr()])
    assert lib.dlb_peer_barrier(one, 1, 0, 4, 1, 100, status.data_ptr(), None) == capi.ERR_INVALID_ARG    # channel
    assert lib.dlb_peer_barrier(one, 1, 0, 0, 1, 0, status.data_ptr(), None) == capi.ERR_INVALID_ARG      # timeout
    assert lib.dlb_peer_barrier(one, 1, 0, 0, 1, 100, None, None) == capi.ERR_INVALID_ARG                 # status
    assert lib.dlb_peer_put(flags.data_ptr(), 24, one, one, 1, 0, 0, 1, 0, 100, status.data_ptr(), None) \
        == capi.ERR_INVALID_ARG                                                                          # 24 bytes
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and torch.equal(em.recv[0], recv_before)
    assert all(float((t - 5.0).abs().sum()) == 0.0 for t in em.tables)
