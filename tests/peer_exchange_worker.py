"""Worker of tests/test_multi_gpu.py: one process per GPU (torchrun), NCCL for the plumbing.

Every rank holds a shard of the tokens.  The table gradient is computed through the peer-memory exchange
(dlb_peer_put of the ids -> one sort -> dlb_embed_rank_plan -> dlb_embed_scatter_bwd_peer ->
dlb_embed_reduce_broadcast_peer -> dlb_peer_wait) three steps in a row with fresh ids and gradients, and
checked on every rank against the dense single-rank gradient of ALL tokens (gathered here only for the
check); so are the small gradients that ride along.  Prints "PEER_EXCHANGE_OK <rank>" on success.
"""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
sys.path.insert(0, str(Path(__file__).resolve().parent))

from conftest import rel_err, rng_for, zipf_ids  # noqa: E402
from dl_cuda_b200 import capi, ops  # noqa: E402
from dl_cuda_b200.sharding import PeerExchange  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    vocab, d, per_rank, small_n = 4000, 512, 3000, 1024
    total = per_rank * world
    px = PeerExchange(dist, vocab, d, min(vocab, total), dev, tokens_per_rank=per_rank, small_n=small_n)
    px.barrier()
    table = px.table_grad()
    for step in range(3):
        ids_all = torch.from_numpy(zipf_ids(rng_for(500 + step, 0), total, vocab).astype(np.int32)).to(dev)
        dy_all = torch.from_numpy(rng_for(500 + step, 1).standard_normal((total, d)).astype(np.float32)).to(dev)
        small_all = torch.from_numpy(rng_for(500 + step, 2).standard_normal((world, small_n)).astype(np.float32)).to(dev)
        if step % 2:  # bf16 storage: rows with one token in all travel as bf16 and are widened by the receivers
            dy_all = dy_all.to(torch.bfloat16)
        ids, dy = ids_all[rank * per_rank:(rank + 1) * per_rank].contiguous(), dy_all[rank * per_rank:(rank + 1) * per_rank].contiguous()
        small = small_all[rank].clone()
        table.fill_(float(3 + step))  # stale contents must vanish
        # The gather of the ids is the barrier that keeps a fast rank from storing rows into a table its
        # owner is still filling (or, in training, still reading): it is stream-ordered after the fill.
        px.gather_ids(ids)
        gathered = px.ids_all[:total]
        global_plan = ops.embed_sort_tokens(gathered, vocab, d)
        rank_plan = ops.embed_rank_plan(global_plan, total, per_rank, world, rank, vocab, d)
        pushed, done = px.next_epoch(px.CH_PUSHED), px.next_epoch(px.CH_DONE)
        ops.embed_scatter_bwd_peer(dy, global_plan, total, rank_plan, per_rank, px.group, small, min(vocab, total), vocab,
                                   px.CH_PUSHED, pushed)
        ops.embed_reduce_broadcast_peer(rank_plan, per_rank, px.group, small, vocab, d, capi.dtype_of(dy), px.CH_PUSHED,
                                        pushed, px.CH_DONE, done)
        px.wait(px.CH_DONE)
        torch.cuda.synchronize()
        assert px.timed_out() == 0, "a wait gave up or the receive area was too small"
        assert torch.equal(gathered, ids_all)
        want = torch.zeros(vocab, d, device=dev)
        ops.embed_scatter_bwd(dy_all, ids_all, vocab, ops.embed_sort_tokens(ids_all, vocab, d), grad=want)
        err = rel_err(table.cpu().numpy(), want.cpu().numpy())
        assert err <= 3e-5, (step, rank, err)
        want_small = small_all[0].clone()
        for r in range(1, world):
            want_small = want_small + small_all[r]
        assert torch.equal(small, want_small), (step, rank)
        # every rank holds the same bits
        mine = table.clone()
        dist.broadcast(mine, src=0)
        assert torch.equal(mine, table), (step, rank)
    print(f"PEER_EXCHANGE_OK {rank}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
