"""Worker of tests/test_multi_gpu.py: one process per GPU (torchrun), NCCL for the plumbing.

Every rank holds a shard of the tokens.  The table gradient is computed through the peer-memory exchange
(dlb_embed_scatter_bwd_peer -> dlb_peer_barrier -> dlb_embed_reduce_broadcast_peer -> dlb_peer_barrier) three
steps in a row with fresh ids and gradients, and checked on every rank against the dense single-rank
gradient of ALL tokens (gathered here only for the check).  Prints "PEER_EXCHANGE_OK <rank>" on success.
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
from dl_cuda_b200 import ops  # noqa: E402
from dl_cuda_b200.sharding import PeerExchange  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    vocab, d, per_rank = 4000, 512, 3000
    total = per_rank * world
    px = PeerExchange(dist, vocab, d, min(vocab, total), dev)
    table = px.table_grad()
    side = torch.cuda.Stream()
    for step in range(3):
        ids_all = torch.from_numpy(zipf_ids(rng_for(500 + step, 0), total, vocab).astype(np.int32)).to(dev)
        dy_all = torch.from_numpy(rng_for(500 + step, 1).standard_normal((total, d)).astype(np.float32)).to(dev)
        ids, dy = ids_all[rank * per_rank:(rank + 1) * per_rank].contiguous(), dy_all[rank * per_rank:(rank + 1) * per_rank].contiguous()
        gathered = torch.empty(total, dtype=torch.int32, device=dev)
        dist.all_gather_into_tensor(gathered, ids)
        assert torch.equal(gathered, ids_all)
        local_plan = ops.embed_sort_tokens(ids, vocab, d)
        global_plan = ops.embed_sort_tokens(gathered, vocab, d)
        compact = ops.embed_compact_plan(global_plan, total, local_plan, per_rank, vocab, d)
        used = int(compact[:4].view(torch.int32)[0].item())
        table.fill_(float(3 + step))  # stale contents must vanish
        torch.cuda.synchronize()
        dist.barrier()                # nobody pushes rows into a table that is still being filled
        ops.embed_scatter_bwd_peer(dy, local_plan, compact, px.recv_ptrs, rank, px.cap_rows,
                                   used if step == 0 else min(vocab, total), vocab)
        side.wait_stream(torch.cuda.current_stream())
        ops.embed_expand_rows(None, compact, table, what=1, stream=side.cuda_stream)
        px.barrier(0)
        ops.embed_reduce_broadcast_peer(px.recv, compact, px.grad_ptrs, rank, px.cap_rows, vocab, d)
        torch.cuda.current_stream().wait_stream(side)
        px.barrier(1)
        torch.cuda.synchronize()
        assert px.timed_out() == 0, "a barrier wait gave up"
        want = torch.zeros(vocab, d, device=dev)
        ops.embed_scatter_bwd(dy_all, ids_all, vocab, global_plan, grad=want)
        err = rel_err(table.cpu().numpy(), want.cpu().numpy())
        assert err <= 3e-5, (step, rank, err)
        assert float(px.recv.abs().sum()) == 0.0, "receive area must be zero again"
        # every rank holds the same bits
        mine = table.clone()
        dist.broadcast(mine, src=0)
        assert torch.equal(mine, table), (step, rank)
    print(f"PEER_EXCHANGE_OK {rank}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
