"""Token-row sharding of the layer chain over the GPUs of one box.

Every kernel of the path is independent per token row, so rank r of N owns a contiguous
slice of the rows and runs the kernels on it alone; parameters are replicated.  Only the
gradients of parameters couple rows: they are summed over ranks with an all-reduce
(torch.distributed; NCCL on GPUs, gloo in the CPU tests)."""
from __future__ import annotations


def shard_rows(total_rows: int, world_size: int, rank: int, multiple_of: int = 1) -> tuple[int, int]:
    """(first row, row count) of `rank`.  Rows are dealt in units of `multiple_of` rows (e.g. a whole
    sequence, so that a row's position t mod seq_len is the same locally and globally); earlier
    ranks take the remainder units."""
    if not (0 <= rank < world_size) or total_rows < 0 or multiple_of <= 0:
        raise ValueError("bad sharding arguments")
    if total_rows % multiple_of:
        raise ValueError(f"{total_rows} rows are not a multiple of {multiple_of}")
    units = total_rows // multiple_of
    base, extra = divmod(units, world_size)
    mine = base + (1 if rank < extra else 0)
    first = rank * base + min(rank, extra)
    return first * multiple_of, mine * multiple_of


def allreduce_param_grads(dist, small_grads, table_grad) -> None:
    """Sums the parameter gradients over the ranks: one call for the buffer holding every small
    gradient (gamma/beta of the layer norms, biases), one for the embedding-table gradient."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return
    dist.all_reduce(small_grads)
    dist.all_reduce(table_grad)


class PeerExchange:
    """Buffers of the peer-memory exchange of the embedding-table gradient, one object per rank.

    Three symmetric allocations (torch.distributed._symmetric_memory: the same buffer on every rank,
    each mapped into every rank's address space): the receive area [world][cap_rows][d] fp32 that
    peers push partial rows into, the dense [vocab, d] gradient that owners broadcast reduced rows
    into, and the flag words of the barrier.  The kernels and the barrier are the library's own
    (dlb_embed_scatter_bwd_peer, dlb_embed_reduce_broadcast_peer, dlb_peer_barrier); torch only
    allocates and exchanges the memory handles.
    """

    def __init__(self, dist, vocab, d, max_used_rows, device):
        import torch
        import torch.distributed._symmetric_memory as symm
        from . import capi
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        self.vocab, self.d = vocab, d
        self.cap_rows = (max_used_rows + self.world - 1) // self.world
        group = dist.group.WORLD
        self.recv = symm.empty(self.world * self.cap_rows * d, dtype=torch.float32, device=device)
        self.grad = symm.empty(vocab * d, dtype=torch.float32, device=device)
        self.flags = symm.empty(capi.lib().dlb_peer_flags_bytes() // 4, dtype=torch.int32, device=device)
        self.recv.zero_()
        self.flags.zero_()
        self._handles = [symm.rendezvous(t, group) for t in (self.recv, self.grad, self.flags)]
        self.recv_ptrs = [int(p) for p in self._handles[0].buffer_ptrs]
        self.grad_ptrs = [int(p) for p in self._handles[1].buffer_ptrs]
        self.flag_ptrs = [int(p) for p in self._handles[2].buffer_ptrs]
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch = [0, 0, 0, 0]
        torch.cuda.synchronize(device)
        dist.barrier()  # every receive area and flag word is zero before anyone writes

    def table_grad(self):
        return self.grad.view(self.vocab, self.d)

    def barrier(self, channel, stream=None, timeout_ms=2000):
        from . import ops
        self.epoch[channel] += 1
        ops.peer_barrier(self.flag_ptrs, self.rank, channel, self.epoch[channel], self.status, timeout_ms, stream)

    def timed_out(self) -> int:
        """Bit mask of barrier channels whose wait gave up (synchronises)."""
        return int(self.status.item())
