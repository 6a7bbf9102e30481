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


def shard_positions(batch: int, seq_len: int, world_size: int, rank: int) -> tuple[int, int, int]:
    """(first position, positions, local token rows) of `rank` when every rank takes the same slice of
    positions of ALL `batch` sequences instead of whole sequences.  A rank's local rows are ordered
    [sequence][position of its slice], so a row's position is first + (local row mod positions) and the
    rank reads only its `positions` rows of the positional-encoding table, each shared by `batch` token
    rows (with whole sequences per rank, a rank with one sequence reads one table row per token).
    seq_len must divide evenly; shard_rows is the fallback."""
    if not (0 <= rank < world_size) or batch <= 0 or seq_len <= 0:
        raise ValueError("bad sharding arguments")
    if seq_len % world_size:
        raise ValueError(f"{seq_len} positions do not divide over {world_size} ranks")
    positions = seq_len // world_size
    return rank * positions, positions, batch * positions


def allreduce_param_grads(dist, small_grads, table_grad) -> None:
    """Sums the parameter gradients over the ranks: one call for the buffer holding every small
    gradient (gamma/beta of the layer norms, biases), one for the embedding-table gradient."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return
    dist.all_reduce(small_grads)
    dist.all_reduce(table_grad)


class PeerExchange:
    """Buffers and step counters of the peer-memory exchange of the embedding-table gradient, one
    object per rank.

    Symmetric allocations (torch.distributed._symmetric_memory: the same buffer on every rank, each
    mapped into every rank's address space): the receive area [world][cap_rows][d] fp32 that peers push
    shared rows into, the dense [vocab, d] gradient that finished rows are stored into, the area the
    small parameter gradients of every rank land in, the gathered token ids of all ranks, the staging
    rows for gradients that travel as bf16, and the flag words.  The kernels, the flags and the waits are the library's own (dlb_peer_put,
    dlb_embed_scatter_bwd_peer, dlb_embed_reduce_broadcast_peer, dlb_peer_wait); torch only allocates
    the memory and exchanges its handles.

    Channels: 0 = partial rows pushed, 1 = tables complete, 2 = token ids gathered, 3 = set-up barrier.
    """

    CH_PUSHED, CH_DONE, CH_IDS, CH_SETUP = 0, 1, 2, 3

    def __init__(self, dist, vocab, d, max_used_rows, device, tokens_per_rank=0, small_n=0, timeout_ms=2000,
                 narrow_rows=True):
        import torch
        import torch.distributed._symmetric_memory as symm
        from . import capi, ops
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        self.vocab, self.d = vocab, d
        self.cap_rows = (max_used_rows + self.world - 1) // self.world
        self.small_n = small_n
        self.timeout_ms = timeout_ms
        group = dist.group.WORLD
        f32 = dict(dtype=torch.float32, device=device)
        self.recv = symm.empty(self.world * self.cap_rows * d, **f32)
        self.grad = symm.empty(vocab * d, **f32)
        self.flags = symm.empty(capi.lib().dlb_peer_flags_bytes() // 4, dtype=torch.int32, device=device)
        self.small = symm.empty(max(self.world * small_n, 4), **f32)
        self.ids_all = symm.empty(max(self.world * tokens_per_rank, 4), dtype=torch.int32, device=device)
        # rows that travel as bf16 (one token in all): [cap_rows * world][d] bf16 on every rank
        self.stage = symm.empty(self.world * self.cap_rows * d if narrow_rows else 8, dtype=torch.bfloat16, device=device)
        self.flags.zero_()
        buffers = (self.recv, self.grad, self.flags, self.small, self.ids_all, self.stage)
        self._handles = [symm.rendezvous(t, group) for t in buffers]
        ptrs = [[int(p) for p in h.buffer_ptrs] for h in self._handles]
        self.recv_ptrs, self.grad_ptrs, self.flag_ptrs, self.small_ptrs, self.ids_ptrs, self.stage_ptrs = ptrs
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.group = ops.peer_group(self.world, self.rank, self.cap_rows, self.flag_ptrs, self.recv_ptrs,
                                    self.grad_ptrs, self.status, self.small_ptrs if small_n else None, small_n,
                                    timeout_ms, self.stage_ptrs if narrow_rows else None)
        self.epoch = [0, 0, 0, 0]
        torch.cuda.synchronize(device)
        dist.barrier()  # every flag word is zero before anyone writes

    def table_grad(self):
        return self.grad.view(self.vocab, self.d)

    def next_epoch(self, channel) -> int:
        self.epoch[channel] += 1
        return self.epoch[channel]

    def barrier(self, channel=CH_SETUP, stream=None):
        from . import ops
        ops.peer_barrier(self.flag_ptrs, self.rank, channel, self.next_epoch(channel), self.status, self.timeout_ms, stream)

    def wait(self, channel, stream=None):
        """Waits for the announcement a kernel made with the channel's current epoch."""
        from . import ops
        ops.peer_wait(self.flag_ptrs, self.rank, channel, self.epoch[channel], self.status, self.timeout_ms, stream)

    def gather_ids(self, ids, stream=None):
        """All-gather of this rank's token ids into ids_all on every rank (one kernel: push, announce, wait)."""
        from . import ops
        ops.peer_put(ids, self.ids_ptrs, self.flag_ptrs, self.rank, self.CH_IDS, self.next_epoch(self.CH_IDS),
                     self.status, True, self.timeout_ms, stream)

    def timed_out(self) -> int:
        """Status bits (synchronises): bit c = a wait on channel c gave up; bit 31 = cap_rows too small."""
        return int(self.status.item()) & 0xffffffff
