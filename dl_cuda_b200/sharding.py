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
