"""Host-side partitioning of the path across GPUs (one process per GPU).

Nothing here touches a device: the functions compute which slice of a tensor a rank owns and
which part of a sorted index list belongs to a rank's slice of an embedding table.  The
element-wise, softmax and pooling operators shard on the leading dimension with no exchange;
`sumall_except_dim<1>` shards on dimension 0 and combines its per-rank partial sums with one
all-reduce; AddTakeGradLargeBatch shards the table by rows, each rank receiving the run of
the sorted list whose keys fall into its rows (the list is sorted, so that run is contiguous).
"""
import numpy as np


def shard_range(n, rank, world):
    """[begin, end) of `n` items owned by `rank`: contiguous, sizes differing by at most one."""
    base, extra = divmod(n, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def route_sorted_indices(sorted_keys, order, num_rows, rank, world):
    """Part of a sorted (key, source-row) list that targets the table rows owned by `rank`.

    Returns (local_keys, local_order, row_begin, row_end); local keys are relative to row_begin,
    and keep their order, so per-row accumulation order is unchanged by the routing.
    """
    row_begin, row_end = shard_range(num_rows, rank, world)
    lo = int(np.searchsorted(sorted_keys, row_begin, side="left"))
    hi = int(np.searchsorted(sorted_keys, row_end, side="left"))
    local = np.ascontiguousarray(sorted_keys[lo:hi] - row_begin, dtype=sorted_keys.dtype)
    return local, np.ascontiguousarray(order[lo:hi]), row_begin, row_end


def allreduce_sum(tensor):
    """In-place sum over all ranks of the default process group (NCCL on GPUs, gloo on CPU)."""
    import torch.distributed as dist
    dist.all_reduce(tensor)
    return tensor
