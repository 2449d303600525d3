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


def hot_rows(sorted_keys, count):
    """The `count` table rows named most often in a sorted key list, ascending.

    With Zipf-distributed indices a few rows receive a large share of the batch (the hottest
    one about 13 % at exponent 1.1), so any ownership rule leaves the owner of those rows with
    far more than 1/world of the work.  These rows are handled by every rank instead.
    """
    if count <= 0 or sorted_keys.size == 0:
        return np.zeros(0, dtype=sorted_keys.dtype)
    uniq, counts = np.unique(sorted_keys, return_counts=True)
    take = np.argsort(-counts, kind="stable")[:count]
    return np.sort(uniq[take]).astype(sorted_keys.dtype)


def route_cyclic_with_hot_rows(sorted_keys, order, num_sources, rank, world, hot):
    """Split a sorted (key, source-row) list for cyclic table ownership with replicated hot rows.

    Table row r is owned by rank r % world and stored there as local row r // world.
      tail  entries whose key is not hot go to the key's owner, keys rewritten to local rows;
            the list stays sorted and every row keeps its accumulation order, so tail rows come
            out bit-identical to the unsharded result.
      hot   entries whose key is hot stay with the rank that owns their SOURCE row (sources are
            sharded contiguously over the batch); their keys are rewritten to positions in
            `hot`.  Each rank sums them into a len(hot) x D partial table; one all-reduce of that
            small table follows, and owners add its rows to theirs.  This changes the order of
            the additions for hot rows only (rounding-level differences).
    Returns (tail_keys, tail_order, hot_keys, hot_order).
    """
    is_hot = np.isin(sorted_keys, hot)
    mine = (~is_hot) & (sorted_keys % world == rank)
    tail_keys = np.ascontiguousarray(sorted_keys[mine] // world, dtype=sorted_keys.dtype)
    tail_order = np.ascontiguousarray(order[mine])
    begin, end = shard_range(num_sources, rank, world)
    local_src = is_hot & (order >= begin) & (order < end)
    hot_keys = np.ascontiguousarray(np.searchsorted(hot, sorted_keys[local_src]), dtype=sorted_keys.dtype)
    hot_order = np.ascontiguousarray(order[local_src])
    return tail_keys, tail_order, hot_keys, hot_order


def rank_order_sum(parts):
    """What the peer-store exchange (mshadow::ps::PeerModel) hands to every rank: the ranks'
    contributions added one after the other in rank order, ((p0 + p1) + p2) + ..., each addition
    rounded to the element type.  `parts` is a sequence of equally shaped numpy arrays, one per
    rank.  Because every rank adds the same values in the same order, all ranks hold the same bits.
    """
    total = np.array(parts[0], copy=True)
    for part in parts[1:]:
        total = (total + part).astype(total.dtype)
    return total


def allreduce_sum(tensor):
    """In-place sum over all ranks of the default process group (NCCL on GPUs, gloo on CPU)."""
    import torch.distributed as dist
    dist.all_reduce(tensor)
    return tensor
