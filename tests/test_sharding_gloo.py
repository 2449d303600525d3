"""The multi-GPU host logic on CPU: two gloo ranks, oracle arithmetic instead of kernels."""
import os

import numpy as np
import pytest

import cpu_checkers as cc
from mshadow_b200 import sharding

torch = pytest.importorskip("torch")


def test_shard_range_covers_everything():
    for n in (0, 1, 7, 256, 1000):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1


def _worker(rank, world, port, tmpdir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    orc = cc.load("orc")
    rng = np.random.default_rng(77)  # same data on every rank
    T = rng.standard_normal((10, 6, 5, 8)).astype(np.float32)
    full = orc.reduce_keep_highdim(np.zeros(6, np.float32), T)
    b, e = sharding.shard_range(T.shape[0], rank, world)
    part = orc.reduce_keep_highdim(np.zeros(6, np.float32), np.ascontiguousarray(T[b:e]))
    total = sharding.allreduce_sum(torch.from_numpy(part.copy())).numpy()
    ok_red = bool(np.allclose(total, full, rtol=1e-5, atol=1e-5 * np.sqrt(np.mean(full ** 2))))
    # the peer-store exchange: every rank gathers all partial vectors and adds them in rank order,
    # so the ranks agree bit for bit and stay within tolerance of the unsharded sum
    gathered = [torch.zeros(6) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(part))
    ordered = sharding.rank_order_sum([g.numpy() for g in gathered])
    theirs = [torch.zeros(6) for _ in range(world)]
    dist.all_gather(theirs, torch.from_numpy(ordered))
    ok_red = ok_red and all(np.array_equal(t.numpy().view(np.uint32), ordered.view(np.uint32)) for t in theirs)
    ok_red = ok_red and bool(np.allclose(ordered, full, rtol=1e-5, atol=1e-5 * np.sqrt(np.mean(full ** 2))))

    k, d, n = 23, 12, 400
    idx = rng.integers(0, k, n).astype(np.int32)
    src = rng.standard_normal((n, d)).astype(np.float32)
    t0 = rng.standard_normal((k, d)).astype(np.float32)
    keys, order = idx.copy(), np.arange(n, dtype=np.int32)
    orc.sort_by_key(keys, order, True)
    want = orc.addtakegrad_largebatch(t0.copy(), keys, order, src)
    lk, lo, rb, re = sharding.route_sorted_indices(keys, order, k, rank, world)
    mine = np.ascontiguousarray(t0[rb:re]).copy()
    if lk.size:
        orc.addtakegrad_largebatch(mine, lk, lo, src)
    # routing keeps per-row order, so the owner's rows are bit-identical to the unsharded result
    ok_emb = bool(np.array_equal(mine.view(np.uint32), want[rb:re].view(np.uint32)))
    counts = torch.tensor([lk.size], dtype=torch.int64)
    dist.all_reduce(counts)
    ok_cnt = int(counts.item()) == n
    # cyclic ownership with replicated hot rows, on a skewed index list
    k, d, n = 40, 8, 3000
    p = (np.arange(k) + 1.0) ** -1.1
    idx = rng.choice(k, size=n, p=p / p.sum()).astype(np.int32)
    src = rng.standard_normal((n, d)).astype(np.float32)
    t0 = rng.standard_normal((k, d)).astype(np.float32)
    keys, order = idx.copy(), np.arange(n, dtype=np.int32)
    orc.sort_by_key(keys, order, True)
    want = orc.addtakegrad_largebatch(t0.copy(), keys, order, src)
    hot = sharding.hot_rows(keys, 4)
    tk, to, hk, ho = sharding.route_cyclic_with_hot_rows(keys, order, n, rank, world, hot)
    mine = np.ascontiguousarray(t0[rank::world]).copy()
    if tk.size:
        orc.addtakegrad_largebatch(mine, tk, to, src)
    partial = np.zeros((hot.size, d), np.float32)
    if hk.size:
        orc.addtakegrad_largebatch(partial, hk, ho, src)
    partial = sharding.allreduce_sum(torch.from_numpy(partial)).numpy()
    for i, r in enumerate(hot):
        if r % world == rank:
            mine[r // world] += partial[i]
    ref_rows = want[rank::world]
    cold = np.array([r not in set(hot.tolist()) for r in range(rank, k, world)])
    ok_cold = bool(np.array_equal(mine[cold].view(np.uint32), ref_rows[cold].view(np.uint32)))
    rms = np.sqrt(np.mean(ref_rows.astype(np.float64) ** 2, axis=1, keepdims=True))
    err = np.abs(mine.astype(np.float64) - ref_rows) / np.maximum(np.abs(ref_rows), rms)
    ok_hot = bool(err.max() <= 1e-5)
    load = torch.tensor([float(tk.size + hk.size)])
    total_load = load.clone()
    dist.all_reduce(total_load)
    peak = load.clone()
    dist.all_reduce(peak, op=dist.ReduceOp.MAX)
    # all entries are handled exactly once and no rank carries much more than its share
    ok_bal = int(total_load.item()) == n and peak.item() <= 0.6 * n
    with open(os.path.join(tmpdir, "rank%d.txt" % rank), "w") as f:
        f.write("%d %d %d %d %d %d" % (ok_red, ok_emb, ok_cnt, ok_cold, ok_hot, ok_bal))
    dist.destroy_process_group()


def test_two_ranks_reduce_and_route(tmp_path):
    import torch.multiprocessing as mp
    port = 29600 + os.getpid() % 300
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert open(tmp_path / ("rank%d.txt" % r)).read() == "1 1 1 1 1 1"


def test_hot_rows_balance_a_zipf_batch():
    """Contiguous row ownership leaves one rank with almost everything; cyclic ownership plus a
    handful of replicated hot rows brings every rank close to 1/world of the entries."""
    rng = np.random.default_rng(3)
    k, n, world = 262144, 1 << 18, 8
    p = (np.arange(k) + 1.0) ** -1.1
    keys = np.sort(rng.choice(k, size=n, p=p / p.sum()).astype(np.int32))
    order = rng.permutation(n).astype(np.int32)
    contiguous = [sharding.route_sorted_indices(keys, order, k, r, world)[0].size for r in range(world)]
    assert max(contiguous) > 0.8 * n
    hot = sharding.hot_rows(keys, 64)
    loads, seen = [], 0
    for r in range(world):
        tk, to, hk, ho = sharding.route_cyclic_with_hot_rows(keys, order, n, r, world, hot)
        assert np.all(np.diff(tk) >= 0) and np.all(np.diff(hk) >= 0)
        loads.append(tk.size + hk.size)
        seen += tk.size + hk.size
    assert seen == n
    assert max(loads) <= 1.1 * n / world
