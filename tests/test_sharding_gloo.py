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
    total = sharding.allreduce_sum(torch.from_numpy(part)).numpy()
    ok_red = bool(np.allclose(total, full, rtol=1e-5, atol=1e-5 * np.sqrt(np.mean(full ** 2))))

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
    with open(os.path.join(tmpdir, "rank%d.txt" % rank), "w") as f:
        f.write("%d %d %d" % (ok_red, ok_emb, ok_cnt))
    dist.destroy_process_group()


def test_two_ranks_reduce_and_route(tmp_path):
    import torch.multiprocessing as mp
    port = 29600 + os.getpid() % 300
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert open(tmp_path / ("rank%d.txt" % r)).read() == "1 1 1"
