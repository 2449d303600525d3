"""The multi-GPU synchronisation models (mshadow-ps interface): NCCL all-reduce, and direct
peer stores over NVLink for small tensors.

Without a GPU: the library loads, exports what include/mshadow_b200_ps.h declares and validates
arguments.  With one GPU: a group of one process exercises the stream ordering, pitched tensors,
SetWeight / CheckWeight.  With two or more GPUs: two processes push different tensors and both
receive the sum (small integers, so the sum is exact), as guide/mshadow-ps/local_sum-inl.h of the
reference does with two devices in one process.
"""
import ctypes as C
import os
import time

import numpy as np
import pytest

from mshadow_b200 import ps

torch = pytest.importorskip("torch")


def test_ps_library_exports_every_declared_symbol():
    assert os.path.exists(ps.LIB_PATH), "build the library first (python -m mshadow_b200.build)"
    names = ps.declared_symbols()
    for required in ["msb_ps_create", "msb_ps_init_key", "msb_ps_push", "msb_ps_pull_req", "msb_ps_pull_wait",
                     "msb_ps_set_weight", "msb_ps_check_weight", "msb_ps_new_unique_id", "msb_ps_last_error"]:
        assert required in names
    dll = C.CDLL(ps.LIB_PATH)
    assert not [n for n in names if not hasattr(dll, n)]
    assert set(names) <= set(ps._SIGNATURES) | {"msb_ps_last_error"}


def test_ps_argument_errors_need_no_gpu():
    with pytest.raises(ps.PsError, match="rank outside"):
        ps.SharedModel(rank=2, world=2, unique_id="00" * 128)
    with pytest.raises(ps.PsError, match="identifier"):
        ps.SharedModel(rank=0, world=2, unique_id=None)
    buf = C.create_string_buffer(8)
    assert ps.dll().msb_ps_new_unique_id(buf, 8) != 0
    assert ps.dll().msb_ps_pull_wait(None, 0) != 0
    with pytest.raises(ps.PsError, match="rank outside"):
        ps.PeerModel(rank=3, world=2)
    assert ps.dll().msb_ps_peer_handle(None, buf, 8) != 0
    assert ps.dll().msb_ps_peer_connect(None, b"00") != 0


@pytest.mark.gpu
def test_single_process_group_orders_streams_and_handles_pitch():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    m = ps.SharedModel(rank=0, world=1, device=0)
    try:
        m.init_key(0, (6, 10))
        m.init_key(1, (3, 4, 8))
        a = torch.arange(60, dtype=torch.float32, device="cuda").reshape(6, 10)
        wide = torch.full((6, 16), -1.0, device="cuda")
        pitched = wide[:, :10]
        pitched.copy_(a * 2)
        m.push(a, 0)
        out = torch.zeros(6, 10, device="cuda")
        m.pull_req(out, 0)
        m.pull_wait(0)
        assert torch.equal(out, a)
        m.push(pitched, 0)           # rows 16 floats apart: packed before the all-reduce
        m.pull_req(pitched, 0)       # and scattered back with the pitch
        m.pull_wait(0)
        assert torch.equal(pitched, a * 2) and bool((wide[:, 10:] == -1.0).all())
        t = torch.randn(3, 4, 8, device="cuda")
        m.push(t, 1)
        m.pull_req(t, 1)
        m.pull_wait(1)
        m.set_weight(t, 1)
        m.check_weight(t, 1)
        with pytest.raises(ps.PsError, match="shape differs"):
            m.push(a, 1)
        with pytest.raises(ps.PsError, match="not been initialised"):
            m.push(a, 7)
    finally:
        m.close()


def _worker(rank, world, id_file, out_dir):
    torch.cuda.set_device(rank)
    if rank == 0:
        uid = ps.new_unique_id()
        with open(id_file + ".tmp", "w") as f:
            f.write(uid)
        os.replace(id_file + ".tmp", id_file)
    else:
        deadline = time.time() + 120
        while not os.path.exists(id_file):
            if time.time() > deadline:
                raise RuntimeError("no identifier from rank 0")
            time.sleep(0.05)
        uid = open(id_file).read()
    m = ps.SharedModel(rank=rank, world=world, unique_id=uid, device=rank)
    ok = True
    m.init_key(0, (2, 3))
    m.init_key(1, (257, 130))
    small = torch.ones(2, 3, device="cuda")
    small[1] += rank                       # rows: 1, 1 + rank  (the reference example's data)
    big = (torch.arange(257 * 130, device="cuda") % 17).float().reshape(257, 130) * (rank + 1)
    for _ in range(3):                     # repeated rounds reuse the buffers and events
        a, b = small.clone(), big.clone()
        m.push(a, 0)
        m.pull_req(a, 0)
        m.push(b, 1)
        m.pull_req(b, 1)
        m.pull_wait(0)
        m.pull_wait(1)
        want_small = torch.ones(2, 3, device="cuda") * world
        want_small[1] += sum(range(world))
        want_big = (torch.arange(257 * 130, device="cuda") % 17).float().reshape(257, 130) * sum(
            r + 1 for r in range(world))
        ok = ok and torch.equal(a, want_small) and torch.equal(b, want_big)
    w = torch.full((2, 3), float(rank + 5), device="cuda")
    m.set_weight(w, 0)
    ok = ok and bool((w == 5.0).all())
    m.check_weight(w, 0)
    diverged = w + rank                    # differs from rank 0 everywhere but on rank 0
    try:
        m.check_weight(diverged, 0)
        caught = False
    except ps.PsError:
        caught = True
    ok = ok and (caught == (rank != 0))
    m.close()
    with open(os.path.join(out_dir, "rank%d.txt" % rank), "w") as f:
        f.write("1" if ok else "0")


@pytest.mark.gpu
def test_two_processes_sum_over_nvlink(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, str(tmp_path / "nccl_id"), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / ("rank%d.txt" % r)).read() == "1"


# ---- the peer-store model --------------------------------------------------------------------
@pytest.mark.gpu
def test_peer_model_alone_on_one_gpu_runs_its_kernels_and_slot_rotation():
    """A group of one: the contribution goes through the window of this GPU (push kernel, tagged
    words, pull kernel), step after step, so slots are reused several times; the sum of one is the
    data.  Then the same with reduction kernels delivering their results through sinks."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    m = ps.PeerModel(rank=0, world=1, device=0, depth=4)
    try:
        m.init_key(0, (4608,))
        m.init_key(1, (7, 33))            # odd sizes: element-wise path
        m.init_key(2, (64, 1024))         # many CTAs
        g = torch.Generator(device="cuda")
        g.manual_seed(5)
        for step in range(11):
            a = torch.randn(4608, device="cuda", generator=g)
            out = torch.full((4608,), -7.0, device="cuda")
            m.push(a, 0)
            if step % 2:                  # one step pushed ahead of its pull is allowed with depth 4
                b = torch.randn(4608, device="cuda", generator=g)
                m.push(b, 0)
                m.pull_req(out, 0)
                m.pull_wait(0)
                assert torch.equal(out, a)
                m.pull_req(out, 0)
                m.pull_wait(0)
                assert torch.equal(out, b)
            else:
                m.pull_req(out, 0)
                m.pull_wait(0)
                assert torch.equal(out, a)
            wide = torch.full((7, 40), -1.0, device="cuda")
            view = wide[:, :33]
            c = torch.randn(7, 33, device="cuda", generator=g)
            view.copy_(c)
            m.push(view, 1)               # rows 40 floats apart
            m.pull_req(view, 1)
            m.pull_wait(1)
            assert torch.equal(view, c) and bool((wide[:, 33:] == -1.0).all())
            d = torch.randn(64, 1024, device="cuda", generator=g)
            o2 = torch.zeros_like(d)
            m.push(d, 2)
            m.pull_req(o2, 2)
            m.pull_wait(2)
            assert torch.equal(o2, d)
        # reductions that deliver their own results: a column sum large enough to need the finishing
        # kernel, a small one that does not, and a channel sum, as segments of one row
        import mshadow_b200
        lib = mshadow_b200.load()
        lib.init(0)
        m.init_key(3, (2048 + 48 + 24,))
        for step in range(3):
            big = torch.randn(30000, 2048, device="cuda", generator=g)
            small = torch.randn(77, 48, device="cuda", generator=g)
            img = torch.randn(5, 24, 6, 10, device="cuda", generator=g)
            d1, d2, d3 = (torch.zeros(k, device="cuda") for k in (2048, 48, 24))
            lib.reduce_keep_lowest(d1, big, scale=0.5, sink=m.next_sink(3, 0, 2048))
            lib.reduce_keep_lowest(d2, small, sink=m.next_sink(3, 2048, 48))
            lib.reduce_keep_highdim(d3, img, scale=2.0, saver=1, sink=m.next_sink(3, 2048 + 48, 24))
            got = torch.zeros(2048 + 48 + 24, device="cuda")
            m.pull_req(got, 3)
            m.pull_wait(3)
            # d3 was accumulated into (saver plusto) zeros, so it equals what was delivered
            assert torch.equal(got, torch.cat([d1, d2, d3]))
        with pytest.raises(mshadow_b200.MsbError, match="different number"):
            lib.reduce_keep_lowest(d1, big, sink=m.next_sink(3, 2048, 48))   # a segment that opens no step
        w = torch.randn(7, 33, device="cuda", generator=g)
        keep = w.clone()
        m.set_weight(w, 1)
        m.check_weight(w, 1)
        assert torch.equal(w, keep)
        with pytest.raises(ps.PsError, match="shape differs"):
            m.push(w, 0)
        with pytest.raises(ps.PsError, match="nothing pushed"):
            m.pull_req(torch.zeros(4608, device="cuda"), 0)
        m.push(torch.zeros(4608, device="cuda"), 0)
        m.push(torch.zeros(4608, device="cuda"), 0)
        with pytest.raises(ps.PsError, match="too many steps"):
            m.push(torch.zeros(4608, device="cuda"), 0)
    finally:
        torch.cuda.synchronize()
        m.close()


@pytest.mark.gpu
def test_peer_model_raw_regions():
    """Regions of the window for the caller's own kernels: offsets follow the keys, are 256-byte
    aligned and reproducible; addresses are base + offset; a region beyond the window is refused."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    m = ps.PeerModel(rank=0, world=1, device=0, window_bytes=1 << 20)
    try:
        m.init_key(0, (100,))
        a = m.reserve(1000)
        b = m.reserve(4096)
        assert a % 256 == 0 and b % 256 == 0 and b >= a + 1000
        base = m.window(0, 0)
        assert m.window(0, a) == base + a and m.window(0, b) == base + b
        x = torch.arange(256, dtype=torch.float32, device="cuda")
        import mshadow_b200
        lib = mshadow_b200.load()
        lib.init(0)
        lib.copy_2d(m.window(0, b), 256, x, 256, 1, 256, mshadow_b200.capi.D2D)
        y = torch.zeros(256, device="cuda")
        lib.copy_2d(y, 256, m.window(0, b), 256, 1, 256, mshadow_b200.capi.D2D)
        assert torch.equal(x, y)
        with pytest.raises(ps.PsError):
            m.reserve(2 << 20)
        with pytest.raises(ps.PsError):
            m.window(1, 0)
    finally:
        m.close()


@pytest.mark.gpu
def test_peer_model_pull_gives_up_when_a_peer_never_answers():
    """A group of two whose second member does not exist: both handles name this rank's window, so
    the flag of rank 1 is never set.  The pull kernel polls for the configured 30 ms, leaves the
    destination alone and records a status; pull_wait reports it; the GPU carries on."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    m = ps.PeerModel(rank=0, world=2, device=0, wait_limit_ms=30)
    try:
        h = m.export_handle()
        assert len(h) == 128
        m.connect([h, h])
        m.init_key(0, (512,))
        a = torch.ones(512, device="cuda")
        out = torch.full((512,), 3.0, device="cuda")
        m.push(a, 0)
        m.pull_req(out, 0)
        t0 = time.time()
        with pytest.raises(ps.PsError, match="timeout"):
            m.pull_wait(0)
        assert time.time() - t0 < 5.0
        assert bool((out == 3.0).all())
        m.pull_wait(0)                    # the mark is cleared once reported
        assert float((a + 1).sum().item()) == 1024.0
    finally:
        torch.cuda.synchronize()
        m.close()


def _exchange_handles(rank, world, handle, tmp):
    with open(os.path.join(tmp, "h%d.tmp" % rank), "w") as f:
        f.write(handle)
    os.replace(os.path.join(tmp, "h%d.tmp" % rank), os.path.join(tmp, "h%d" % rank))
    deadline = time.time() + 120
    out = []
    for r in range(world):
        path = os.path.join(tmp, "h%d" % r)
        while not os.path.exists(path):
            if time.time() > deadline:
                raise RuntimeError("no handle from rank %d" % r)
            time.sleep(0.02)
        out.append(open(path).read())
    return out


def _file_barrier(rank, world, tmp, name):
    open(os.path.join(tmp, "%s.%d" % (name, rank)), "w").close()
    deadline = time.time() + 120
    while not all(os.path.exists(os.path.join(tmp, "%s.%d" % (name, r))) for r in range(world)):
        if time.time() > deadline:
            raise RuntimeError("barrier %s" % name)
        time.sleep(0.02)


def _peer_worker(rank, world, tmp):
    from mshadow_b200 import sharding
    torch.cuda.set_device(rank)
    m = ps.PeerModel(rank=rank, world=world, device=rank, depth=4, wait_limit_ms=20000)
    m.connect(_exchange_handles(rank, world, m.export_handle(), tmp))
    m.init_key(0, (4608,))
    m.init_key(1, (64, 1024))
    ok = True

    def data(r, step, shape):
        g = torch.Generator()
        g.manual_seed(1000 * step + r)
        return torch.randn(shape, generator=g)

    def want(step, shape):
        return torch.from_numpy(sharding.rank_order_sum([data(r, step, shape).numpy() for r in range(world)]))

    # steady state of a training loop: push step s + 1, then pull step s; ranks drift apart on purpose
    steps = 40
    outs = []
    mine = [data(rank, s, (4608,)).cuda() for s in range(steps)]
    m.push(mine[0], 0)
    for s in range(steps):
        if (s + rank) % 3 == 0:
            torch.cuda._sleep(2000000)   # about a millisecond of delay on this rank's stream
        if s + 1 < steps:
            m.push(mine[s + 1], 0)
        out = torch.zeros(4608, device="cuda")
        m.pull_req(out, 0)
        outs.append(out)
    m.pull_wait(0)
    for s in range(steps):
        ok = ok and torch.equal(outs[s].cpu(), want(s, (4608,)))
    # a larger tensor (several CTAs per peer), push and pull in turn
    for s in range(6):
        big = data(rank, 100 + s, (64, 1024)).cuda()
        m.push(big, 1)
        m.pull_req(big, 1)
        m.pull_wait(1)
        ok = ok and torch.equal(big.cpu(), want(100 + s, (64, 1024)))
    # reductions delivering their results themselves: every rank sums its own matrix, all receive
    # the rank-order sum of the per-rank column sums
    import mshadow_b200
    lib = mshadow_b200.load()
    lib.init(rank)
    for s in range(4):
        mat = data(rank, 200 + s, (9000, 4608)).cuda()
        mine_sum = torch.zeros(4608, device="cuda")
        lib.reduce_keep_lowest(mine_sum, mat, sink=m.next_sink(0, 0, 4608))
        got = torch.zeros(4608, device="cuda")
        m.pull_req(got, 0)
        m.pull_wait(0)
        parts = []
        for r in range(world):
            other = torch.zeros(4608, device="cuda")
            lib.reduce_keep_lowest(other, data(r, 200 + s, (9000, 4608)).cuda())
            parts.append(other.cpu().numpy())
        ok = ok and torch.equal(got.cpu(), torch.from_numpy(sharding.rank_order_sum(parts)))
    # raw regions: every rank's segmented sum stores the sums of its runs straight into the owner's
    # window (row t of the table lives on rank t % world), the row numbers beside them, and a small
    # key pushed afterwards carries the counts and tells the owner that the rows have arrived
    table_rows, d, n_loc = 500, 64, 3000
    kp = (table_rows + world - 1) // world
    m.init_key(2, (world * world,))
    off_rows, off_keys = m.reserve(world * kp * d * 4), m.reserve(world * kp * 4)

    def batch(r):
        rng = np.random.default_rng(77 + r)
        p = (np.arange(table_rows) + 1.0) ** -1.1
        return (rng.choice(table_rows, size=n_loc, p=p / p.sum()).astype(np.int32),
                rng.standard_normal((n_loc, d)).astype(np.float32))

    idx, src = batch(rank)
    ck = torch.from_numpy(((idx % world) * kp + idx // world).astype(np.int32)).cuda()
    pos = torch.arange(n_loc, dtype=torch.int32, device="cuda")
    lib.sort_by_key(ck, pos, bits=int(world * kp - 1).bit_length())
    run_of, run_keys = torch.empty_like(pos), torch.empty_like(pos)
    total = torch.zeros(1, dtype=torch.int32, device="cuda")
    first = torch.zeros(world + 1, dtype=torch.int32, device="cuda")
    lib.run_index(run_of, run_keys, total, ck)
    lib.run_bounds(first, run_keys, total, world, kp)
    lib.take_sum_to_owners([m.window(q, off_rows) + rank * kp * d * 4 for q in range(world)], first, run_of, pos,
                           torch.from_numpy(src).cuda(), world)
    lib.run_keys_to_owners([m.window(q, off_keys) + rank * kp * 4 for q in range(world)], first, run_keys, world, kp)
    counts_mine = torch.zeros(world * world, device="cuda")
    counts_mine[rank * world:(rank + 1) * world] = (first[1:] - first[:-1]).float()
    counts = torch.zeros(world * world, device="cuda")
    m.push(counts_mine, 2)
    m.pull_req(counts, 2)
    m.pull_wait(2)
    got_counts = counts.view(world, world)[:, rank].cpu().numpy().astype(np.int64)
    rows_in = torch.empty(world * kp, d, device="cuda")
    keys_in = torch.empty(world * kp, dtype=torch.int32, device="cuda")
    lib.copy_2d(rows_in, d, m.window(rank, off_rows), d, world * kp, d, mshadow_b200.capi.D2D)
    lib.copy_2d(keys_in, world * kp, m.window(rank, off_keys), world * kp, 1, world * kp, mshadow_b200.capi.D2D)
    rows_in, keys_in = rows_in.cpu().numpy(), keys_in.cpu().numpy()
    for r in range(world):
        ridx, rsrc = batch(r)
        to_me = np.unique(ridx[ridx % world == rank])
        ok = ok and int(got_counts[r]) == to_me.size
        ok = ok and np.array_equal(keys_in[r * kp:r * kp + to_me.size], (to_me // world).astype(np.int32))
        for j, t in enumerate(to_me):
            want_row = rsrc[ridx == t].astype(np.float64).sum(axis=0)
            err = np.abs(rows_in[r * kp + j] - want_row).max() / max(1e-30, np.abs(want_row).max())
            ok = ok and err <= 1e-5
    w = torch.full((64, 1024), float(rank + 5), device="cuda")
    m.set_weight(w, 1)
    ok = ok and bool((w == 5.0).all())
    m.check_weight(w, 1)
    try:
        m.check_weight(w + rank, 1)
        caught = False
    except ps.PsError:
        caught = True
    ok = ok and (caught == (rank != 0))
    torch.cuda.synchronize()
    _file_barrier(rank, world, tmp, "done")   # nobody frees a window that a peer may still write
    m.close()
    with open(os.path.join(tmp, "rank%d.txt" % rank), "w") as f:
        f.write("1" if ok else "0")


@pytest.mark.gpu
def test_two_processes_exchange_by_peer_stores(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_peer_worker, args=(world, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / ("rank%d.txt" % r)).read() == "1"
