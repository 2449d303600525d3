"""The multi-GPU synchronisation model (mshadow-ps interface over NCCL all-reduce).

Without a GPU: the library loads, exports what include/mshadow_b200_ps.h declares and validates
arguments.  With one GPU: a group of one process exercises the stream ordering, pitched tensors,
SetWeight / CheckWeight.  With two or more GPUs: two processes push different tensors and both
receive the sum (small integers, so the sum is exact), as guide/mshadow-ps/local_sum-inl.h of the
reference does with two devices in one process.
"""
import ctypes as C
import os
import time

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
