"""The allocation-free column sum (msb_reduce_keep_lowest_sum_f32_noalloc).

Some users of the library cannot let a call allocate device memory: they run while their
framework's memory pool is frozen, on a latency-critical path where cudaMalloc's implicit
synchronisation is not acceptable, or with all device memory already assigned.  For them the
library keeps a fixed 1 MiB scratch array in its own device image and offers this one extra
entry point.  The test calls it through the C ABI twice in a row on different data and
requires the same result as the regular entry point, msb_reduce_keep_lowest_f32, which
takes its scratch from a cudaMalloc'ed cache, and agreement with the CPU oracle.  The second
call matters: every call reuses the array, so a result that depended on left-over contents
would show up there.  Around that second call the free device memory and the library's own
scratch cache must not move: that is the property in the entry point's name.

The file name sorts last on purpose, so that a run stopped at the first failure has already
been through every other test.
"""
import numpy as np
import pytest

import cpu_checkers as cc

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

orc = cc.load("orc")


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import mshadow_b200
    L = mshadow_b200.load()
    L.init(0)
    return L


def scaled_err(got, want):
    want64 = want.astype(np.float64)
    scale = np.maximum(np.abs(want64), np.sqrt(np.mean(want64 ** 2)))
    return float(np.max(np.abs(got.astype(np.float64) - want64) / np.maximum(scale, 1e-30)))


# (rows, cols, extra elements per row, offset of the first element in floats)
#   20000 x 4096  128-bit path, several clusters per column tile: partial rows go through the array
#   3000 x 261    element-at-a-time path with several clusters (odd width)
#   3000 x 260    128-bit path
#   2000 x 256 with rows 260 apart, and the same starting one float past a 16-byte boundary
#   65 x 33       one cluster: nothing is parked
CASES = [(20000, 4096, 0, 0), (3000, 261, 0, 0), (3000, 260, 0, 0), (2000, 256, 4, 0), (2000, 256, 4, 1), (65, 33, 0, 0)]


@pytest.mark.parametrize("rows,cols,pad,offset", CASES)
def test_two_calls_match_the_allocating_entry_point_and_allocate_nothing(lib, rows, cols, pad, offset):
    g = torch.Generator(device="cuda")
    g.manual_seed(rows + cols + pad + offset)
    for call in range(2):
        # different data and scale on the second call: nothing may carry over in the scratch
        store = torch.randn(rows * (cols + pad) + 8, device="cuda", generator=g) * (1.0 + 3.0 * call)
        src = store[offset:offset + rows * (cols + pad)].view(rows, cols + pad)[:, :cols]
        scale = 0.5 + call
        want = lib.reduce_keep_lowest(torch.zeros(cols, device="cuda"), src, scale=scale, saver=0, reducer=0)
        got = torch.full((cols,), -1.0, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        held_before = lib.scratch_bytes(None)
        lib.reduce_keep_lowest_sum_noalloc(got, src, scale=scale)
        lib.stream_wait(None)
        # the library's scratch cache never moves; on the second call (the first one may make the
        # driver load the kernels' code, which takes device memory of its own) neither does the
        # driver's count of free memory
        assert lib.scratch_bytes(None) == held_before
        if call == 1:
            assert torch.cuda.mem_get_info()[0] == free_before
        w, o = want.cpu().numpy(), got.cpu().numpy()
        # the two entry points share kernels and launch geometry: identical results
        assert scaled_err(o, w) <= 1e-5
        assert np.array_equal(o.view(np.uint32), w.view(np.uint32))
        # and agree with the CPU: with a binary64 column sum always, with the oracle's binary32
        # left-to-right sum where that sum's own rounding stays below the tolerance (few rows)
        host = np.ascontiguousarray(src.cpu().numpy())
        exact = (host.sum(axis=0, dtype=np.float64) * np.float64(np.float32(scale))).astype(np.float32)
        assert scaled_err(o, exact) <= 1e-5
        if rows <= 4096:
            assert scaled_err(o, orc.reduce_keep_lowest(np.zeros(cols, np.float32), host, scale=scale)) <= 1e-5


def test_oversized_input_is_rejected_without_launching(lib):
    import ctypes as C
    # a matrix so wide that one partial row per cluster no longer fits the 1 MiB array.  How many
    # clusters a shape gets depends on the SM count, so the width is taken large enough for any
    # split into two or more clusters: 2 * cols floats > 1 MiB.
    rows, cols = 2100, 151040
    src = torch.zeros(rows, cols, device="cuda")
    dst = torch.full((cols,), 5.0, device="cuda")
    st, msg = lib.status("msb_reduce_keep_lowest_sum_f32_noalloc", C.c_void_p(dst.data_ptr()),
                         C.c_void_p(src.data_ptr()), rows, cols, cols, C.c_float(1.0), None)
    torch.cuda.synchronize()
    if st == 0:
        # a device on which this shape is covered by one cluster per column tile: nothing to refuse
        pytest.skip("the launch plan of this device parks no partial rows for the shape")
    assert st == 2 and "1 MiB" in msg
    assert bool((dst == 5.0).all())
