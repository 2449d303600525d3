"""The engine compiled with -DMSHADOW_B200_CHECK_BOUNDS=1 (tests/cxx/libmsb_bounds_suite.so).

In that build every access that a tensor leaf of an expression plan serves on the GPU is compared
with the extent of the tensor's storage; an access outside it is refused (a load reads zero, a
store is dropped) and recorded, and the kernel carries on.  The cases are user-written plans with
an index bug, the kind of mistake the build is for; nothing ever touches memory outside an
allocation, and the device stays usable afterwards.
"""
import ctypes as C
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PATH = os.path.join(ROOT, "tests", "cxx", "libmsb_bounds_suite.so")
ROWS, COLS = 6, 40


@pytest.fixture(scope="module")
def suite():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    assert os.path.exists(PATH), "tests/cxx/libmsb_bounds_suite.so is missing: run python -m mshadow_b200.build"
    dll = C.CDLL(PATH)
    dll.msb_bounds_suite_error.restype = C.c_char_p

    def call(cid, a, shift=0):
        out = np.zeros((ROWS, COLS), np.float32)
        rec = (C.c_longlong * 4)()
        f32p = C.POINTER(C.c_float)
        rc = dll.msb_bounds_suite_run(cid, a.ctypes.data_as(f32p), out.ctypes.data_as(f32p), ROWS, COLS, shift, rec)
        assert rc == 0, dll.msb_bounds_suite_error()
        return out, [int(v) for v in rec]

    return call


@pytest.fixture(scope="module")
def a():
    return np.random.default_rng(2).uniform(1, 2, (ROWS, COLS)).astype(np.float32)


def test_a_correct_expression_leaves_no_record(suite, a):
    out, rec = suite(0, a)
    assert rec[0] == 0
    assert np.array_equal(out, a + np.float32(1))


def test_reads_past_the_storage_are_refused_and_recorded(suite, a):
    shift = 7
    out, rec = suite(1, a, shift)
    hit, width, offset, limit = rec
    assert hit == 1 and width == 1 and limit == ROWS * COLS and offset >= limit
    flat = a.ravel()
    want = np.zeros(ROWS * COLS, np.float32)  # refused loads read zero
    want[:ROWS * COLS - shift] = flat[shift:]  # a shift inside the storage reads the neighbouring row
    assert np.array_equal(out.ravel(), want)


def test_stores_past_the_storage_are_dropped_and_recorded(suite, a):
    shift = 5
    out, rec = suite(2, a, shift)
    hit, width, offset, limit = rec
    assert hit == 1 and width == 1 and limit == ROWS * COLS and offset >= limit
    want = np.full(ROWS * COLS, -1, np.float32)  # the target's initial value where nothing was stored
    want[shift:] = a.ravel()[:ROWS * COLS - shift]
    assert np.array_equal(out.ravel(), want)


def test_the_device_stays_usable(suite, a):
    suite(1, a, 1000)  # every load of the last rows refused
    out, rec = suite(0, a)
    assert rec[0] == 0 and np.array_equal(out, a + np.float32(1))
