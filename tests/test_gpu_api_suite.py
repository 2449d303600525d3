"""The header-level C++ API, exercised by tests/cxx/api_suite.cu the way user code of the
reference is written (Tensor / TensorContainer / NewTensor / Copy / Slice / expressions /
reductions over expressions / user functors / type casts / double precision), checked here
against numpy restatements in fp32.  Element-wise results must be bit-exact, sums within 1e-5.
"""
import ctypes as C
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

SUITE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cxx", "libmsb_api_suite.so")
ROWS, COLS = 12, 100  # 100 columns: pitched by AllocSpace; 12 rows: divisible by 2, 3


@pytest.fixture(scope="module")
def run():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    assert os.path.exists(SUITE), "tests/cxx/libmsb_api_suite.so missing: run the build"
    dll = C.CDLL(SUITE)
    fp = C.POINTER(C.c_float)
    dll.msb_api_suite_run.argtypes = [C.c_int, fp, fp, fp, C.c_int, C.c_int]

    def call(cid, a, b, out_size, rows=ROWS, cols=COLS):
        out = np.full(out_size, np.nan, np.float32)
        rc = dll.msb_api_suite_run(cid, a.ctypes.data_as(fp), b.ctypes.data_as(fp), out.ctypes.data_as(fp), rows, cols)
        return rc, out
    return call


@pytest.fixture(scope="module")
def data():
    rng = np.random.default_rng(11)
    a = rng.uniform(-1, 1, (ROWS, COLS)).astype(np.float32)
    b = rng.uniform(-1, 1, (ROWS, COLS)).astype(np.float32)
    return a, b


def bits_equal(x, y):
    return np.array_equal(np.ascontiguousarray(x).view(np.uint32), np.ascontiguousarray(y).view(np.uint32))


def sums_close(got, want):
    scale = np.maximum(np.abs(want), np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    return np.max(np.abs(got.astype(np.float64) - want) / scale) <= 1e-5


def test_containers_pitch_and_scalars(run, data):
    a, b = data
    rc, out = run(0, a, b, ROWS * COLS + 1)
    assert rc == 0
    assert bits_equal(out[:-1].reshape(ROWS, COLS), a + b * np.float32(2))
    assert out[-1] >= COLS and int(out[-1]) % 4 == 0  # rows were pitched by AllocSpace


def test_sum_rows_scaled_and_accumulated(run, data):
    a, b = data
    rc, out = run(1, a, b, COLS)
    assert rc == 0
    assert sums_close(out, np.float32(0.5) * a.sum(0, dtype=np.float64) + b.sum(0, dtype=np.float64))


def test_sumall_except_dim0_of_3d(run, data):
    a, b = data
    rc, out = run(2, a, b, 3)
    assert rc == 0
    assert sums_close(out, a.reshape(3, -1).sum(1, dtype=np.float64))


def test_reduction_over_expression_plusto(run, data):
    a, b = data
    rc, out = run(3, a, b, ROWS // 2)
    assert rc == 0
    prod = (a * b).reshape(2, ROWS // 2, 2, COLS // 2)
    assert sums_close(out, 1.0 + prod.sum(axis=(0, 2, 3), dtype=np.float64))


def test_transpose(run, data):
    a, b = data
    rc, out = run(4, a, b, ROWS * COLS)
    assert rc == 0 and bits_equal(out.reshape(COLS, ROWS), a.T + np.float32(1))


def test_typecast_chain(run, data):
    a, b = data
    rc, out = run(5, a, b, ROWS * COLS)
    want = ((a * np.float32(10)).astype(np.int32) + 3).astype(np.float32)
    assert rc == 0 and bits_equal(out.reshape(ROWS, COLS), want)


def test_slice_and_row_index(run, data):
    a, b = data
    rc, out = run(6, a, b, ROWS * COLS)
    want = np.full((ROWS, COLS), -1, np.float32)
    want[1:-1] = a[1:-1] + b[0]
    assert rc == 0 and bits_equal(out.reshape(ROWS, COLS), want)


def test_reduce_except_dim_maximum(run, data):
    a, b = data
    rc, out = run(7, a, b, COLS)
    assert rc == 0 and bits_equal(out, np.maximum(a, b).max(0))


def test_double_precision(run, data):
    a, b = data
    rc, out = run(8, a, b, ROWS * COLS)
    a64 = a.astype(np.float64)
    want = ((a64 * a64 + 0.25) / (a64 * 0.0 + 3.0)).astype(np.float32)
    assert rc == 0 and bits_equal(out.reshape(ROWS, COLS), want)


def test_in_place_user_functors(run, data):
    a, b = data
    rc, out = run(9, a, b, ROWS * COLS)
    t = (a + np.float32(1)) * (a + np.float32(1))
    want = np.float32(1) / (np.float32(1) + np.exp(-(t * np.float32(0.5)).astype(np.float64)).astype(np.float32))
    got = out.reshape(ROWS, COLS)
    ulp = np.abs(got.view(np.int32).astype(np.int64) - want.view(np.int32).astype(np.int64))
    assert rc == 0 and ulp.max() <= 1


def test_softmax_in_place_then_grad(run, data):
    a, b = data
    b = b.copy()
    b[:, 0] = np.arange(ROWS) % COLS
    rc, out = run(10, a, b, ROWS * COLS)
    e = np.exp(a.astype(np.float64) - a.max(1, keepdims=True))
    want = e / e.sum(1, keepdims=True)
    want[np.arange(ROWS), np.arange(ROWS)] -= 1.0
    assert rc == 0 and np.allclose(out.reshape(ROWS, COLS), want, rtol=1e-5, atol=1e-7)


def _pool_max(x, k=3, s=2):
    p = (x.shape[-1] - k) // s + 1
    out = np.full(x.shape[:-2] + (p, p), -np.inf, np.float32)
    for dy in range(k):
        for dx in range(k):
            out = np.maximum(out, x[..., dy:dy + s * p:s, dx:dx + s * p:s][..., :p, :p])
    return out


def test_pool_over_expression(run):
    rng = np.random.default_rng(5)
    side, imgs = 9, 6
    a = rng.uniform(0, 1, (imgs, side, side)).astype(np.float32)
    rc, out = run(11, a, a, imgs * 4 * 4, rows=imgs, cols=side)
    assert rc == 0 and bits_equal(out.reshape(imgs, 4, 4), _pool_max(a * np.float32(2)))


def test_pool_unpool_chpool_chain(run):
    import cpu_checkers as cc
    orc = cc.load("orc")
    rng = np.random.default_rng(6)
    side, imgs = 9, 6
    a = (rng.integers(0, 5, (imgs, side, side)) / 4.0).astype(np.float32)
    rc, out = run(12, a, a, imgs * side * side, rows=imgs, cols=side)
    p = orc.pool(np.zeros((imgs, 4, 4), np.float32), a, 3, 3, 2, 2, reducer=1)
    g = orc.unpool(np.zeros_like(a), a, p, p, 3, 3, 2, 2, reducer=1)
    want = orc.chpool(np.zeros((2, imgs // 2, side, side), np.float32), g.reshape(2, imgs // 2, side, side), 3)
    assert rc == 0 and bits_equal(out.reshape(want.shape), want)


def test_shape_mismatch_raises(run, data):
    a, b = data
    rc, _ = run(13, a, b, 1)
    assert rc == 100


def test_half_precision_expression(run, data):
    """binary16 tensors: numpy's float16 arithmetic rounds every operation to half, as the engine does."""
    a, b = data
    rc, out = run(14, a, b, ROWS * COLS)
    ah, bh = a.astype(np.float16), b.astype(np.float16)
    want = ah * bh + ah * np.float16(0.5) - bh / (ah * ah + np.float16(2.0))
    want = want + np.maximum(ah, bh)
    assert rc == 0
    assert np.array_equal(out.reshape(ROWS, COLS).astype(np.float16).view(np.uint16), want.view(np.uint16))


def test_half_casts_and_exact_reduction(run, data):
    a, b = data
    rc, out = run(15, a, b, ROWS * COLS + COLS)
    ah = a.astype(np.float16)
    assert rc == 0
    assert bits_equal(out[:ROWS * COLS].reshape(ROWS, COLS), ah.astype(np.float32) * np.float32(2))
    assert bits_equal(out[ROWS * COLS:], ah.max(axis=0).astype(np.float32))


def test_patch_columns_with_accumulating_savers(run, data):
    """unpack_patch2col / pack_col2patch on a 3-d image with +=, -= (the dedicated kernels take any saver),
    unit stride with a compile-time patch size and a strided 4 x 2 patch."""
    a, b = data
    rc, out = run(16, a, b, ROWS * COLS)
    shape = (1, 2, 24, ROWS * COLS // 48)
    img, g = a.reshape(shape), b.reshape(shape)
    import cpu_checkers as cc
    orc = cc.load("orc")
    m = np.float32(1) + orc.unpack_patch2col(img, 3, 3, 1, 1, 1, 1)
    g = g - orc.pack_col2patch(m, shape, 3, 3, 1, 1, 1, 1)
    m2 = orc.unpack_patch2col(img, 4, 2, 2, 1, 1, 1)
    g = g + orc.pack_col2patch(m2, shape, 4, 2, 2, 1, 1, 1)
    assert rc == 0 and bits_equal(out.reshape(shape), g)


def test_patch_columns_on_pitched_tensors(run):
    """Row pitch != width on the image and on the matrix; the runs are 16-byte aligned, so the matrix
    leaves the kernel in 16-byte groups."""
    import cpu_checkers as cc
    orc = cc.load("orc")
    rng = np.random.default_rng(21)
    shape = (1, 2, 12, 68)
    a, b = (rng.uniform(-1, 1, shape).astype(np.float32) for _ in range(2))
    rc, out = run(17, a, b, a.size + 1)
    assert rc == 0 and out[-1] == 3.0  # both the image and the matrix were pitched
    m = np.float32(1) + orc.unpack_patch2col(a, 3, 3, 1, 1, 1, 1)
    assert bits_equal(out[:-1].reshape(shape), b - orc.pack_col2patch(m, shape, 3, 3, 1, 1, 1, 1))


def test_patch_columns_in_double_precision(run):
    import cpu_checkers as cc
    orc = cc.load("orc")
    rng = np.random.default_rng(22)
    shape = (1, 2, 24, 26)
    a, b = (rng.uniform(-1, 1, shape).astype(np.float32) for _ in range(2))
    rc, out = run(18, a, b, a.size)
    want = b.astype(np.float64) + orc.pack_col2patch(orc.unpack_patch2col(a, 3, 3, 1, 1, 1, 1), shape, 3, 3, 1, 1, 1, 1)
    assert rc == 0
    np.testing.assert_allclose(out.reshape(shape), want, rtol=2e-6, atol=2e-6)
