"""The engine's headers on Tensor<cpu>, compiled by g++ alone, against the CPU oracle.

An expression plan's Eval(y, x) is the same code on the host and in the element-at-a-time GPU
kernel, so the index arithmetic of the index-remapping plans (reciprocal division included) is
checked here without a GPU.  tests/cxx/libmsb_host_suite.so is built by mshadow_b200/build.py.
"""
import ctypes as C
import os

import numpy as np
import pytest

import cpu_checkers as cc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PATH = os.path.join(ROOT, "tests", "cxx", "libmsb_host_suite.so")
orc = cc.load("orc")
i64 = C.c_int64
f32p = C.POINTER(C.c_float)


@pytest.fixture(scope="module")
def host():
    if not os.path.exists(PATH):
        import mshadow_b200.build as b
        b.build_all(verbose=False)
    dll = C.CDLL(PATH)
    dll.hostmsb_last_error.restype = C.c_char_p
    return dll


def run(dll, cid, A, B, p0, p1, fill=9.0):
    n, c, h, w = A.shape
    shape = (i64 * 4)()
    assert dll.hostmsb_remap_case(cid, None, None, None, i64(n), i64(c), i64(h), i64(w), i64(p0), i64(p1), shape) == 0
    dst = np.full(tuple(int(v) for v in shape), np.float32(fill), np.float32)
    st = dll.hostmsb_remap_case(cid, dst.ctypes.data_as(f32p), A.ctypes.data_as(f32p), B.ctypes.data_as(f32p), i64(n),
                                i64(c), i64(h), i64(w), i64(p0), i64(p1), shape)
    assert st == 0, dll.hostmsb_last_error()
    return dst


@pytest.mark.parametrize("cid", range(cc.NUM_REMAP_CASES))
@pytest.mark.parametrize("shape", [(2, 3, 4, 5), (1, 8, 6, 16), (3, 5, 1, 7), (2, 2, 3, 1), (2, 7, 9, 12)])
def test_remap_plans_on_the_host(host, cid, shape):
    rng = np.random.default_rng(cid * 100 + sum(shape))
    A = rng.uniform(-1, 1, shape).astype(np.float32)
    B = rng.uniform(-1, 1, shape).astype(np.float32)
    for p0, p1 in cc.remap_params(cid, shape):
        want = orc.remap_case(cid, A, B, p0, p1, fill=9.0)
        got = run(host, cid, A, B, p0, p1)
        assert got.shape == want.shape
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (cid, p0, p1)


def test_expression_checks_fire_on_the_host(host):
    A = np.zeros((2, 3, 4, 5), np.float32)
    shape = (i64 * 4)()
    assert host.hostmsb_remap_case(1, None, None, None, i64(2), i64(3), i64(4), i64(5), i64(2), i64(9), shape) == 1
    assert b"slice" in host.hostmsb_last_error().lower()
    assert host.hostmsb_remap_case(10, None, None, None, i64(2), i64(3), i64(4), i64(5), i64(7), i64(2), shape) == 1
    assert b"height" in host.hostmsb_last_error()
    del A


def test_half_conversions_match_ieee_binary16(host):
    """half_t's host conversions against numpy's float16: every bit pattern one way, a dense
    sample of floats (ties, subnormals, overflow, signed zeros) the other way."""
    u16p = C.POINTER(C.c_uint16)
    bits = np.arange(65536, dtype=np.uint16)
    as_float = np.zeros(65536, np.float32)
    host.hostmsb_half_to_float(bits.ctypes.data_as(u16p), as_float.ctypes.data_as(f32p), i64(65536))
    want = bits.view(np.float16).astype(np.float32)
    finite = ~np.isnan(want)
    assert np.array_equal(as_float[finite].view(np.uint32), want[finite].view(np.uint32))
    assert np.isnan(as_float[~finite]).all()
    rng = np.random.default_rng(5)
    samples = [rng.uniform(-70000, 70000, 200000), rng.uniform(-1e-4, 1e-4, 200000), rng.standard_normal(200000),
               np.array([0.0, -0.0, 65504.0, 65519.99, 65520.0, 1e9, -1e9, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001,
                         2.0 ** -14, np.inf, -np.inf])]
    # every midpoint between neighbouring halves (the ties) and its float neighbours
    pos = np.arange(0, 0x7C00, dtype=np.uint16).view(np.float16).astype(np.float64)
    mid = ((pos[:-1] + pos[1:]) / 2).astype(np.float32)
    samples += [mid, np.nextafter(mid, np.float32(np.inf)), np.nextafter(mid, np.float32(-np.inf)), -mid]
    x = np.concatenate([np.asarray(s, dtype=np.float32) for s in samples])
    got = np.zeros(x.size, np.uint16)
    host.hostmsb_half_from_float(x.ctypes.data_as(f32p), got.ctypes.data_as(u16p), i64(x.size))
    with np.errstate(over="ignore"):
        want16 = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, want16)


def test_half_expression_on_the_host(host):
    u16p = C.POINTER(C.c_uint16)
    rng = np.random.default_rng(6)
    a = rng.uniform(-1, 1, (7, 33)).astype(np.float16)
    b = rng.uniform(-1, 1, (7, 33)).astype(np.float16)
    out = np.zeros((7, 33), np.uint16)
    host.hostmsb_half_expr(a.view(np.uint16).ctypes.data_as(u16p), b.view(np.uint16).ctypes.data_as(u16p),
                           out.ctypes.data_as(u16p), i64(7), i64(33))
    want = a * b + a * np.float16(0.5) - b / (a * a + np.float16(2.0))
    assert np.array_equal(out, want.view(np.uint16))


@pytest.mark.parametrize("cid", range(cc.NUM_SELECT_CASES))
@pytest.mark.parametrize("rows,cols", [(5, 7), (16, 64), (1, 1), (33, 12)])
def test_select_plans_on_the_host(host, cid, rows, cols):
    rng = np.random.default_rng(cid * 100 + rows + cols)
    A, B, ir, ic = cc.select_inputs(rng, rows, cols)
    for p0 in ((1, 2, 3) if cid == 5 else (1,)):
        want = orc.select_case(cid, A, B, ir, ic, p0)
        got = np.full(want.shape, np.float32(9.0), np.float32)
        st = host.hostmsb_select_case(cid, got.ctypes.data_as(f32p), A.ctypes.data_as(f32p), B.ctypes.data_as(f32p),
                                      ir.ctypes.data_as(f32p), ic.ctypes.data_as(f32p), i64(rows), i64(cols), i64(p0))
        assert st == 0, host.hostmsb_last_error()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (cid, p0)


def run_axis(dll, cid, A, p0, p1):
    n, c, h, w = A.shape
    shape, ndim = (i64 * 4)(), C.c_int(0)
    dims = (i64(n), i64(c), i64(h), i64(w), i64(p0), i64(p1))
    st = dll.hostmsb_axis_case(cid, None, None, *dims, shape, C.byref(ndim))
    if st != 0:
        return st, None
    dst = np.full(tuple(int(v) for v in shape[:ndim.value]), np.float32(9.0), np.float32)
    st = dll.hostmsb_axis_case(cid, dst.ctypes.data_as(f32p), A.ctypes.data_as(f32p), *dims, shape, C.byref(ndim))
    return st, dst


@pytest.mark.parametrize("cid", range(cc.NUM_AXIS_CASES))
@pytest.mark.parametrize("shape", [(2, 3, 4, 5), (1, 8, 6, 16), (3, 5, 1, 7), (2, 2, 3, 1), (2, 7, 9, 12)])
def test_axis_plans_on_the_host(host, cid, shape):
    rng = np.random.default_rng(cid * 100 + sum(shape))
    A = rng.uniform(-1, 1, shape).astype(np.float32)
    if cid == 5:
        A[0, 0] = A[-1, -1]
    for p0, p1 in cc.axis_params(cid, shape):
        want = orc.axis_case(cid, A, p0, p1)
        st, got = run_axis(host, cid, A, p0, p1)
        assert st == 0, host.hostmsb_last_error()
        assert got.shape == want.shape
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (cid, p0, p1)


@pytest.mark.parametrize("cid", range(cc.NUM_COMPLEX_CASES))
@pytest.mark.parametrize("rows,cols", [(3, 4), (5, 16), (1, 8), (7, 36)])
def test_complex_plans_on_the_host(host, cid, rows, cols):
    rng = np.random.default_rng(cid * 100 + rows + cols)
    A = rng.uniform(-1, 1, (rows, cols)).astype(np.float32)
    B = rng.uniform(-1, 1, (rows, cols)).astype(np.float32)
    want = orc.complex_case(cid, A, B)
    got = np.full(want.shape, np.float32(9.0), np.float32)
    st = host.hostmsb_complex_case(cid, got.ctypes.data_as(f32p), A.ctypes.data_as(f32p), B.ctypes.data_as(f32p),
                                   i64(rows), i64(cols))
    assert st == 0, host.hostmsb_last_error()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), cid


def test_complex_shape_rules(host):
    z = np.zeros((2, 6), np.float32)
    p = z.ctypes.data_as(f32p)
    assert host.hostmsb_complex_case(0, p, p, p, i64(2), i64(6)) == 2  # cols not a multiple of 4
    assert host.hostmsb_complex_shape_error() == 1
    assert b"CR" in host.hostmsb_last_error()


def test_axis_arguments_outside_the_domain_are_refused(host):
    A = np.zeros((2, 3, 4, 5), np.float32)
    assert run_axis(host, 4, A, 4, 0)[0] == 2   # no such axis
    assert run_axis(host, 0, A, 0, 0)[0] == 2   # an empty range
    assert run_axis(host, 7, A, 0, 0)[0] == 2   # a broadcast extent of zero
    assert run_axis(host, 11, A, 0, 1)[0] == 2  # no such case


@pytest.mark.parametrize("case", cc.PATCH_CASES)
def test_patch_plans_on_the_host(host, case):
    shape, psy, psx, sy, sx, dy, dx = case
    n, c, h, w = shape
    rng = np.random.default_rng(sum(shape) + psy * 7 + sx)
    img = rng.uniform(-1, 1, shape).astype(np.float32)
    want = orc.unpack_patch2col(img, psy, psx, sy, sx, dy, dx)
    got = np.full(want.shape, np.float32(9.0), np.float32)
    args = (i64(n), i64(c), i64(h), i64(w), psy, psx, sy, sx, dy, dx)
    assert host.hostmsb_patch(0, got.ctypes.data_as(f32p), img.ctypes.data_as(f32p), *args) == 0
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    grad = rng.uniform(-1, 1, want.shape).astype(np.float32)
    want_img = orc.pack_col2patch(grad, shape, psy, psx, sy, sx, dy, dx)
    got_img = np.full(shape, np.float32(9.0), np.float32)
    assert host.hostmsb_patch(1, got_img.ctypes.data_as(f32p), grad.ctypes.data_as(f32p), *args) == 0
    assert np.array_equal(got_img.view(np.uint32), want_img.view(np.uint32))


def _numpy_remap(cid, A, B, p0, p1):
    """numpy's own formulation of the remap cases that have one (independent of the C oracle)."""
    n, c, h, w = A.shape
    if cid == 0:
        return A.reshape(n, h, c, w)
    if cid == 1:
        return A[:, p0:p1]
    if cid == 2:
        return A[..., p0:p1]
    if cid == 3:
        return np.concatenate([A, B], axis=1)
    if cid == 4:
        return np.concatenate([A, B], axis=3)
    if cid == 5:
        return A.swapaxes(1, 2)
    if cid == 6:
        return A.swapaxes(1, 3)
    if cid == 7:
        return A.transpose(0, 2, 1, 3)
    if cid == 8:
        return A.transpose(3, 1, 0, 2)
    if cid == 9:
        return np.pad(A, ((0, 0), (0, 0), (p0, p0), (p1, p1)))
    if cid == 12:
        return A[..., ::-1]
    if cid == 13:
        return A[:, ::-1]
    if cid == 16:
        return A + A[..., ::-1]
    return None


def test_remap_plans_against_numpy_on_random_shapes(host):
    hyp = pytest.importorskip("hypothesis")
    st = hyp.strategies

    @hyp.settings(max_examples=120, deadline=None)
    @hyp.given(st.integers(1, 4), st.integers(1, 9), st.integers(1, 9), st.integers(1, 20),
               st.sampled_from([0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 12, 13, 16]), st.integers(0, 3), st.integers(0, 5),
               st.integers(0, 2 ** 31 - 1))
    def check(n, c, h, w, cid, a, b, seed):
        rng = np.random.default_rng(seed)
        A = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float32)
        B = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float32)
        if cid == 1:
            p0 = a % c
            p1 = p0 + 1 + b % (c - p0)
        elif cid == 2:
            p0 = a % w
            p1 = p0 + 1 + b % (w - p0)
        else:
            p0, p1 = a, b
        want = np.ascontiguousarray(_numpy_remap(cid, A, B, p0, p1))
        got = run(host, cid, A, B, p0, p1)
        assert got.shape == want.shape
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))

    check()


def test_reciprocal_division_is_exact(host):
    """expr::FastDiv (multiply-high, add, shift) against / and % for every index below 2^31 that
    matters: small and large divisors, powers of two and their neighbours, multiples of the divisor
    and their neighbours, and random numbers."""
    rng = np.random.default_rng(11)
    divisors = np.unique(np.concatenate([
        np.arange(1, 2050), 2 ** np.arange(1, 31), 2 ** np.arange(2, 31) - 1, 2 ** np.arange(1, 31) + 1,
        np.array([3, 7, 54, 56, 641, 2916, 3136, 65521, 186624, 746496, 2 ** 31 - 1]),
        rng.integers(1, 2 ** 31, 2000)])).astype(np.uint32)
    numbers = np.concatenate([np.arange(0, 4100), 2 ** 31 - 1 - np.arange(0, 4100), 2 ** np.arange(0, 31),
                              2 ** np.arange(1, 31) - 1, rng.integers(0, 2 ** 31, 20000)]).astype(np.uint32)
    host.hostmsb_fastdiv_mismatches.restype = C.c_int64
    u32p = C.POINTER(C.c_uint32)
    bad = host.hostmsb_fastdiv_mismatches(divisors.ctypes.data_as(u32p), i64(divisors.size),
                                          numbers.ctypes.data_as(u32p), i64(numbers.size))
    assert bad == 0
