"""Pins the plain-C oracle to the reference.

Two anchors: (1) bit-for-bit agreement with the unmodified reference headers compiled
into oracle/_ref/libmshadow_ref.so (skipped where that library was never built), and
(2) the known-answer cases the reference's own tests and guides describe
(test/test.cu ramp tensor, test/pairtest.cu 6x6 ramp pooling, all-ones pooling cases).
The committed fixtures under tests/golden/ are covered by test_golden.py.
"""
import numpy as np
import pytest

import cpu_checkers as cc
from cpu_checkers import pitched, pool_out

orc = cc.load("orc")
ref = cc.load("ref")
needs_ref = pytest.mark.skipif(ref is None, reason="reference build (oracle/_ref) not present")

NUM_EXPR_CASES = 10


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


def same_bits(a, b):
    return np.array_equal(bits(a), bits(b))


def rnd(rng, shape, lo=-1.0, hi=1.0):
    return rng.uniform(lo, hi, size=shape).astype(np.float32)


# ---------------------------------------------------------------- reference pins
@needs_ref
@pytest.mark.parametrize("cid", range(NUM_EXPR_CASES))
@pytest.mark.parametrize("shape,pad", [((7, 13), 0), ((33, 64), 0), ((5, 100), 4), ((3, 31), 1),
                                       ((64, 257), 7)])
def test_expr_cases_match_reference(cid, shape, pad):
    rng = np.random.default_rng(100 + cid)
    A, B, Cm = (pitched(rnd(rng, shape), pad) for _ in range(3))
    Cm = pitched(rnd(rng, shape, 0.5, 1.5), pad)
    bias = rng.standard_normal(max(shape)).astype(np.float32)
    d0 = rnd(rng, shape, 0.5, 2.0)
    outs = []
    for lib in (orc, ref):
        d = pitched(d0, pad)
        lib.expr_case(cid, d, A, B, Cm, bias)
        outs.append(np.array(d))
    assert same_bits(*outs)


@needs_ref
@pytest.mark.parametrize("reducer", [0, 1, 2])
@pytest.mark.parametrize("saver", [0, 1, 2, 3, 4])
def test_reductions_match_reference(reducer, saver):
    rng = np.random.default_rng(7 * reducer + saver)
    src = pitched(rng.standard_normal((67, 45)).astype(np.float32), 3)
    t4 = pitched(rng.standard_normal((5, 6, 7, 9)).astype(np.float32), 2)
    for fn, s, n in (("reduce_keep_lowest", src, 45), ("reduce_keep_highdim", t4, 6)):
        d0 = rnd(rng, (n,), 1.0, 2.0)
        outs = []
        for lib in (orc, ref):
            d = d0.copy()
            getattr(lib, fn)(d, s, scale=0.75, saver=saver, reducer=reducer)
            outs.append(d)
        assert same_bits(*outs), fn


@needs_ref
@pytest.mark.parametrize("rows,cols,pad", [(1, 1, 0), (4, 8, 0), (9, 1000, 0), (3, 33, 5)])
def test_softmax_family_matches_reference(rows, cols, pad):
    rng = np.random.default_rng(rows * 1000 + cols)
    src = pitched((2.0 * rng.standard_normal((rows, cols))).astype(np.float32), pad)
    outs = []
    for lib in (orc, ref):
        d = pitched(np.zeros((rows, cols), np.float32), pad)
        lib.softmax(d, src)
        outs.append(np.array(d))
    assert same_bits(*outs)
    prob = outs[0]
    label = rng.integers(0, cols, size=rows).astype(np.float32)
    label[0] = cols - 1
    if cols == 1:
        return  # smooth variants divide by cols-1
    for mode in range(4):
        res = []
        for lib in (orc, ref):
            d = np.full((rows, cols), 9.0, np.float32)
            lib.softmax_grad(d, prob, label, mode=mode, ignore_label=float(label[-1]),
                             alpha=0.1)
            res.append(d)
        assert same_bits(*res), mode


@needs_ref
@pytest.mark.parametrize("reducer", [0, 1, 2])
@pytest.mark.parametrize("h,w,ky,kx,sy,sx,pad", [(6, 6, 2, 2, 2, 2, 0), (13, 11, 3, 3, 2, 2, 0),
                                                 (8, 9, 3, 2, 1, 3, 3), (7, 7, 7, 7, 1, 1, 0),
                                                 (10, 10, 2, 2, 3, 3, 0)])
def test_pool_unpool_match_reference(reducer, h, w, ky, kx, sy, sx, pad):
    rng = np.random.default_rng(h * w + reducer)
    # quantised values force ties, which exercise the equality mask of unpool
    src = pitched((rng.integers(0, 4, size=(5, h, w)) * 0.25).astype(np.float32), pad)
    ph, pw = pool_out(h, ky, sy), pool_out(w, kx, sx)
    res = []
    for lib in (orc, ref):
        p = np.zeros((5, ph, pw), np.float32)
        lib.pool(p, src, ky, kx, sy, sx, reducer=reducer)
        g = rnd(np.random.default_rng(3), (5, ph, pw), 0.0, 1.0)
        u = pitched(np.zeros((5, h, w), np.float32), pad)
        lib.unpool(u, src, p, g, ky, kx, sy, sx, reducer=reducer)
        res.append((p, np.array(u)))
    assert same_bits(res[0][0], res[1][0])
    assert same_bits(res[0][1], res[1][1])


@needs_ref
@pytest.mark.parametrize("reducer", [0, 1])
@pytest.mark.parametrize("c,nsize,stride,pad", [(8, 5, 1, 2), (7, 3, 1, 1), (9, 3, 2, 1),
                                                (5, 5, 1, 2), (6, 1, 1, 0)])
def test_chpool_matches_reference(reducer, c, nsize, stride, pad):
    rng = np.random.default_rng(c + nsize)
    src = pitched(rnd(rng, (3, c, 4, 6)), 2)
    co = (c - nsize + 2 * pad + 1) // stride
    res = []
    for lib in (orc, ref):
        d = np.zeros((3, co, 4, 6), np.float32)
        lib.chpool(d, src, nsize, stride, pad, reducer=reducer)
        res.append(d)
    assert same_bits(*res)


@needs_ref
@pytest.mark.parametrize("reducer", [0, 1, 2])
@pytest.mark.parametrize("c,nsize", [(8, 5), (7, 3), (6, 1), (12, 7)])
def test_ch_unpool_matches_reference(reducer, c, nsize):
    rng = np.random.default_rng(c * nsize + reducer)
    shape = (2, c, 3, 5)
    src = pitched((rng.integers(0, 4, shape) / 4.0).astype(np.float32), 1)
    pooled = orc.chpool(np.zeros(shape, np.float32), src, nsize, reducer=reducer)
    g = rnd(rng, shape, 0.0, 1.0)
    res = [lib.ch_unpool(np.zeros(shape, np.float32), src, pooled, g, nsize, reducer=reducer) for lib in (orc, ref)]
    assert same_bits(*res)


@needs_ref
@needs_ref
@pytest.mark.parametrize("power_kind", [0, 1])
@pytest.mark.parametrize("shape,nsize", [((2, 7, 3, 4), 3), ((1, 16, 5, 8), 5), ((3, 20, 4, 4), 7), ((2, 5, 2, 2), 5),
                                         ((1, 9, 1, 1), 9)])
def test_lrn_matches_reference_composition(power_kind, shape, nsize):
    """Local response normalisation as a layer composes it from chpool<red::sum>, F<square> and
    F<power> through the reference's own plans."""
    rng = np.random.default_rng(sum(shape) + nsize)
    x, g = rnd(rng, shape, -2, 2), rnd(rng, shape)
    salpha, beta, knorm = np.float32(0.0001 * 5 / nsize * 40), 0.75, 1.0
    o1, n1 = orc.lrn_forward(x, nsize, salpha, beta, knorm, power_kind)
    o2, n2 = ref.lrn_forward(x, nsize, salpha, beta, knorm, power_kind)
    assert same_bits(o1, o2) and same_bits(n1, n2)
    assert same_bits(orc.lrn_backward(g, x, n1, nsize, salpha, beta, power_kind),
                     ref.lrn_backward(g, x, n2, nsize, salpha, beta, power_kind))


def test_lrn_known_answer():
    # all ones, five channels, window 3, salpha 1, knorm 1, beta 0.75 by roots: the window holds
    # two squares at the ends and three inside, so norm = 3 / 4 and out = norm ^ -0.75
    x = np.ones((1, 5, 1, 1), np.float32)
    out, norm = orc.lrn_forward(x, 3, 1.0, 0.75, 1.0, 1)
    assert norm.ravel().tolist() == [3.0, 4.0, 4.0, 4.0, 3.0]
    r3, r4 = np.sqrt(np.float32(3)), np.float32(2)
    want = [np.float32(1) / (r3 * np.sqrt(r3)), np.float32(1) / (r4 * np.sqrt(r4))]
    assert out.ravel().tolist() == [want[0], want[1], want[1], want[1], want[0]]


def test_addtakegrad_matches_reference():
    rng = np.random.default_rng(5)
    k, d, n = 11, 20, 300
    src = rnd(rng, (n, d))
    idx = rng.integers(-3, k + 3, size=n).astype(np.int32)  # AddTakeGrad clips
    res = []
    for lib in (orc, ref):
        t = rnd(np.random.default_rng(1), (k, d))
        lib.addtakegrad(t, idx, src)
        res.append(t)
    assert same_bits(*res)
    inb = np.clip(idx, 0, k - 1).astype(np.int32)
    res = []
    for lib in (orc, ref):
        keys, vals = inb.copy(), np.arange(n, dtype=np.int32)
        lib.sort_by_key(keys, vals, True)
        t = rnd(np.random.default_rng(1), (k, d))
        lib.addtakegrad_largebatch(t, keys, vals, src)
        res.append((keys, vals, t))
    assert np.array_equal(res[0][0], res[1][0]) and np.array_equal(res[0][1], res[1][1])
    assert same_bits(res[0][2], res[1][2])
    for asc in (True, False):
        pair = []
        for lib in (orc, ref):
            keys, vals = inb.copy(), np.arange(n, dtype=np.int32)
            lib.sort_by_key(keys, vals, asc)
            pair.append((keys, vals))
        assert np.array_equal(pair[0][0], pair[1][0]) and np.array_equal(pair[0][1], pair[1][1])


@needs_ref
@pytest.mark.parametrize("batch,classes,npos,pad", [(1, 1, 1, 0), (2, 5, 7, 0), (3, 21, 64, 0), (2, 9, 33, 3),
                                                    (1, 300, 4, 0)])
def test_softmax3d_family_matches_reference(batch, classes, npos, pad):
    rng = np.random.default_rng(batch * 1000 + classes * 10 + npos)
    src = pitched(rnd(rng, (batch, classes, npos), -4.0, 4.0), pad)
    res = [lib.softmax3d(pitched(np.zeros((batch, classes, npos), np.float32), pad), src) for lib in (orc, ref)]
    assert same_bits(*res)
    label = pitched(rng.integers(0, classes, size=(batch, npos)).astype(np.float32), pad)
    ignore = float(label[0, 0])
    for mode in range(4):
        out = [lib.softmax_grad3d(np.full((batch, classes, npos), 9.0, np.float32), res[0], label, mode, ignore,
                                  0.125) for lib in (orc, ref)]
        assert same_bits(*out), mode


@needs_ref
def test_index_fill_and_vectorized_sort_match_reference():
    rng = np.random.default_rng(77)
    k, d, n = 13, 9, 40
    src = pitched(rnd(rng, (n, d)), 2)
    idx = rng.integers(0, k, size=n).astype(np.int32)  # rows named several times: the later source wins
    res = [lib.index_fill(pitched(np.full((k, d), 3.0, np.float32), 1), idx, src) for lib in (orc, ref)]
    assert same_bits(*res)
    seg = np.sort(rng.integers(0, 6, size=200)).astype(np.int32)
    vals = (rng.integers(0, 20, size=200) / 4.0).astype(np.float32)  # ties inside segments
    out = [lib.vectorized_sort(vals.copy(), seg.copy()) for lib in (orc, ref)]
    assert same_bits(out[0][0], out[1][0]) and np.array_equal(out[0][1], out[1][1])
    assert np.array_equal(out[0][1], seg)
    for s in range(6):
        assert np.array_equal(out[0][0][seg == s], np.sort(vals[seg == s]))


@needs_ref
@pytest.mark.parametrize("cid", range(cc.NUM_REMAP_CASES))
@pytest.mark.parametrize("shape", [(2, 3, 4, 5), (1, 8, 6, 16), (3, 5, 1, 7), (2, 2, 3, 1)])
def test_remap_cases_match_reference(cid, shape):
    rng = np.random.default_rng(cid * 100 + sum(shape))
    A, B = rnd(rng, shape), rnd(rng, shape)
    for p0, p1 in cc.remap_params(cid, shape):
        assert orc.remap_shape(cid, shape, p0, p1) == ref.remap_shape(cid, shape, p0, p1)
        res = [lib.remap_case(cid, A, B, p0, p1, fill=9.0) for lib in (orc, ref)]
        assert same_bits(*res), (cid, p0, p1)


@needs_ref
@pytest.mark.parametrize("cid", range(cc.NUM_AXIS_CASES))
@pytest.mark.parametrize("shape", [(2, 3, 4, 5), (1, 8, 6, 16), (3, 5, 1, 7), (2, 2, 3, 1)])
def test_axis_cases_match_reference(cid, shape):
    rng = np.random.default_rng(cid * 100 + sum(shape))
    A = rnd(rng, shape)
    if cid == 5:
        A[0, 0] = A[-1, -1]  # ties along every axis: the position reported must be the reference's
    for p0, p1 in cc.axis_params(cid, shape):
        assert orc.axis_shape(cid, shape, p0, p1) == ref.axis_shape(cid, shape, p0, p1)
        res = [lib.axis_case(cid, A, p0, p1) for lib in (orc, ref)]
        assert same_bits(*res), (cid, p0, p1)


@needs_ref
@pytest.mark.parametrize("cid", range(cc.NUM_COMPLEX_CASES))
@pytest.mark.parametrize("rows,cols", [(3, 4), (5, 16), (1, 8), (7, 36)])
def test_complex_cases_match_reference(cid, rows, cols):
    rng = np.random.default_rng(cid * 100 + rows + cols)
    A, B = rnd(rng, (rows, cols)), rnd(rng, (rows, cols))
    res = [lib.complex_case(cid, A, B) for lib in (orc, ref)]
    assert same_bits(*res), cid


def test_complex_known_answers():
    rng = np.random.default_rng(9)
    A, B = rnd(rng, (4, 12)), rnd(rng, (4, 12))
    za = A[:, 0::2].astype(np.complex128) + 1j * A[:, 1::2]
    zb = B[:, 0::2].astype(np.complex128) + 1j * B[:, 1::2]

    def inter(z):
        out = np.empty((z.shape[0], z.shape[1] * 2))
        out[:, 0::2], out[:, 1::2] = z.real, z.imag
        return out

    ah, bh = A.ravel()[:24].reshape(4, 6).astype(np.float64), B.ravel()[:24].reshape(4, 6).astype(np.float64)
    want = {0: inter(za * zb), 1: inter(za * bh), 2: inter(ah * zb), 3: inter(za / zb), 4: inter(za / bh),
            5: inter(ah / zb), 6: inter(za.conj()), 7: inter(za.imag + 1j * za.real), 8: inter(ah + 0j),
            9: za.real, 10: np.abs(za) ** 2, 11: za.real + za.imag,
            12: inter(za.conj() * zb + 0.5 * np.abs(zb) ** 2)}
    for cid, w in want.items():
        np.testing.assert_allclose(orc.complex_case(cid, A, B), w, rtol=2e-5, atol=1e-6, err_msg=str(cid))


def test_axis_known_answers():
    rng = np.random.default_rng(5)
    A = rnd(rng, (2, 3, 4, 5))
    assert np.array_equal(orc.axis_case(0, A, 3, 2), np.repeat(np.float32(3) + np.arange(4, dtype=np.float32) * 0.5, 2))
    assert np.array_equal(orc.axis_case(1, A, 3, 4), np.array([7, 5.5, 4], dtype=np.float32))
    assert np.array_equal(orc.axis_case(2, A, 1, 2), A[1:, 2:, 1:3, 2:])
    want = A * 2
    want[1:, 2:, 1:3, 2:] = A[1:, 2:, 1:3, 2:] + 1
    assert np.array_equal(orc.axis_case(3, A, 1, 2), want)
    for axis in range(4):
        seq = np.zeros(np.delete(A.shape, axis), dtype=np.float32)
        for k in range(A.shape[axis]):
            seq = seq + np.take(A, k, axis=axis)  # the reference adds along the axis in order
        assert np.array_equal(orc.axis_case(4, A, axis), seq)
        assert np.array_equal(orc.axis_case(5, A, axis), A.argmax(axis=axis).astype(np.float32))
        assert np.array_equal(orc.axis_case(6, A, axis), A.min(axis=axis, keepdims=True))
        A3 = A.reshape(6, 4, 5)
        assert np.array_equal(orc.axis_case(7, A, axis, 3), np.repeat(np.expand_dims(A3, axis), 3, axis=axis))
    assert np.array_equal(orc.axis_case(8, A, 0, 4), np.repeat(A[:, :1], 4, axis=1))
    S = A.ravel()[:8].reshape(2, 1, 4, 1)
    assert np.array_equal(orc.axis_case(9, A, 3, 2), np.broadcast_to(S, (2, 3, 4, 2)))
    S = A.ravel()[:15].reshape(1, 3, 1, 5)
    assert np.array_equal(orc.axis_case(10, A, 2, 3), np.broadcast_to(S, (2, 3, 3, 5)))


@needs_ref
@pytest.mark.parametrize("cid", range(cc.NUM_SELECT_CASES))
@pytest.mark.parametrize("rows,cols", [(5, 7), (16, 64), (1, 1), (33, 12)])
def test_select_cases_match_reference(cid, rows, cols):
    rng = np.random.default_rng(cid * 100 + rows + cols)
    A, B, ir, ic = cc.select_inputs(rng, rows, cols)
    for p0 in ((1, 2, 3) if cid == 5 else (1,)):
        res = [lib.select_case(cid, A, B, ir, ic, p0) for lib in (orc, ref)]
        assert same_bits(*res), (cid, p0)


@needs_ref
@pytest.mark.parametrize("case", cc.PATCH_CASES)
def test_patch_conversions_match_reference(case):
    shape, psy, psx, sy, sx, dy, dx = case
    rng = np.random.default_rng(sum(shape) + psy * 7 + sx)
    img = rnd(rng, shape)
    mats = [lib.unpack_patch2col(img, psy, psx, sy, sx, dy, dx) for lib in (orc, ref)]
    assert same_bits(*mats)
    grad = rnd(rng, mats[0].shape)
    backs = [lib.pack_col2patch(grad, shape, psy, psx, sy, sx, dy, dx) for lib in (orc, ref)]
    assert same_bits(*backs)


def test_patch_conversions_known_answers():
    # 1 x 1 x 3 x 3 image, 2 x 2 patches, stride 1: four patches, rows (ky, kx), columns (oy, ox)
    img = np.arange(9, dtype=np.float32).reshape(1, 1, 3, 3)
    mat = orc.unpack_patch2col(img, 2, 2, 1, 1)
    assert np.array_equal(mat, np.array([[0, 1, 3, 4], [1, 2, 4, 5], [3, 4, 6, 7], [4, 5, 7, 8]], np.float32))
    # packing ones back counts how many patches cover each pixel
    cover = orc.pack_col2patch(np.ones_like(mat), img.shape, 2, 2, 1, 1)
    assert np.array_equal(cover[0, 0], np.array([[1, 2, 1], [2, 4, 2], [1, 2, 1]], np.float32))


def test_select_known_answers():
    A = np.arange(12, dtype=np.float32).reshape(3, 4)
    B = -A
    ir, ic = np.array([2, 0, 2], np.float32), np.array([3, 0, 1], np.float32)
    assert np.array_equal(orc.select_case(0, A, B, ir, ic), A[[2, 0, 2]])
    assert np.array_equal(orc.select_case(1, A, B, ir, ic), np.eye(4, dtype=np.float32)[[3, 0, 1]])
    assert np.array_equal(orc.select_case(2, A, B, ir, ic), np.array([3, 4, 9], np.float32))
    want = A.copy()
    want[0, 3], want[1, 0], want[2, 1] = B.reshape(-1)[:3]
    assert np.array_equal(orc.select_case(3, A, B, ir, ic), want)
    assert np.array_equal(orc.select_case(4, A, B, ir, ic), A * ic[:, None])
    assert np.array_equal(orc.select_case(5, A, B, ir, ic, 2), A.repeat(2, axis=0).repeat(2, axis=1))
    want = np.zeros_like(A)
    want[2] = A[0] + A[2]
    want[0] = A[1]
    assert np.array_equal(orc.select_case(6, A, B, ir, ic), want)


def test_remap_known_answers():
    A = np.arange(2 * 3 * 2 * 4, dtype=np.float32).reshape(2, 3, 2, 4)
    B = -A
    assert np.array_equal(orc.remap_case(0, A, B), A.reshape(2, 2, 3, 4))
    assert np.array_equal(orc.remap_case(1, A, B, 1, 3), A[:, 1:3])
    assert np.array_equal(orc.remap_case(2, A, B, 1, 4), A[..., 1:4])
    assert np.array_equal(orc.remap_case(3, A, B), np.concatenate([A, B], axis=1))
    assert np.array_equal(orc.remap_case(4, A, B), np.concatenate([A, B], axis=3))
    assert np.array_equal(orc.remap_case(5, A, B), A.swapaxes(1, 2))
    assert np.array_equal(orc.remap_case(6, A, B), A.swapaxes(1, 3))
    assert np.array_equal(orc.remap_case(7, A, B), A.transpose(0, 2, 1, 3))
    assert np.array_equal(orc.remap_case(8, A, B), A.transpose(3, 1, 0, 2))
    assert np.array_equal(orc.remap_case(9, A, B, 1, 2), np.pad(A, ((0, 0), (0, 0), (1, 1), (2, 2))))
    assert np.array_equal(orc.remap_case(10, A, B, 2, 2), A[:, :, :, 1:3])
    assert np.array_equal(orc.remap_case(11, A, B, 1, 3), A[:, :, 1:, 1:])
    assert np.array_equal(orc.remap_case(12, A, B), A[..., ::-1])
    assert np.array_equal(orc.remap_case(13, A, B), A[:, ::-1])
    want = B.copy()
    want[:, 1:3] = A[:, 1:3] + 1
    assert np.array_equal(orc.remap_case(14, A, B, 1, 3), want)
    assert np.array_equal(orc.remap_case(15, A, B), np.concatenate([B, A], axis=0))
    assert np.array_equal(orc.remap_case(16, A, B, 1, 2), A + A[..., ::-1])


def test_softmax3d_and_index_fill_known_answers():
    # constant columns normalise to 1/classes; the gradient subtracts one at the label's class
    p = orc.softmax3d(np.zeros((2, 8, 3), np.float32), np.full((2, 8, 3), 2.5, np.float32))
    assert np.array_equal(p, np.full((2, 8, 3), 0.125, np.float32))
    label = np.array([[0, 7, 3], [1, 1, 1]], np.float32)
    g = orc.softmax_grad3d(np.zeros_like(p), p, label)
    want = p.copy()
    for y in range(2):
        for n in range(3):
            want[y, int(label[y, n]), n] -= 1.0
    assert np.array_equal(g, want)
    g = orc.softmax_grad3d(np.ones_like(p), p, label, mode=2, ignore_label=1.0)
    assert np.array_equal(g[1], np.zeros((8, 3), np.float32)) and np.array_equal(g[0], want[0])
    t = orc.index_fill(np.zeros((4, 2), np.float32), np.array([2, 0, 2], np.int32),
                       np.array([[1, 1], [2, 2], [3, 3]], np.float32))
    assert np.array_equal(t, np.array([[2, 2], [0, 0], [3, 3], [0, 0]], np.float32))


# ---------------------------------------------------------------- known answers
def test_ramp_tensor_known_answers():
    """test/test.cu:12-18 fills (3,2,4) with i*0.1+j*0.2+k*0.1 and reduces batch 0."""
    t = np.zeros((3, 2, 4), np.float32)
    for i in range(3):
        for j in range(2):
            for k in range(4):
                t[i, j, k] = np.float32(i * np.float32(0.1) + j * np.float32(0.2)) + \
                    np.float32(k * np.float32(0.1))
    d = np.zeros(4, np.float32)
    orc.reduce_keep_lowest(d, t[0])
    assert np.allclose(d, [0.2, 0.4, 0.6, 0.8], atol=1e-6)
    d3 = np.zeros(3, np.float32)
    # sumall_except_dim<0> of a 3-D tensor == keep-high-dim with n=1, c=3
    orc.reduce_keep_highdim(d3, t.reshape(1, 3, 2, 4))
    assert np.allclose(d3, [2.0, 2.8, 3.6], atol=1e-5)
    sm = np.zeros((2, 4), np.float32)
    orc.softmax(sm, t[0])
    assert np.allclose(sm.sum(axis=1), 1.0, atol=1e-6)
    e = np.exp(t[0].astype(np.float64))
    assert np.allclose(sm, e / e.sum(axis=1, keepdims=True), atol=1e-6)


def test_pairtest_ramp_pooling_known_answers():
    """test/pairtest.cu:34-39,52-76: 6x6 ramp, max pool K=2 stride 2, unpool of grad 0.1."""
    src = np.arange(36, dtype=np.float32).reshape(1, 6, 6)
    p = np.zeros((1, 3, 3), np.float32)
    orc.pool(p, src, 2, 2, 2, 2, reducer=1)
    assert np.array_equal(p[0], [[7, 9, 11], [19, 21, 23], [31, 33, 35]])
    g = np.full((1, 3, 3), 0.1, np.float32)
    u = np.zeros((1, 6, 6), np.float32)
    orc.unpool(u, src, p, g, 2, 2, 2, 2, reducer=1)
    want = np.zeros((6, 6), np.float32)
    want[1::2, 1::2] = np.float32(0.1)
    assert np.array_equal(u[0], want)
    s = np.zeros((1, 3, 3), np.float32)
    orc.pool(s, src, 2, 2, 2, 2, reducer=0)
    assert np.array_equal(s[0], [[14, 22, 30], [62, 70, 78], [110, 118, 126]])


def test_all_ones_known_answers():
    """Constant planes: every tied position receives the gradient; chpool clamps."""
    x = np.ones((2 * 3, 6, 6), np.float32)
    p = np.zeros((6, 2, 2), np.float32)
    orc.pool(p, x, 3, 3, 2, 2, reducer=1)
    assert np.all(p == 1.0)
    u = np.zeros_like(x)
    orc.unpool(u, x, p, p, 3, 3, 2, 2, reducer=1)
    assert u[0, 2, 2] == 4.0 and u[0, 0, 0] == 1.0 and u[0, 5, 5] == 0.0
    x4 = np.ones((2, 3, 6, 6), np.float32)
    c = np.zeros_like(x4)
    orc.chpool(c, x4, 3)
    assert np.all(c[:, 0] == 2.0) and np.all(c[:, 1] == 3.0) and np.all(c[:, 2] == 2.0)
    d = np.zeros(3, np.float32)
    orc.reduce_keep_highdim(d, x4)
    assert np.all(d == 72.0)
    sm = np.zeros((1, 8), np.float32)
    orc.softmax(sm, np.full((1, 8), 3.0, np.float32))
    assert np.all(sm == 0.125)


def test_softmax_grad_label_edges():
    prob = np.full((3, 5), 0.2, np.float32)
    label = np.array([0, 4, 2], np.float32)
    d = np.zeros_like(prob)
    orc.softmax_grad(d, prob, label)
    want = prob.copy()
    want[0, 0] -= 1
    want[1, 4] -= 1
    want[2, 2] -= 1
    assert np.array_equal(d, want)
    orc.softmax_grad(d, prob, label, mode=2, ignore_label=4.0)
    assert np.all(d[1] == 0.0) and np.array_equal(d[0], want[0])


def test_addtakegrad_clips_and_sort_is_stable():
    t = np.zeros((3, 2), np.float32)
    orc.addtakegrad(t, np.array([-5, 7, 1, 1], np.int32), np.ones((4, 2), np.float32))
    assert np.array_equal(t[:, 0], [1, 2, 1])
    keys = np.array([2, 0, 2, 1, 0], np.int32)
    vals = np.arange(5, dtype=np.int32)
    orc.sort_by_key(keys, vals, True)
    assert list(keys) == [0, 0, 1, 2, 2] and list(vals) == [1, 4, 3, 0, 2]
