"""GPU parity: every C-ABI operator against the CPU oracle on the same seeded inputs.

Tolerances (stated by the task for this path):
  * bit-exact  pooling / unpooling / channel pooling, SoftmaxGrad, sorting, and every
               element-wise expression built from + - * / and comparisons;
  * <= 1 ulp   the sigmoid expression (its exp is evaluated to the host library's rounding);
  * 1e-5       relative, for fp32 sums: reductions, softmax, AddTakeGrad.  For sums the
               error is measured against max(|reference|, RMS of the reference output), since
               an element-wise relative error is meaningless next to a zero crossing; for
               embedding tables the RMS is taken per table row, because rows are sums of very
               different lengths.
"""
import numpy as np
import pytest

import cpu_checkers as cc
from cpu_checkers import pool_out

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


def dev(a, pad=0, fill=7.5):
    """Copy a numpy array to the GPU, optionally with `pad` extra elements per row."""
    a = np.asarray(a)
    if pad == 0:
        return torch.from_numpy(np.ascontiguousarray(a)).cuda()
    buf = torch.full(a.shape[:-1] + (a.shape[-1] + pad,), fill, dtype=torch.from_numpy(a[..., :1].copy()).dtype,
                     device="cuda")
    view = buf[..., : a.shape[-1]]
    view.copy_(torch.from_numpy(np.ascontiguousarray(a)))
    return view


def host(t):
    return t.cpu().numpy()


def ulp_diff(a, b):
    ia = np.ascontiguousarray(a).view(np.int32).astype(np.int64)
    ib = np.ascontiguousarray(b).view(np.int32).astype(np.int64)
    # map the sign-magnitude float order onto a monotone integer line
    ia = np.where(ia < 0, -(ia & 0x7FFFFFFF), ia)
    ib = np.where(ib < 0, -(ib & 0x7FFFFFFF), ib)
    return np.abs(ia - ib)


def assert_bits(got, want):
    got, want = np.ascontiguousarray(got), np.ascontiguousarray(want)
    same = got.view(np.uint32) == want.view(np.uint32)
    assert same.all(), "%d of %d elements differ; first at %s" % (
        (~same).sum(), same.size, np.argwhere(~same)[0])


def assert_sum_close(got, want, tol=1e-5, per_row=False):
    """|got - want| <= tol * max(|want|, s); s is the RMS of the reference output, taken per
    row when rows are sums of very different lengths (embedding tables)."""
    w64 = want.astype(np.float64)
    rms = np.sqrt(np.mean(w64 ** 2, axis=-1, keepdims=True)) if per_row else np.sqrt(np.mean(w64 ** 2))
    scale = np.maximum(np.abs(want), rms)
    err = np.abs(got.astype(np.float64) - want) / np.maximum(scale, 1e-30)
    assert err.max() <= tol, "max scaled error %.3g" % err.max()


def apply_saver(d0, value, saver):
    """mshadow's sv:: savers as single fp32 operations (mshadow/base.h:539-602)."""
    d0, value = d0.astype(np.float32), value.astype(np.float32)
    return [value, d0 + value, d0 - value, d0 * value, d0 / value][saver].astype(np.float32)


SHAPES = [((1, 1), 0), ((7, 13), 0), ((33, 64), 0), ((5, 100), 4), ((3, 31), 1), ((64, 257), 7),
          ((16, 1024), 0), ((9, 1000), 24), ((300, 5), 0), ((2, 4099), 0)]


@pytest.mark.parametrize("cid", range(10))
@pytest.mark.parametrize("shape,pad", SHAPES)
def test_expression_cases(lib, cid, shape, pad):
    rng = np.random.default_rng(100 * cid + shape[0] + shape[1])
    A = rng.uniform(-1, 1, shape).astype(np.float32)
    B = rng.uniform(-1, 1, shape).astype(np.float32)
    Cm = rng.uniform(0.5, 1.5, shape).astype(np.float32)
    bias = rng.standard_normal(max(shape)).astype(np.float32)
    d0 = rng.uniform(0.5, 2.0, shape).astype(np.float32)
    want = orc.expr_case(cid, d0.copy(), A, B, Cm, bias)
    d = dev(d0, pad)
    lib.expr_case(cid, d, dev(A, pad), dev(B, pad), dev(Cm, pad), dev(bias))
    got = host(d)
    if cid == 0:
        assert ulp_diff(got, want).max() <= 1
    else:
        assert_bits(got, want)


def test_expression_in_place_and_padding_untouched(lib):
    rng = np.random.default_rng(3)
    A = rng.uniform(-1, 1, (17, 100)).astype(np.float32)
    buf = torch.full((17, 104), 7.5, device="cuda")
    view = buf[:, :100]
    view.copy_(torch.from_numpy(A))
    # dst aliases A: d *= A + 1.5
    want = orc.expr_case(3, A.copy(), A, A, A, A[0])
    lib.expr_case(3, view, view, view, view, dev(A[0]))
    assert_bits(host(view), want)
    assert bool((buf[:, 100:] == 7.5).all()), "row padding was overwritten"


@pytest.mark.parametrize("reducer", [0, 1, 2])
@pytest.mark.parametrize("saver", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("rows,cols,pad", [(1, 1, 0), (67, 45, 3), (1000, 128, 0), (4097, 260, 0), (33, 1030, 2),
                                           (5000, 8, 0)])
def test_reduce_keep_lowest(lib, reducer, saver, rows, cols, pad):
    rng = np.random.default_rng(rows + cols + reducer)
    src = rng.standard_normal((rows, cols)).astype(np.float32)
    d0 = rng.uniform(1, 2, cols).astype(np.float32)
    want = orc.reduce_keep_lowest(d0.copy(), src, scale=0.75, saver=saver, reducer=reducer)
    got = host(lib.reduce_keep_lowest(dev(d0), dev(src, pad), scale=0.75, saver=saver, reducer=reducer))
    if reducer != 0:
        assert_bits(got, want)
    elif saver == 0:
        assert_sum_close(got, want)
    else:
        # the sum itself is checked with saver 0; a saver is one rounded operation on it
        plain = host(lib.reduce_keep_lowest(dev(d0), dev(src, pad), scale=0.75, saver=0, reducer=0))
        assert_bits(got, apply_saver(d0, plain, saver))


@pytest.mark.parametrize("reducer", [0, 1, 2])
@pytest.mark.parametrize("saver", [0, 1, 4])
@pytest.mark.parametrize("shape,pad", [((1, 1, 1, 1), 0), ((5, 6, 7, 9), 2), ((16, 32, 28, 28), 0),
                                       ((3, 1030, 2, 4), 0), ((600, 3, 5, 8), 0), ((2, 7, 27, 27), 0)])
def test_reduce_keep_highdim(lib, reducer, saver, shape, pad):
    rng = np.random.default_rng(sum(shape) + reducer)
    src = rng.standard_normal(shape).astype(np.float32)
    d0 = rng.uniform(1, 2, shape[1]).astype(np.float32)
    want = orc.reduce_keep_highdim(d0.copy(), src, scale=0.5, saver=saver, reducer=reducer)
    got = host(lib.reduce_keep_highdim(dev(d0), dev(src, pad), scale=0.5, saver=saver, reducer=reducer))
    if reducer != 0:
        assert_bits(got, want)
    elif saver == 0:
        assert_sum_close(got, want)
    else:
        plain = host(lib.reduce_keep_highdim(dev(d0), dev(src, pad), scale=0.5, saver=0, reducer=0))
        assert_bits(got, apply_saver(d0, plain, saver))


@pytest.mark.parametrize("rows,cols,pad", [(1, 1, 0), (4, 8, 0), (9, 1000, 0), (3, 33, 5), (5, 4096, 0),
                                           (4, 32000, 0), (3, 31999, 0), (2, 8193, 0), (2, 40000, 0), (70, 513, 3),
                                           (300, 128, 0),
                                           # many long rows: the persistent, bulk-copy staged kernel
                                           (200, 4096, 0), (333, 12000, 0), (150, 32000, 0), (149, 32768, 0),
                                           (450, 6000, 8),
                                           # rows beyond the register kernels: one pass with a running
                                           # (max, sum), the row split over a cluster when rows are few
                                           (4, 100000, 0), (64, 65536, 0), (3, 40001, 0), (2, 131072, 4),
                                           (200, 33000, 0), (1, 1000003, 0)])
def test_softmax(lib, rows, cols, pad):
    rng = np.random.default_rng(rows * 1000 + cols)
    src = (2.0 * rng.standard_normal((rows, cols))).astype(np.float32)
    want = orc.softmax(np.zeros_like(src), src)
    d = dev(np.zeros_like(src), pad)
    lib.softmax(d, dev(src, pad))
    got = host(d)
    rel = np.abs(got.astype(np.float64) - want) / np.maximum(want, 1e-37)
    # The CPU adds a row's exponentials one after the other in binary32; beyond some ten thousand
    # columns the rounding of that sum alone passes 1e-5.  A binary64 evaluation says how much of a
    # difference is the CPU's: the GPU must be within 1e-5 of the truth, and of the CPU up to that.
    x64 = src.astype(np.float64)
    e64 = np.exp(x64 - x64.max(axis=1, keepdims=True))
    truth = e64 / e64.sum(axis=1, keepdims=True)
    ok = want > 0
    cpu_off = (np.abs(want - truth) / truth)[ok].max()
    assert (np.abs(got - truth) / truth)[ok].max() <= 1e-5
    assert rel[ok].max() <= 1e-5 + cpu_off
    assert np.all(got[want == 0] <= 1e-37)
    # in place, as in Softmax(out, out)
    s = dev(src, pad)
    lib.softmax(s, s)
    assert_bits(host(s), got)


@pytest.mark.parametrize("rows,cols,pad", [(3, 5, 0), (9, 1000, 0), (4, 33, 3), (160, 8000, 0), (2, 40000, 0),
                                           (5, 70001, 0)])
def test_softmax_grad_fused(lib, rows, cols, pad):
    """One pass Softmax + SoftmaxGrad must equal the two library calls it replaces, exactly,
    and the CPU composition within the softmax tolerance."""
    rng = np.random.default_rng(rows + cols)
    logits = (2.0 * rng.standard_normal((rows, cols))).astype(np.float32)
    label = rng.integers(0, cols, rows).astype(np.float32)
    label[0], label[-1] = 0, cols - 1
    fused = dev(np.zeros_like(logits), pad)
    lib.softmax_grad_fused(fused, dev(logits, pad), dev(label))
    prob = dev(np.zeros_like(logits), pad)
    lib.softmax(prob, dev(logits, pad))
    two = dev(np.zeros_like(logits), pad)
    lib.softmax_grad(two, prob, dev(label))
    assert_bits(host(fused), host(two))
    cpu_prob = orc.softmax(np.zeros_like(logits), logits)
    want = orc.softmax_grad(np.zeros_like(logits), cpu_prob, label)
    err = np.abs(host(fused).astype(np.float64) - want) / np.maximum(np.abs(want), 1e-30)
    hit = np.zeros(want.shape, bool)
    hit[np.arange(rows), label.astype(int)] = True
    # the CPU's left-to-right row sum carries its own rounding, beyond 1e-5 for very long rows
    x64 = logits.astype(np.float64)
    e64 = np.exp(x64 - x64.max(axis=1, keepdims=True))
    truth = e64 / e64.sum(axis=1, keepdims=True)
    cpu_off = (np.abs(cpu_prob - truth) / truth)[cpu_prob > 0].max()
    assert err[~hit & (want > 0)].max() <= 1e-5 + cpu_off if (~hit & (want > 0)).any() else True
    assert np.abs(host(fused)[hit] - want[hit]).max() <= 1e-5  # p - 1: absolute, the scale is 1


@pytest.mark.parametrize("mode", [0, 1, 2, 3])
@pytest.mark.parametrize("rows,cols,pad", [(3, 5, 0), (9, 1000, 0), (4, 33, 3), (6, 32000, 0), (64, 260, 4)])
def test_softmax_grad(lib, mode, rows, cols, pad):
    rng = np.random.default_rng(rows + cols + mode)
    prob = rng.uniform(0, 1, (rows, cols)).astype(np.float32)
    label = rng.integers(0, cols, rows).astype(np.float32)
    label[0], label[-1] = 0, cols - 1
    ignore = float(label[1])
    want = orc.softmax_grad(np.zeros_like(prob), prob, label, mode=mode, ignore_label=ignore, alpha=0.1)
    d = dev(np.full_like(prob, 9.0), pad)
    lib.softmax_grad(d, dev(prob, pad), dev(label), mode=mode, ignore_label=ignore, alpha=0.1)
    assert_bits(host(d), want)


POOL_CASES = [(5, 6, 6, 2, 2, 2, 2, 0), (5, 13, 11, 3, 3, 2, 2, 0), (3, 8, 9, 3, 2, 1, 3, 3), (2, 7, 7, 7, 7, 1, 1, 0),
              (4, 10, 10, 2, 2, 3, 3, 0), (9, 56, 56, 3, 3, 2, 2, 0), (8, 27, 27, 3, 3, 2, 2, 0),
              (70, 12, 12, 2, 2, 2, 2, 0), (3, 130, 120, 5, 4, 3, 2, 0),
              # 3 x 3 / 2 on widths that are multiples of four (two outputs per thread), dense and pitched
              (6, 20, 24, 3, 3, 2, 2, 4), (33, 9, 8, 3, 3, 2, 2, 0), (2, 64, 128, 3, 3, 2, 2, 0),
              # planes beyond shared memory: bands of rows (aligned widths, odd widths whose bands start off a
              # 16-byte boundary, a general window, pitched rows, a single plane, 2 x 2 windows)
              (3, 112, 112, 3, 3, 2, 2, 0), (2, 224, 224, 3, 3, 2, 2, 0), (2, 513, 517, 3, 3, 2, 2, 0),
              (1, 513, 517, 5, 4, 3, 2, 0), (3, 150, 131, 3, 3, 2, 2, 3), (1, 300, 260, 2, 2, 2, 2, 0),
              (5, 97, 203, 3, 3, 1, 1, 0)]


@pytest.mark.parametrize("reducer", [0, 1, 2])
@pytest.mark.parametrize("planes,h,w,ky,kx,sy,sx,pad", POOL_CASES)
def test_pool_unpool(lib, reducer, planes, h, w, ky, kx, sy, sx, pad):
    rng = np.random.default_rng(h * w + reducer + planes)
    # values on a coarse grid produce many tied maxima
    src = (rng.integers(0, 8, size=(planes, h, w)) * 0.125).astype(np.float32)
    ph, pw = pool_out(h, ky, sy), pool_out(w, kx, sx)
    g = rng.uniform(0, 1, (planes, ph, pw)).astype(np.float32)
    wp = orc.pool(np.zeros((planes, ph, pw), np.float32), src, ky, kx, sy, sx, reducer=reducer)
    wu = orc.unpool(np.zeros_like(src), src, wp, g, ky, kx, sy, sx, reducer=reducer)
    dsrc = dev(src, pad)
    dp = lib.pool(torch.zeros(planes, ph, pw, device="cuda"), dsrc, ky, kx, sy, sx, reducer=reducer)
    assert_bits(host(dp), wp)
    du = dev(np.zeros_like(src), pad)
    lib.unpool(du, dsrc, dp, dev(g), ky, kx, sy, sx, reducer=reducer)
    assert_bits(host(du), wu)


def test_unpool_all_tied(lib):
    x = np.ones((6, 6, 6), np.float32)
    p = host(lib.pool(torch.zeros(6, 2, 2, device="cuda"), dev(x), 3, 3, 2, 2))
    assert np.all(p == 1.0)
    u = host(lib.unpool(torch.zeros(6, 6, 6, device="cuda"), dev(x), dev(p), dev(p), 3, 3, 2, 2))
    assert u[0, 2, 2] == 4.0 and u[0, 0, 0] == 1.0 and u[0, 5, 5] == 0.0


@pytest.mark.parametrize("reducer", [0, 1])
@pytest.mark.parametrize("shape,nsize,stride,pad", [((3, 8, 4, 6), 5, 1, 2), ((2, 7, 5, 5), 3, 1, 1),
                                                    ((2, 9, 4, 4), 3, 2, 1), ((1, 5, 2, 2), 5, 1, 2),
                                                    ((2, 6, 3, 4), 1, 1, 0), ((2, 40, 14, 14), 5, 1, 2),
                                                    ((2, 20, 7, 9), 7, 1, 3), ((1, 12, 8, 8), 9, 1, 4),
                                                    ((2, 10, 6, 6), 5, 1, 0),
                                                    # shared-memory ring kernel: whole planes, plane tiles,
                                                    # several channel segments
                                                    ((3, 33, 56, 56), 3, 1, 1), ((2, 24, 80, 80), 5, 1, 2),
                                                    ((40, 64, 28, 28), 5, 1, 2), ((1, 19, 4, 4), 9, 1, 4),
                                                    ((2, 300, 12, 12), 7, 1, 3)])
def test_chpool(lib, reducer, shape, nsize, stride, pad):
    rng = np.random.default_rng(sum(shape) + nsize)
    src = rng.uniform(-1, 1, shape).astype(np.float32)
    co = (shape[1] - nsize + 2 * pad + 1) // stride
    out_shape = (shape[0], co, shape[2], shape[3])
    want = orc.chpool(np.zeros(out_shape, np.float32), src, nsize, stride, pad, reducer=reducer)
    got = lib.chpool(torch.zeros(out_shape, device="cuda"), dev(src), nsize, stride, pad, reducer=reducer)
    assert_bits(host(got), want)


@pytest.mark.parametrize("reducer", [0, 1, 2])
@pytest.mark.parametrize("shape,nsize,pad", [((2, 8, 3, 5), 5, 0), ((2, 7, 4, 4), 3, 0), ((3, 16, 6, 6), 5, 2),
                                             ((1, 12, 5, 8), 7, 0), ((2, 6, 3, 3), 1, 3),
                                             ((3, 200, 16, 24), 5, 0),   # channel march cut into segments
                                             ((2, 130, 7, 9), 3, 0),     # segments, one pixel per thread
                                             ((40, 9, 32, 32), 7, 0),    # many images, window wider than half the channels
                                             ((2, 24, 4, 4), 9, 0)])     # window the ring kernel is not built for
def test_ch_unpool(lib, reducer, shape, nsize, pad):
    """Gradient of chpool(src, nsize): pooled has as many channels as the source."""
    rng = np.random.default_rng(sum(shape) + nsize + reducer)
    src = (rng.integers(0, 4, shape) / 4.0).astype(np.float32)  # coarse values: ties
    pooled = orc.chpool(np.zeros(shape, np.float32), src, nsize, reducer=reducer)
    g = rng.uniform(0, 1, shape).astype(np.float32)
    want = orc.ch_unpool(np.zeros(shape, np.float32), src, pooled, g, nsize, reducer=reducer)
    got = lib.ch_unpool(dev(np.zeros(shape, np.float32), pad), dev(src, pad), dev(pooled), dev(g), nsize,
                        reducer=reducer)
    assert_bits(host(got), want)


def zipf_indices(rng, n, k, s=1.1):
    p = (np.arange(k) + 1.0) ** (-s)
    return rng.choice(k, size=n, p=p / p.sum()).astype(np.int32)


@pytest.mark.parametrize("power_kind", [0, 1, 2])
@pytest.mark.parametrize("shape,nsize", [((2, 16, 8, 8), 5), ((3, 32, 12, 12), 3), ((1, 64, 56, 56), 5), ((2, 20, 4, 8), 7),
                                         ((2, 96, 64, 64), 5),          # planes cut into tiles
                                         ((2, 7, 3, 5), 3), ((1, 9, 4, 4), 5)])  # odd planes, few channels: expressions
def test_lrn_forward_backward(lib, power_kind, shape, nsize):
    """One-pass LRN against the composition through chpool<red::sum>: bit-exact when the power functor
    is built from correctly rounded operations (roots), within 1e-5 with powf (the C library's on the
    CPU, CUDA's on the GPU)."""
    rng = np.random.default_rng(sum(shape) + nsize)
    x = rng.uniform(-2, 2, shape).astype(np.float32)
    g = rng.uniform(-1, 1, shape).astype(np.float32)
    salpha, beta, knorm = float(np.float32(0.02 / nsize)), 0.75, 1.0
    want_out, want_norm = orc.lrn_forward(x, nsize, salpha, beta, knorm, power_kind)
    want_g = orc.lrn_backward(g, x, want_norm, nsize, salpha, beta, power_kind)
    out, norm = torch.empty(shape, device="cuda"), torch.empty(shape, device="cuda")
    lib.lrn_forward(out, norm, dev(x), nsize, salpha, beta, knorm, power_kind)
    gs = lib.lrn_backward(torch.empty(shape, device="cuda"), dev(g), dev(x), dev(want_norm), nsize, salpha, beta,
                          power_kind)
    assert_bits(host(norm), want_norm)
    if power_kind == 1:
        assert_bits(host(out), want_out)
        assert_bits(host(gs), want_g)
    else:
        assert np.abs(host(out) - want_out).max() <= 1e-5 * np.abs(want_out).max()
        assert np.abs(host(gs) - want_g).max() <= 1e-5 * np.abs(want_g).max()
    # without keeping the norm (fused shapes only): same output
    if shape[1] >= 2 * nsize and (shape[2] * shape[3]) % 4 == 0:
        out2 = lib.lrn_forward(torch.empty(shape, device="cuda"), None, dev(x), nsize, salpha, beta, knorm, power_kind)
        assert_bits(host(out2), host(out))


@pytest.mark.parametrize("k,d,n,kind", [(11, 20, 300, "uniform"), (50, 64, 600, "uniform"), (1, 8, 1000, "uniform"),
                                        (4000, 128, 3000, "distinct"), (300, 1024, 5000, "zipf"),
                                        (64, 1028, 700, "zipf"), (200, 4, 40000, "zipf"), (7, 33, 1, "uniform"),
                                        # long lists: the staged first level (rows of 1 KB and more), the register
                                        # forms of the first level (narrow and odd-width rows), short-chunk levels above
                                        (300, 1024, 30000, "zipf"), (5000, 256, 25000, "uniform"),
                                        (90, 33, 25000, "zipf"), (3, 512, 20000, "uniform"),
                                        # short lists: every level in the short-chunk register form
                                        (2, 1024, 512, "uniform"), (5, 64, 513, "uniform"), (1, 132, 100, "uniform"),
                                        (40, 256, 37, "distinct"), (400, 12, 511, "zipf")])
def test_addtakegrad_largebatch(lib, k, d, n, kind):
    rng = np.random.default_rng(k + d + n)
    if kind == "uniform":
        idx = rng.integers(0, k, n).astype(np.int32)
    elif kind == "distinct":
        idx = rng.permutation(k)[:n].astype(np.int32)
    else:
        idx = zipf_indices(rng, n, k)
    src = rng.standard_normal((n, d)).astype(np.float32)
    keys, vals = idx.copy(), np.arange(n, dtype=np.int32)
    orc.sort_by_key(keys, vals, True)
    t0 = rng.standard_normal((k, d)).astype(np.float32)
    want = orc.addtakegrad_largebatch(t0.copy(), keys, vals, src)
    got = lib.addtakegrad_largebatch(dev(t0), dev(keys), dev(vals), dev(src))
    assert_sum_close(host(got), want, per_row=True)
    # untouched rows stay bit-identical
    untouched = np.setdiff1d(np.arange(k), idx)
    assert_bits(host(got)[untouched], t0[untouched])


@pytest.mark.parametrize("k,d,n", [(11, 20, 300), (128, 256, 4096), (5, 1024, 513)])
def test_addtakegrad_unsorted_clips(lib, k, d, n):
    rng = np.random.default_rng(k * d + n)
    idx = rng.integers(-3, k + 3, n).astype(np.int32)
    src = rng.standard_normal((n, d)).astype(np.float32)
    t0 = rng.standard_normal((k, d)).astype(np.float32)
    want = orc.addtakegrad(t0.copy(), idx, src)
    got = lib.addtakegrad(dev(t0, 4), dev(idx), dev(src, 4))
    assert_sum_close(host(got), want, per_row=True)


@pytest.mark.parametrize("n", [1, 2, 1000, 70000])
@pytest.mark.parametrize("ascend", [True, False])
def test_sort_by_key(lib, n, ascend):
    rng = np.random.default_rng(n)
    keys = rng.integers(-50, 50, n).astype(np.int32)
    vals = np.arange(n, dtype=np.int32)
    wk, wv = orc.sort_by_key(keys.copy(), vals.copy(), ascend)
    gk, gv = lib.sort_by_key(dev(keys), dev(vals), ascend)
    assert np.array_equal(host(gk), wk) and np.array_equal(host(gv), wv)


@pytest.mark.parametrize("n,rows,count", [(1, 5, 1), (300, 7, 4), (5000, 40, 64), (70000, 3000, 64), (200000, 50000, 64)])
def test_frequent_rows_match_the_host_selection(lib, n, rows, count):
    """msb_frequent_rows_i32 against mshadow_b200.sharding.hot_rows: the same rows, exactly."""
    from mshadow_b200 import sharding
    rng = np.random.default_rng(n + count)
    p = (np.arange(rows) + 1.0) ** -1.1
    keys = np.sort(rng.choice(rows, size=n, p=p / p.sum()).astype(np.int32))
    count = min(count, n)
    out_rows = torch.zeros(count, dtype=torch.int32, device="cuda")
    out_counts = torch.zeros(count, dtype=torch.int32, device="cuda")
    lib.frequent_rows(out_rows, out_counts, dev(keys))
    got_rows, got_counts = host(out_rows), host(out_counts)
    uniq, counts = np.unique(keys, return_counts=True)
    order = np.argsort(-counts, kind="stable")[:count]
    valid = got_counts > 0
    assert valid.sum() == min(count, uniq.size)
    assert np.array_equal(got_rows[valid], uniq[order]) and np.array_equal(got_counts[valid], counts[order])
    assert np.array_equal(np.sort(got_rows[valid]), sharding.hot_rows(keys, count))


@pytest.mark.parametrize("n,rows", [(1, 5), (300, 7), (2048, 2048), (2049, 3), (70000, 3000), (200001, 50000)])
def test_run_numbering_of_a_sorted_list(lib, n, rows):
    """msb_run_index_i32 against numpy: run number of every entry, key of every run, number of runs."""
    rng = np.random.default_rng(n + rows)
    keys = np.sort(rng.integers(0, rows, n).astype(np.int32))
    run_of = torch.full((n,), -7, dtype=torch.int32, device="cuda")
    run_keys = torch.full((n,), -7, dtype=torch.int32, device="cuda")
    total = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib.run_index(run_of, run_keys, total, dev(keys))
    uniq, inverse = np.unique(keys, return_inverse=True)
    assert int(host(total)[0]) == uniq.size
    assert np.array_equal(host(run_of), inverse.astype(np.int32))
    assert np.array_equal(host(run_keys)[:uniq.size], uniq) and np.all(host(run_keys)[uniq.size:] == -7)


@pytest.mark.parametrize("n,table_rows,d,world", [(1, 5, 8, 1), (300, 40, 20, 2), (5000, 300, 1024, 3),
                                                 (30000, 5000, 256, 8), (40000, 64, 1024, 4)])
def test_sums_stored_into_the_owners_blocks(lib, n, table_rows, d, world):
    """The sender's half of the placement 'source rows sharded by batch position': entries sorted by
    (owner, local row), runs numbered, owners' blocks found, every run's sum STORED into its row of
    its owner's block and the local row number beside it.  The blocks here are all in this GPU's
    memory; the sums are compared with the CPU evaluation of AddTakeGradLargeBatch on a zero table."""
    rng = np.random.default_rng(n + world)
    idx = zipf_indices(rng, n, table_rows)
    src = rng.standard_normal((n, d)).astype(np.float32)
    per_owner = (table_rows + world - 1) // world
    ck = ((idx % world) * per_owner + idx // world).astype(np.int32)
    pos = np.arange(n, dtype=np.int32)
    dck, dpos = lib.sort_by_key(dev(ck), dev(pos), True)
    run_of = torch.empty(n, dtype=torch.int32, device="cuda")
    run_keys = torch.empty(n, dtype=torch.int32, device="cuda")
    total = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib.run_index(run_of, run_keys, total, dck)
    first = torch.full((world + 1,), -1, dtype=torch.int32, device="cuda")
    lib.run_bounds(first, run_keys, total, world, per_owner)
    uniq = np.unique(ck)
    want_first = np.searchsorted(uniq, np.arange(world + 1) * per_owner).astype(np.int32)
    assert np.array_equal(host(first), want_first)
    rows = [torch.full((per_owner, d), 7.5, device="cuda") for _ in range(world)]
    keys = [torch.full((per_owner,), -7, dtype=torch.int32, device="cuda") for _ in range(world)]
    dsrc = dev(src)
    lib.take_sum_to_owners([t.data_ptr() for t in rows], first, run_of, dpos, dsrc, world)
    lib.run_keys_to_owners([t.data_ptr() for t in keys], first, run_keys, world, per_owner)
    order = np.argsort(idx, kind="stable").astype(np.int32)
    table = orc.addtakegrad_largebatch(np.zeros((table_rows, d), np.float32), idx[order], order, src)
    for q in range(world):
        cnt = int(want_first[q + 1] - want_first[q])
        local = uniq[want_first[q]:want_first[q + 1]] - q * per_owner
        assert np.array_equal(host(keys[q])[:cnt], local) and np.all(host(keys[q])[cnt:] == -7)
        got = host(rows[q])
        assert np.all(got[cnt:] == 7.5)                       # rows beyond the owner's runs stay untouched
        if cnt:
            assert_sum_close(got[:cnt], table[local * world + q], per_row=True)


@pytest.mark.parametrize("n,rows,nhot", [(1, 5, 0), (300, 7, 2), (5000, 40, 8), (70000, 3000, 64), (200001, 50000, 64)])
@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_routing_on_the_device_matches_the_host_routing(lib, n, rows, nhot, world):
    """msb_route_cyclic_hot_i32 against mshadow_b200.sharding.route_cyclic_with_hot_rows for every
    rank of the group: the same entries in the same order, exactly."""
    from mshadow_b200 import sharding
    rng = np.random.default_rng(n + world)
    p = (np.arange(rows) + 1.0) ** -1.1
    idx = rng.choice(rows, size=n, p=p / p.sum()).astype(np.int32)
    order = np.argsort(idx, kind="stable").astype(np.int32)
    keys = idx[order]
    hot = sharding.hot_rows(keys, nhot)
    dk, do = dev(keys), dev(order)
    dhot = dev(hot) if hot.size else None
    for rank in range(world):
        tk, to, hk, ho = sharding.route_cyclic_with_hot_rows(keys, order, n, rank, world, hot)
        b, e = sharding.shard_range(n, rank, world)
        rows_mine = (rows - rank + world - 1) // world
        ok = torch.full((n,), -7, dtype=torch.int32, device="cuda")
        oo = torch.full((n,), -7, dtype=torch.int32, device="cuda")
        totals = torch.zeros(2, dtype=torch.int32, device="cuda")
        lib.route_cyclic_hot(ok, oo, totals, dk, do, dhot, world, rank, b, e, rows_mine)
        nt, nh = (int(v) for v in host(totals))
        assert (nt, nh) == (tk.size, hk.size)
        assert np.array_equal(host(ok)[:nt], tk) and np.array_equal(host(oo)[:nt], to)
        assert np.array_equal(host(ok)[nt:nt + nh], hk + rows_mine) and np.array_equal(host(oo)[nt:nt + nh], ho)
        assert np.all(host(ok)[nt + nh:] == -7)


@pytest.mark.parametrize("n,bits", [(2, 1), (1000, 7), (70000, 18), (70000, 19), (300000, 31)])
def test_sort_by_key_on_the_significant_bits(lib, n, bits):
    rng = np.random.default_rng(n + bits)
    keys = rng.integers(0, 2 ** bits, n, dtype=np.int64).astype(np.int32)
    vals = np.arange(n, dtype=np.int32)
    order = np.argsort(keys, kind="stable")
    gk, gv = lib.sort_by_key(dev(keys), dev(vals), True, bits=bits)
    assert np.array_equal(host(gk), keys[order]) and np.array_equal(host(gv), vals[order])


@pytest.mark.parametrize("batch,classes,npos,pad", [
    (1, 1, 1, 0), (2, 5, 7, 0), (3, 21, 64, 0), (2, 9, 33, 3), (2, 21, 1024, 0), (1, 19, 4100, 4),
    (2, 100, 512, 0),    # 128-bit tile too large for shared memory: one position per thread
    (1, 600, 1024, 0),   # no tile fits: exponentials parked in dst
    (1, 600, 130, 2),
])
def test_softmax3d_family(lib, batch, classes, npos, pad):
    rng = np.random.default_rng(batch * 100000 + classes * 1000 + npos)
    src = (rng.standard_normal((batch, classes, npos)) * 2).astype(np.float32)
    want = orc.softmax3d(np.zeros_like(src), src)
    got = lib.softmax3d(dev(np.zeros_like(src), pad), dev(src, pad))
    rel = np.abs(host(got).astype(np.float64) - want) / np.maximum(np.abs(want), 1e-30)
    assert rel.max() <= 1e-5, rel.max()
    # in place, as the reference allows
    buf = dev(src, pad)
    lib.softmax3d(buf, buf)
    assert_bits(host(buf), host(got))
    label = rng.integers(0, classes, size=(batch, npos)).astype(np.float32)
    ignore = float(label[0, 0])
    for mode in range(4):
        w = orc.softmax_grad3d(np.full_like(src, 9.0), want, label, mode, ignore, 0.125)
        g = lib.softmax_grad3d(dev(np.full_like(src, 9.0), pad), dev(want, pad), dev(label, pad), mode, ignore, 0.125)
        assert_bits(host(g), w)


@pytest.mark.parametrize("k,d,n", [(13, 9, 40), (64, 1024, 5000), (1000, 256, 300), (7, 4, 1)])
def test_index_fill_keeps_the_last_entry(lib, k, d, n):
    rng = np.random.default_rng(k + d + n)
    idx = rng.integers(0, k, n).astype(np.int32)
    src = rng.standard_normal((n, d)).astype(np.float32)
    t0 = rng.standard_normal((k, d)).astype(np.float32)
    want = orc.index_fill(t0.copy(), idx, src)
    got = lib.index_fill(dev(t0), dev(idx), dev(src))
    assert_bits(host(got), want)
    # entries outside the table are skipped, the rest behaves as before
    idx2 = idx.copy()
    idx2[::3] = np.where(np.arange(len(idx2[::3])) % 2 == 0, -1, k)
    keep = (idx2 >= 0) & (idx2 < k)
    want2 = orc.index_fill(t0.copy(), idx2[keep], np.ascontiguousarray(src[keep])) if keep.any() else t0
    got2 = lib.index_fill(dev(t0), dev(idx2), dev(src))
    assert_bits(host(got2), want2)


@pytest.mark.parametrize("n,nseg", [(1, 1), (200, 6), (70000, 300)])
def test_vectorized_sort(lib, n, nseg):
    rng = np.random.default_rng(n)
    seg = np.sort(rng.integers(0, nseg, size=n)).astype(np.int32)
    vals = (rng.integers(-40, 40, size=n) / 4.0).astype(np.float32)
    wv, ws = orc.vectorized_sort(vals.copy(), seg.copy())
    gv, gs = lib.vectorized_sort(dev(vals), dev(seg))
    assert_bits(host(gv), wv)
    assert np.array_equal(host(gs), ws)


@pytest.mark.parametrize("cid", range(cc.NUM_REMAP_CASES))
@pytest.mark.parametrize("shape", [(2, 3, 4, 5), (3, 8, 16, 64), (2, 5, 7, 33), (1, 4, 8, 128), (2, 2, 3, 1),
                                   (4, 12, 20, 24)])
def test_remap_expressions(lib, cid, shape):
    """Index-remapping expressions are data movement: bit-exact, on the 128-bit path (aligned
    widths and boundaries) and on the element path alike."""
    rng = np.random.default_rng(cid * 1000 + sum(shape))
    A = rng.uniform(-1, 1, shape).astype(np.float32)
    B = rng.uniform(-1, 1, shape).astype(np.float32)
    for p0, p1 in cc.remap_params(cid, shape):
        want = orc.remap_case(cid, A, B, p0, p1, fill=9.0)
        assert lib.remap_shape(cid, shape, p0, p1) == want.shape
        got = lib.remap_case(cid, torch.full(want.shape, 9.0, device="cuda"), dev(A), dev(B), p0, p1)
        assert_bits(host(got), want)


@pytest.mark.parametrize("cid", range(cc.NUM_SELECT_CASES))
@pytest.mark.parametrize("rows,cols", [(5, 7), (16, 64), (1, 1), (33, 12), (300, 1024), (257, 130)])
def test_select_expressions(lib, cid, rows, cols):
    """take / one_hot_encode / mat_choose_row_element / mat_fill_row_element / mask / upsampling_nearest /
    take_grad: bit-exact (take_grad adds in batch order on both sides)."""
    if cid == 6 and rows * cols > 40000:
        rows = 64  # the expression form walks the whole batch for every element
    rng = np.random.default_rng(cid * 1000 + rows + cols)
    A, B, ir, ic = cc.select_inputs(rng, rows, cols)
    for p0 in ((1, 2, 3) if cid == 5 else (1,)):
        want = orc.select_case(cid, A, B, ir, ic, p0)
        got = lib.select_case(cid, torch.full(want.shape, 9.0, device="cuda"), dev(A), dev(B), dev(ir), dev(ic), p0)
        assert_bits(host(got), want)


@pytest.mark.parametrize("case", cc.PATCH_CASES + [((4, 16, 28, 28), 3, 3, 1, 1, 1, 1), ((2, 8, 31, 33), 5, 5, 2, 2, 1, 1),
                                                   ((2, 3, 20, 20), 3, 3, 1, 1, 2, 2),
                                                   # planes large enough for the staged kernels: odd widths,
                                                   # strides that leave border pixels uncovered, dilation,
                                                   # and a plane that needs nearly all shared memory
                                                   ((2, 5, 28, 30), 5, 3, 2, 1, 1, 1), ((1, 4, 32, 32), 2, 2, 2, 2, 1, 1),
                                                   ((2, 2, 23, 29), 3, 3, 1, 2, 2, 2), ((3, 2, 41, 20), 4, 4, 3, 3, 1, 1),
                                                   ((2, 3, 24, 24), 1, 1, 1, 1, 1, 1), ((1, 2, 224, 224), 7, 7, 2, 2, 1, 1),
                                                   ((1, 1, 250, 250), 3, 3, 1, 1, 1, 1)])
def test_patch_conversions(lib, case):
    """unpack_patch2col is data movement (bit-exact); pack_col2patch adds the covering patches in the
    reference's order (bit-exact as well)."""
    shape, psy, psx, sy, sx, dy, dx = case
    rng = np.random.default_rng(sum(shape) + psy * 7 + sx)
    img = rng.uniform(-1, 1, shape).astype(np.float32)
    want = orc.unpack_patch2col(img, psy, psx, sy, sx, dy, dx)
    got = lib.unpack_patch2col(torch.full(want.shape, 9.0, device="cuda"), dev(img), psy, psx, sy, sx, dy, dx)
    assert_bits(host(got), want)
    grad = rng.uniform(-1, 1, want.shape).astype(np.float32)
    want_img = orc.pack_col2patch(grad, shape, psy, psx, sy, sx, dy, dx)
    got_img = lib.pack_col2patch(torch.full(shape, 9.0, device="cuda"), dev(grad), psy, psx, sy, sx, dy, dx)
    assert_bits(host(got_img), want_img)


@pytest.mark.parametrize("cid", range(cc.NUM_AXIS_CASES))
@pytest.mark.parametrize("shape", [(2, 3, 4, 5), (3, 8, 16, 64), (2, 5, 7, 33), (1, 4, 8, 128), (2, 2, 3, 1),
                                   (4, 12, 20, 24)])
def test_axis_expressions(lib, cid, shape):
    """range / slice(begin, end) / reduce_with_axis / reduce_keepdim / broadcast_with_axis / broadcast_keepdim /
    broadcast_to / broadcast_multi_axes: bit-exact (the reductions add along their axis in order on both sides)."""
    rng = np.random.default_rng(cid * 1000 + sum(shape))
    A = rng.uniform(-1, 1, shape).astype(np.float32)
    if cid == 5:
        A[0, 0] = A[-1, -1]  # ties: the reported position must be the reference's
    for p0, p1 in cc.axis_params(cid, shape):
        want = orc.axis_case(cid, A, p0, p1)
        assert lib.axis_shape(cid, shape, p0, p1) == want.shape
        got = lib.axis_case(cid, torch.full(want.shape, 9.0, device="cuda"), dev(A), p0, p1)
        assert_bits(host(got), want)


@pytest.mark.parametrize("cid", range(cc.NUM_COMPLEX_CASES))
@pytest.mark.parametrize("rows,cols", [(3, 4), (5, 16), (7, 36), (64, 1024), (33, 260)])
def test_complex_expressions(lib, cid, rows, cols):
    """complex_mul / complex_div in their cc, cr, rc forms, conj, exchange, pad_imag, toreal, abs_square,
    sum_real_imag: every product, sum and quotient rounded on its own, so bit-exact."""
    rng = np.random.default_rng(cid * 1000 + rows + cols)
    A = rng.uniform(-1, 1, (rows, cols)).astype(np.float32)
    B = rng.uniform(-1, 1, (rows, cols)).astype(np.float32)
    want = orc.complex_case(cid, A, B)
    got = lib.complex_case(cid, torch.full(want.shape, 9.0, device="cuda"), dev(A), dev(B))
    assert_bits(host(got), want)


def test_results_do_not_depend_on_the_run(lib):
    """No atomics and no arrival-order folds anywhere: floating-point sums are bit-identical from run
    to run (cluster and chunk partials are always combined in index order), also while other kernels
    share the GPU."""
    g = torch.Generator(device="cuda").manual_seed(3)
    M = torch.randn(20000, 1536, device="cuda", generator=g)
    T4 = torch.randn(96, 40, 28, 28, device="cuda", generator=g)
    L = torch.randn(300, 32000, device="cuda", generator=g)
    k, d, n = 5000, 512, 60000
    idx = (torch.rand(n, device="cuda", generator=g) ** 3 * k).to(torch.int32)  # skewed: long runs of hot rows
    src = torch.randn(n, d, device="cuda", generator=g)

    def once():
        out = [lib.reduce_keep_lowest(torch.zeros(1536, device="cuda"), M),
               lib.reduce_keep_highdim(torch.zeros(40, device="cuda"), T4),
               lib.softmax(torch.empty_like(L), L),
               lib.addtakegrad(torch.zeros(k, d, device="cuda"), idx, src)]
        return [host(t) for t in out]

    first = once()
    noise = torch.randn(4096, 4096, device="cuda")
    for _ in range(3):
        noise = noise * 1.0001  # unrelated work in flight changes the scheduling of the next kernels
        for a, b in zip(first, once()):
            assert_bits(a, b)


def test_a_wait_that_nothing_signals_gives_up_and_is_reported(lib):
    """The failure path behind every device-side wait: a bounded wait on a barrier that nothing signals
    runs out, marks the status word, the next stream wait reports MSB_ERR_TIMEOUT (6), the mark is
    cleared and the device keeps working.  No fault, trap or endless loop is involved."""
    import time
    assert lib.status("msb_selftest_bounded_wait", 0, None)[0] == 1      # limit outside 1..1000
    t0 = time.time()
    assert lib.status("msb_selftest_bounded_wait", 30, None)[0] == 0
    st, msg = lib.status("msb_stream_wait", None)
    assert st == 6 and "bounded wait" in msg
    assert time.time() - t0 < 5.0                                         # the wait ended near its 30 ms limit
    assert lib.status("msb_stream_wait", None)[0] == 0                   # reported once
    x = torch.arange(12, dtype=torch.float32, device="cuda").reshape(3, 4)
    got = lib.reduce_keep_lowest(torch.zeros(4, device="cuda"), x)
    lib.stream_wait(None)
    assert np.array_equal(host(got), host(x).sum(0))


def test_axis_argument_errors(lib):
    import ctypes as C
    z = torch.zeros(2, 3, 4, 5, device="cuda")
    p = C.c_void_p(z.data_ptr())
    assert lib.status("msb_axis_case_f32", 4, p, p, 2, 3, 4, 5, 4, 0, None)[0] == 2    # no such axis
    assert lib.status("msb_axis_case_f32", 0, p, p, 2, 3, 4, 5, 0, 0, None)[0] == 2    # an empty range
    assert lib.status("msb_axis_case_f32", 11, p, p, 2, 3, 4, 5, 0, 1, None)[0] == 1   # no such case


def test_remap_argument_errors(lib):
    import ctypes as C
    z = torch.zeros(2, 3, 4, 5, device="cuda")
    p = C.c_void_p(z.data_ptr())
    st, msg = lib.status("msb_remap_case_f32", 1, p, p, p, 2, 3, 4, 5, 2, 9, None)   # slice beyond the channels
    assert st == 2 and "slice" in msg.lower()
    st, msg = lib.status("msb_remap_case_f32", 10, p, p, p, 2, 3, 4, 5, 7, 2, None)  # crop taller than the image
    assert st == 2 and "height" in msg
    st, _ = lib.status("msb_remap_case_f32", 99, p, p, p, 2, 3, 4, 5, 0, 0, None)
    assert st == 1


def test_errors_are_status_codes(lib):
    import ctypes as C
    z = torch.zeros(4, 4, device="cuda")
    st, msg = lib.status("msb_softmax_f32", C.c_void_p(z.data_ptr()), C.c_void_p(z.data_ptr()), 4, 4, 2, 4, None)
    assert st == 2 and "extent" in msg
    st, _ = lib.status("msb_reduce_keep_lowest_f32", C.c_void_p(z.data_ptr()), C.c_void_p(z.data_ptr()), 0, 4, 4,
                       C.c_float(1.0), 0, 0, None)
    assert st == 2
    st, _ = lib.status("msb_pool_f32", C.c_void_p(z.data_ptr()), C.c_void_p(z.data_ptr()), 1, 2, 2, 3, 3, 1, 1, 2, 1,
                       1, None)
    assert st == 2
    st, _ = lib.status("msb_expr_case_f32", 99, None, None, None, None, None, 1, 1, 1, 1, 1, 1, None)
    assert st == 1
    # empty inputs are accepted and do nothing
    lib.softmax(torch.zeros(0, 8, device="cuda"), torch.zeros(0, 8, device="cuda"))
    lib.addtakegrad_largebatch(z, torch.zeros(0, dtype=torch.int32, device="cuda"),
                               torch.zeros(0, dtype=torch.int32, device="cuda"), torch.zeros(0, 4, device="cuda"))
    lib.stream_wait(None)


def test_memory_and_streams(lib):
    p, ld = lib.alloc_space(10, 100, 4, True)
    assert ld >= 100 and ld % 4 == 0
    q, ld2 = lib.alloc_space(10, 27, 4, True)
    assert ld2 == 27  # narrow rows are never pitched
    hbuf = lib.alloc_host(4000)
    s = lib.stream_create()
    import ctypes as C
    src = (C.c_float * 1000).from_address(hbuf)
    for i in range(1000):
        src[i] = float(i)
    lib.copy_2d(p, ld, hbuf, 100, 10, 100, 1, stream=s)
    out = torch.zeros(10, 100, device="cuda")
    lib.copy_2d(out, 100, p, ld, 10, 100, 3, stream=s)
    lib.stream_wait(s)
    assert np.array_equal(host(out).ravel(), np.arange(1000, dtype=np.float32))
    lib.stream_destroy(s)
    lib.free_host(hbuf)
    lib.free_space(p)
    lib.free_space(q)


def test_workspace_survives_operators_on_the_same_stream(lib):
    """The buffer msb_workspace hands out belongs to the caller: a column sum large enough to park
    partial rows in the engine's own scratch (and, the first time, to allocate that scratch) on the
    same stream must neither overwrite nor move it."""
    s = lib.stream_create()
    n = 1 << 16
    w = lib.workspace(4 * n, stream=s)
    assert w and lib.workspace(4 * n, stream=s) == w and lib.workspace(64, stream=s) == w
    pattern = torch.arange(n, dtype=torch.float32, device="cuda")
    lib.copy_2d(w, n, pattern, n, 1, n, 3, stream=s)
    rng = np.random.default_rng(12)
    M = rng.integers(-8, 9, (40000, 2048)).astype(np.float32)  # small integers: every sum is exact
    got = lib.reduce_keep_lowest(torch.zeros(2048, device="cuda"), dev(M), stream=s)
    idx = rng.integers(0, 300, 5000).astype(np.int32)
    lib.addtakegrad(torch.zeros(300, 64, device="cuda"), dev(idx), dev(rng.standard_normal((5000, 64)).astype(np.float32)),
                    stream=s)
    back = torch.zeros(n, device="cuda")
    lib.copy_2d(back, n, w, n, 1, n, 3, stream=s)
    lib.stream_wait(s)
    assert torch.equal(back, pattern)
    assert_bits(host(got), M.sum(axis=0, dtype=np.float64).astype(np.float32))
    assert lib.workspace(4 * n, stream=s) == w
    lib.stream_destroy(s)
