"""ctypes bindings for the two CPU checkers under oracle/ (test infrastructure).

`load("orc")` binds oracle/liboracle.so (the plain-C restatement); `load("ref")` binds
oracle/_ref/libmshadow_ref.so (the unmodified reference headers behind a C shim) and
returns None when that file has not been built.  Both expose the same numpy-level API,
so a test can run the same call against either one.
"""
import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PATHS = {
    "orc": os.path.join(ROOT, "oracle", "liboracle.so"),
    "ref": os.path.join(ROOT, "oracle", "_ref", "libmshadow_ref.so"),
}

_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int32)
i64 = C.c_int64


def _fp(a):
    assert a.dtype == np.float32
    return a.ctypes.data_as(_f32p)


def _ip(a):
    assert a.dtype == np.int32 and a.flags.c_contiguous
    return a.ctypes.data_as(_i32p)


def _ld(a):
    """Leading dimension (elements) of a 2-D+ array whose last axis is dense."""
    assert a.strides[-1] == 4
    return a.strides[-2] // 4 if a.ndim >= 2 else a.shape[0]


class Checker:
    def __init__(self, kind):
        self.kind = kind
        self.lib = C.CDLL(PATHS[kind])
        self.p = kind + "_"
        self.lib[self.p + "num_threads"].restype = C.c_int

    def _fn(self, name):
        f = self.lib[self.p + name]
        f.restype = None
        return f

    def num_threads(self):
        return int(self.lib[self.p + "num_threads"]())

    def set_num_threads(self, n):
        """OpenMP threads of later calls; overrides an OMP_NUM_THREADS that a launcher exported."""
        f = self.lib[self.p + "set_num_threads"]
        f.restype = None
        f(C.c_int(int(n)))
        return self.num_threads()

    # ---- elementwise -------------------------------------------------------------
    def expr_case(self, cid, dst, A, B, Cm, bias):
        rows, cols = dst.shape
        self._fn("expr_case")(C.c_int(cid), _fp(dst), _fp(A), _fp(B), _fp(Cm), _fp(bias),
                              i64(rows), i64(cols), i64(_ld(dst)), i64(_ld(A)), i64(_ld(B)),
                              i64(_ld(Cm)))
        return dst

    # ---- reductions --------------------------------------------------------------
    def reduce_keep_lowest(self, dst, src, scale=1.0, saver=0, reducer=0):
        rows, cols = src.shape
        self._fn("reduce_keep_lowest")(_fp(dst), _fp(src), i64(rows), i64(cols), i64(_ld(src)),
                                       C.c_float(scale), C.c_int(saver), C.c_int(reducer))
        return dst

    def reduce_keep_highdim(self, dst, src, scale=1.0, saver=0, reducer=0):
        n, c, h, w = src.shape
        self._fn("reduce_keep_highdim")(_fp(dst), _fp(src), i64(n), i64(c), i64(h), i64(w),
                                        i64(_ld(src)), C.c_float(scale), C.c_int(saver),
                                        C.c_int(reducer))
        return dst

    # ---- softmax -----------------------------------------------------------------
    def softmax(self, dst, src):
        rows, cols = src.shape
        self._fn("softmax")(_fp(dst), _fp(src), i64(rows), i64(cols), i64(_ld(dst)),
                            i64(_ld(src)))
        return dst

    def softmax_grad(self, dst, src, label, mode=0, ignore_label=0.0, alpha=0.0):
        rows, cols = src.shape
        self._fn("softmax_grad")(_fp(dst), _fp(src), _fp(label), i64(rows), i64(cols),
                                 i64(_ld(dst)), i64(_ld(src)), C.c_int(mode),
                                 C.c_float(ignore_label), C.c_float(alpha))
        return dst

    # ---- pooling -----------------------------------------------------------------
    def pool(self, dst, src, ky, kx, sy, sx, reducer=1):
        planes, h, w = src.shape
        self._fn("pool")(_fp(dst), _fp(src), i64(planes), i64(h), i64(w), C.c_int(ky),
                         C.c_int(kx), C.c_int(sy), C.c_int(sx), i64(_ld(src)), i64(_ld(dst)),
                         C.c_int(reducer))
        return dst

    def unpool(self, dst, src, pooled, gpooled, ky, kx, sy, sx, reducer=1):
        planes, h, w = src.shape
        _, ph, pw = pooled.shape
        assert _ld(pooled) == _ld(gpooled)
        self._fn("unpool")(_fp(dst), _fp(src), _fp(pooled), _fp(gpooled), i64(planes), i64(h),
                           i64(w), i64(ph), i64(pw), C.c_int(ky), C.c_int(kx), C.c_int(sy),
                           C.c_int(sx), i64(_ld(src)), i64(_ld(pooled)), i64(_ld(dst)),
                           C.c_int(reducer))
        return dst

    def chpool(self, dst, src, nsize, stride=1, pad=None, reducer=0):
        n, c, h, w = src.shape
        pad = nsize // 2 if pad is None else pad
        self._fn("chpool")(_fp(dst), _fp(src), i64(n), i64(c), i64(h), i64(w), C.c_int(nsize),
                           C.c_int(stride), C.c_int(pad), i64(_ld(src)), i64(_ld(dst)),
                           C.c_int(reducer))
        return dst

    def ch_unpool(self, dst, src, pooled, gpooled, nsize, stride=1, pad=None, reducer=0):
        n, c, h, w = src.shape
        pc = pooled.shape[1]
        pad = nsize // 2 if pad is None else pad
        assert _ld(pooled) == _ld(gpooled)
        self._fn("ch_unpool")(_fp(dst), _fp(src), _fp(pooled), _fp(gpooled), i64(n), i64(c), i64(pc), i64(h),
                              i64(w), C.c_int(nsize), C.c_int(stride), C.c_int(pad), i64(_ld(src)),
                              i64(_ld(pooled)), i64(_ld(dst)), C.c_int(reducer))
        return dst

    # ---- local response normalisation (chpool<sum> with its surrounding arithmetic) ------------
    def lrn_forward(self, src, nsize, salpha, beta, knorm, power_kind=0):
        """Returns (out, norm) for a dense (n, c, h, w) input."""
        assert src.flags.c_contiguous
        n, c, h, w = src.shape
        out, norm = np.empty_like(src), np.empty_like(src)
        self._fn("lrn_forward")(_fp(out), _fp(norm), _fp(src), i64(n), i64(c), i64(h), i64(w), C.c_int(nsize),
                                C.c_float(salpha), C.c_float(beta), C.c_float(knorm), C.c_int(power_kind))
        return out, norm

    def lrn_backward(self, gout, src, norm, nsize, salpha, beta, power_kind=0):
        assert src.flags.c_contiguous and gout.flags.c_contiguous and norm.flags.c_contiguous
        n, c, h, w = src.shape
        gsrc = np.empty_like(src)
        self._fn("lrn_backward")(_fp(gsrc), _fp(gout), _fp(src), _fp(norm), i64(n), i64(c), i64(h), i64(w),
                                 C.c_int(nsize), C.c_float(salpha), C.c_float(beta), C.c_int(power_kind))
        return gsrc

    # ---- embedding backward ------------------------------------------------------
    def addtakegrad(self, dst, index, src):
        k, d = dst.shape
        self._fn("addtakegrad")(_fp(dst), _ip(index), _fp(src), i64(k), i64(d),
                                i64(index.shape[0]), i64(_ld(dst)), i64(_ld(src)))
        return dst

    def addtakegrad_largebatch(self, dst, sorted_, index, src):
        k, d = dst.shape
        assert dst.flags.c_contiguous and src.flags.c_contiguous
        self._fn("addtakegrad_largebatch")(_fp(dst), _ip(sorted_), _ip(index), _fp(src), i64(k),
                                           i64(d), i64(index.shape[0]))
        return dst

    def sort_by_key(self, keys, values, ascend=True):
        self._fn("sort_by_key")(_ip(keys), _ip(values), i64(keys.shape[0]),
                                C.c_int(1 if ascend else 0))
        return keys, values

    # ---- softmax over the middle axis, IndexFill, VectorizedSort -------------------
    def softmax3d(self, dst, src):
        batch, classes, npos = src.shape
        self._fn("softmax3d")(_fp(dst), _fp(src), i64(batch), i64(classes), i64(npos), i64(_ld(dst)),
                              i64(_ld(src)))
        return dst

    def softmax_grad3d(self, dst, src, label, mode=0, ignore_label=0.0, alpha=0.0):
        batch, classes, npos = src.shape
        self._fn("softmax_grad3d")(_fp(dst), _fp(src), _fp(label), i64(batch), i64(classes), i64(npos),
                                   i64(_ld(dst)), i64(_ld(src)), i64(_ld(label)), C.c_int(mode),
                                   C.c_float(ignore_label), C.c_float(alpha))
        return dst

    def index_fill(self, dst, index, src):
        self._fn("index_fill")(_fp(dst), _ip(index), _fp(src), i64(src.shape[1]), i64(index.shape[0]),
                               i64(_ld(dst)), i64(_ld(src)))
        return dst

    def remap_shape(self, cid, shape, p0=0, p1=0):
        out = (i64 * 4)()
        n, c, h, w = shape
        self._fn("remap_shape")(C.c_int(cid), i64(n), i64(c), i64(h), i64(w), i64(p0), i64(p1), out)
        return tuple(int(v) for v in out)

    def remap_case(self, cid, A, B, p0=0, p1=0, fill=0.0):
        """Evaluates index-remapping case `cid` on dense (n, c, h, w) inputs; returns the result."""
        assert A.flags.c_contiguous and B.flags.c_contiguous and A.shape == B.shape
        n, c, h, w = A.shape
        dst = np.full(self.remap_shape(cid, A.shape, p0, p1), np.float32(fill), dtype=np.float32)
        self._fn("remap_case")(C.c_int(cid), _fp(dst), _fp(A), _fp(B), i64(n), i64(c), i64(h), i64(w), i64(p0),
                               i64(p1))
        return dst

    def axis_shape(self, cid, shape, p0=0, p1=1):
        out = (i64 * 4)()
        n, c, h, w = shape
        fn = self._fn("axis_shape")
        fn.restype = C.c_int
        ndim = fn(C.c_int(cid), i64(n), i64(c), i64(h), i64(w), i64(p0), i64(p1), out)
        return tuple(int(v) for v in out[:ndim])

    def axis_case(self, cid, A, p0=0, p1=1):
        """Evaluates axis/box-addressed case `cid` on a dense (n, c, h, w) input; returns the result."""
        assert A.flags.c_contiguous
        n, c, h, w = A.shape
        dst = np.full(self.axis_shape(cid, A.shape, p0, p1), np.float32(9.0), dtype=np.float32)
        self._fn("axis_case")(C.c_int(cid), _fp(dst), _fp(A), i64(n), i64(c), i64(h), i64(w), i64(p0), i64(p1))
        return dst

    def complex_case(self, cid, A, B):
        """Evaluates complex-arithmetic case `cid` on dense (rows, cols) inputs (re, im interleaved)."""
        assert A.flags.c_contiguous and B.flags.c_contiguous and A.shape == B.shape and A.shape[1] % 4 == 0
        rows, cols = A.shape
        dst = np.full((rows, cols // 2 if 9 <= cid <= 11 else cols), np.float32(9.0), dtype=np.float32)
        self._fn("complex_case")(C.c_int(cid), _fp(dst), _fp(A), _fp(B), i64(rows), i64(cols))
        return dst

    def select_case(self, cid, A, B, idx_r, idx_c, p0=1):
        """Evaluates index-selecting case `cid` on dense (rows, cols) inputs; returns the result."""
        rows, cols = A.shape
        dst = np.full(select_shape(cid, rows, cols, p0), np.float32(9.0), dtype=np.float32)
        self._fn("select_case")(C.c_int(cid), _fp(dst), _fp(A), _fp(B), _fp(idx_r), _fp(idx_c), i64(rows), i64(cols),
                                i64(p0))
        return dst

    def unpack_patch2col(self, img, psy, psx, sy, sx, dy=1, dx=1):
        n, c, h, w = img.shape
        mat = np.full(patch_matrix_shape(img.shape, psy, psx, sy, sx, dy, dx), np.float32(9.0), np.float32)
        self._fn("unpack_patch2col")(_fp(mat), _fp(img), i64(n), i64(c), i64(h), i64(w), C.c_int(psy), C.c_int(psx),
                                     C.c_int(sy), C.c_int(sx), C.c_int(dy), C.c_int(dx))
        return mat

    def pack_col2patch(self, mat, imshape, psy, psx, sy, sx, dy=1, dx=1):
        n, c, h, w = imshape
        assert mat.shape == patch_matrix_shape(imshape, psy, psx, sy, sx, dy, dx) and mat.flags.c_contiguous
        img = np.full(imshape, np.float32(9.0), np.float32)
        self._fn("pack_col2patch")(_fp(img), _fp(mat), i64(n), i64(c), i64(h), i64(w), C.c_int(psy), C.c_int(psx),
                                   C.c_int(sy), C.c_int(sx), C.c_int(dy), C.c_int(dx))
        return img

    def vectorized_sort(self, values, segments):
        assert values.flags.c_contiguous
        self._fn("vectorized_sort")(_fp(values), _ip(segments), i64(values.shape[0]))
        return values, segments


NUM_REMAP_CASES = 17
NUM_SELECT_CASES = 8


def patch_matrix_shape(imshape, psy, psx, sy, sx, dy=1, dx=1):
    """Shape of unpack_patch2col's result for an (n, c, h, w) image."""
    n, c, h, w = imshape
    oh = (h - (dy * (psy - 1) + 1)) // sy + 1
    ow = (w - (dx * (psx - 1) + 1)) // sx + 1
    return (psy * psx * c, oh * ow * n)


# (image shape, patch y, patch x, stride y, stride x, dilate y, dilate x)
PATCH_CASES = [((2, 3, 6, 6), 3, 3, 1, 1, 1, 1), ((1, 2, 7, 9), 3, 2, 2, 1, 1, 1), ((2, 1, 8, 8), 2, 2, 2, 2, 1, 1),
               ((1, 3, 9, 11), 3, 3, 1, 2, 2, 2), ((2, 2, 5, 5), 5, 5, 1, 1, 1, 1), ((1, 1, 10, 7), 2, 3, 3, 2, 2, 1),
               ((3, 4, 12, 16), 3, 3, 2, 2, 1, 1)]


def select_shape(cid, rows, cols, p0=1):
    """Result shape of index-selecting case `cid` (see oracle.h)."""
    if cid == 2:
        return (rows,)
    if cid == 5:
        return (rows * p0, cols * p0)
    return (rows, cols)


def select_inputs(rng, rows, cols):
    """(A, B, idx_r, idx_c): matrices and index vectors (integers stored as floats, with repeats)."""
    A = rng.uniform(-1, 1, (rows, cols)).astype(np.float32)
    B = rng.uniform(-1, 1, (rows, cols)).astype(np.float32)
    idx_r = rng.integers(0, rows, rows).astype(np.float32)
    idx_c = rng.integers(0, cols, rows).astype(np.float32)
    return A, B, idx_r, idx_c


def remap_params(cid, shape):
    """Valid (p0, p1) pairs for index-remapping case `cid` on an (n, c, h, w) input: ranges that
    touch the borders, unaligned and 4-aligned boundaries."""
    n, c, h, w = shape
    if cid in (1, 14):
        cand = {(0, c), (1, c), (0, max(1, c - 1)), (c // 2, c), (min(4, c - 1), c)}
        return sorted(p for p in cand if p[0] < p[1])
    if cid == 2:
        cand = {(0, w), (1, w), (0, max(1, w - 1)), (min(4, w - 1), w), (w // 2, w)}
        return sorted(p for p in cand if p[0] < p[1])
    if cid in (9, 16):
        return [(0, 0), (1, 2), (2, 4), (3, 0)]
    if cid in (10, 11):
        return sorted({(h, w), (1, 1), (max(1, h - 2), max(1, w - 8)), (max(1, h - 1), max(1, w - 3))})
    return [(0, 0)]


NUM_AXIS_CASES = 11
NUM_COMPLEX_CASES = 13


def axis_params(cid, shape):
    """Valid (p0, p1) pairs for axis/box-addressed case `cid` on an (n, c, h, w) input."""
    n, c, h, w = shape
    if cid in (0, 1):
        return [(0, 1), (3, 7), (-5, 12), (100, 64)]
    if cid in (2, 3):
        return [(0, 0), (1, 1), (2, 4), (5, 3)]
    if cid in (4, 5, 6):
        return [(axis, 0) for axis in range(4)]
    if cid == 7:
        return [(axis, size) for axis in range(4) for size in (1, 3)]
    if cid == 8:
        return [(0, 1), (0, 4), (0, 7)]
    return [(1, 1), (2, 3), (4, 4), (3, 1), (1, 5)]


_cache = {}


def load(kind):
    if kind not in _cache:
        _cache[kind] = Checker(kind) if os.path.exists(PATHS[kind]) else None
    return _cache[kind]


def pool_out(h, k, s):
    return (h - k) // s + 1


def pitched(rng_array, pad):
    """Return a view of a copy of `rng_array` whose rows are `pad` elements apart wider."""
    shape = rng_array.shape
    buf = np.full(shape[:-1] + (shape[-1] + pad,), np.float32(7.5), dtype=np.float32)
    buf[..., : shape[-1]] = rng_array
    return buf[..., : shape[-1]]
