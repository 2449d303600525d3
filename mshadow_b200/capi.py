"""ctypes binding of the C ABI in include/mshadow_b200.h.

The shared library is the product; this module only marshals arguments.  Device memory is
passed as raw addresses, so any owner of CUDA memory works: the helpers below accept objects
with a ``data_ptr()`` method (torch tensors) and take shapes and strides from them.  There is
no host fallback: if the library is missing, loading raises; if a call fails, ``MsbError``
carries the library's own message.
"""
import ctypes as C
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmshadow_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "mshadow_b200.h")

STATUS_NAMES = {0: "MSB_OK", 1: "MSB_ERR_ARGUMENT", 2: "MSB_ERR_SHAPE", 3: "MSB_ERR_LAYOUT",
                4: "MSB_ERR_CUDA", 5: "MSB_ERR_MEMORY", 6: "MSB_ERR_TIMEOUT"}

SAVETO, PLUSTO, MINUSTO, MULTO, DIVTO = range(5)
RED_SUM, RED_MAX, RED_MIN = range(3)
H2D, D2H, D2D = 1, 2, 3


class MsbError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("%s: %s" % (STATUS_NAMES.get(status, status), message))
        self.status = status


def declared_symbols(header_path=HEADER_PATH):
    """Names of every function the C header declares."""
    text = open(header_path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(msb_[a-z0-9_]+)\s*\(", text)))


i64, f32, cint, vp = C.c_int64, C.c_float, C.c_int, C.c_void_p

_SIGNATURES = {
    "msb_init": [cint],
    "msb_set_device": [cint],
    "msb_shutdown": [],
    "msb_stream_create": [C.POINTER(vp)],
    "msb_stream_destroy": [vp],
    "msb_stream_wait": [vp],
    "msb_stream_idle": [vp, C.POINTER(cint)],
    "msb_selftest_bounded_wait": [cint, vp],
    "msb_alloc_space": [C.POINTER(vp), C.POINTER(i64), i64, i64, i64, cint],
    "msb_free_space": [vp],
    "msb_alloc_host": [C.POINTER(vp), i64],
    "msb_free_host": [vp],
    "msb_copy_2d": [vp, i64, vp, i64, i64, i64, i64, cint, vp],
    "msb_workspace": [vp, i64, C.POINTER(vp)],
    "msb_scratch_bytes": [vp, C.POINTER(i64), C.POINTER(i64)],
    "msb_expr_case_f32": [cint, vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, vp],
    "msb_reduce_keep_lowest_f32": [vp, vp, i64, i64, i64, f32, cint, cint, vp],
    "msb_reduce_keep_lowest_sum_f32_noalloc": [vp, vp, i64, i64, i64, f32, vp],
    "msb_reduce_keep_highdim_f32": [vp, vp, i64, i64, i64, i64, i64, f32, cint, cint, vp],
    "msb_reduce_keep_lowest_f32_sink": [vp, vp, i64, i64, i64, f32, cint, cint, vp, vp],
    "msb_reduce_keep_highdim_f32_sink": [vp, vp, i64, i64, i64, i64, i64, f32, cint, cint, vp, vp],
    "msb_softmax_f32": [vp, vp, i64, i64, i64, i64, vp],
    "msb_softmax_grad_f32": [vp, vp, vp, i64, i64, i64, i64, cint, f32, f32, vp],
    "msb_softmax_grad_fused_f32": [vp, vp, vp, i64, i64, i64, i64, vp],
    "msb_pool_f32": [vp, vp, i64, i64, i64, cint, cint, cint, cint, i64, i64, cint, vp],
    "msb_unpool_f32": [vp, vp, vp, vp, i64, i64, i64, i64, i64, cint, cint, cint, cint, i64, i64, i64,
                       cint, vp],
    "msb_chpool_f32": [vp, vp, i64, i64, i64, i64, cint, cint, cint, i64, i64, cint, vp],
    "msb_ch_unpool_f32": [vp, vp, vp, vp, i64, i64, i64, i64, i64, cint, cint, cint, i64, i64, i64, cint, vp],
    "msb_lrn_forward_f32": [vp, vp, vp, i64, i64, i64, i64, cint, f32, f32, f32, cint, vp],
    "msb_lrn_backward_f32": [vp, vp, vp, vp, i64, i64, i64, i64, cint, f32, f32, cint, vp],
    "msb_addtakegrad_f32_i32": [vp, vp, vp, i64, i64, i64, i64, i64, vp],
    "msb_addtakegrad_largebatch_f32_i32": [vp, vp, vp, vp, i64, i64, i64, vp],
    "msb_sort_by_key_i32": [vp, vp, i64, cint, vp],
    "msb_sort_by_key_lowbits_i32": [vp, vp, i64, cint, vp],
    "msb_vectorized_sort_f32_i32": [vp, vp, i64, vp],
    "msb_frequent_rows_i32": [vp, vp, vp, i64, i64, vp],
    "msb_run_index_i32": [vp, vp, vp, vp, i64, vp],
    "msb_run_bounds_i32": [vp, vp, vp, cint, i64, vp],
    "msb_run_keys_to_owners_i32": [vp, vp, vp, i64, cint, i64, vp],
    "msb_take_sum_to_owners_f32_i32": [vp, vp, vp, vp, vp, i64, i64, cint, vp],
    "msb_route_cyclic_hot_i32": [vp, vp, vp, vp, vp, i64, vp, i64, cint, cint, i64, i64, i64, vp],
    "msb_index_fill_f32_i32": [vp, vp, vp, i64, i64, i64, vp],
    "msb_remap_shape": [cint, i64, i64, i64, i64, i64, i64, vp],
    "msb_complex_case_f32": [cint, vp, vp, vp, i64, i64, vp],
    "msb_axis_shape": [cint, i64, i64, i64, i64, i64, i64, vp, vp],
    "msb_axis_case_f32": [cint, vp, vp, i64, i64, i64, i64, i64, i64, vp],
    "msb_remap_case_f32": [cint, vp, vp, vp, i64, i64, i64, i64, i64, i64, vp],
    "msb_select_case_f32": [cint, vp, vp, vp, vp, vp, i64, i64, i64, vp],
    "msb_unpack_patch2col_f32": [vp, vp, i64, i64, i64, i64, cint, cint, cint, cint, cint, cint, vp],
    "msb_pack_col2patch_f32": [vp, vp, i64, i64, i64, i64, cint, cint, cint, cint, cint, cint, vp],
    "msb_softmax3d_f32": [vp, vp, i64, i64, i64, i64, i64, vp],
    "msb_softmax_grad3d_f32": [vp, vp, vp, i64, i64, i64, i64, i64, i64, cint, f32, f32, vp],
}


def _ptr(t):
    return vp(t.data_ptr() if hasattr(t, "data_ptr") else int(t))


def _ld(t):
    """Leading dimension in elements: distance between consecutive rows of the last axis."""
    assert t.stride(-1) == 1 or t.shape[-1] <= 1, "last axis must be dense"
    if t.dim() < 2:
        return t.shape[0]
    return t.stride(-2)


class Library:
    """The loaded shared object with typed entry points and status checking."""

    def __init__(self, path=LIB_PATH):
        if not os.path.exists(path):
            raise FileNotFoundError(
                "%s not found: build it with `python -c 'import __graft_entry__ as g; g.build()'`; "
                "there is no fallback implementation" % path)
        self.path = path
        self.dll = C.CDLL(path)
        self.dll.msb_last_error.restype = C.c_char_p
        self.dll.msb_version.restype = cint
        self.dll.msb_launch_count.restype = i64
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(self.dll, name)
            fn.argtypes = argtypes
            fn.restype = cint

    def call(self, name, *args):
        status = getattr(self.dll, name)(*args)
        if status != 0:
            raise MsbError(status, self.dll.msb_last_error().decode("utf-8", "replace"))

    def status(self, name, *args):
        """Raw status code without raising (for tests of error behaviour)."""
        return getattr(self.dll, name)(*args), self.dll.msb_last_error().decode("utf-8", "replace")

    # ---- engine ---------------------------------------------------------------------
    def launch_count(self):
        return int(self.dll.msb_launch_count())

    def init(self, device=0):
        self.call("msb_init", device)

    def shutdown(self):
        self.call("msb_shutdown")

    def stream_create(self):
        s = vp()
        self.call("msb_stream_create", C.byref(s))
        return s

    def stream_destroy(self, s):
        self.call("msb_stream_destroy", s)

    def stream_wait(self, s=None):
        self.call("msb_stream_wait", s)

    def alloc_space(self, rows, cols, elem_size=4, pad=True):
        p, ld = vp(), i64()
        self.call("msb_alloc_space", C.byref(p), C.byref(ld), rows, cols, elem_size, int(pad))
        return p.value, ld.value

    def free_space(self, p):
        self.call("msb_free_space", vp(p))

    def alloc_host(self, nbytes):
        p = vp()
        self.call("msb_alloc_host", C.byref(p), nbytes)
        return p.value

    def free_host(self, p):
        self.call("msb_free_host", vp(p))

    def workspace(self, nbytes, stream=None):
        """Device address of the caller's scratch buffer of `stream` (at least `nbytes`)."""
        p = vp()
        self.call("msb_workspace", stream, nbytes, C.byref(p))
        return p.value

    def scratch_bytes(self, stream=None):
        """(engine, caller): bytes the library holds for `stream` as internal scratch and as workspace."""
        a, b = i64(), i64()
        self.call("msb_scratch_bytes", stream, C.byref(a), C.byref(b))
        return a.value, b.value

    def copy_2d(self, dst, ld_dst, src, ld_src, rows, cols, kind, elem_size=4, stream=None):
        self.call("msb_copy_2d", _ptr(dst), ld_dst, _ptr(src), ld_src, rows, cols, elem_size, kind, stream)

    # ---- operators (tensor-like arguments) ---------------------------------------------
    def expr_case(self, cid, dst, A, B, Cm, bias, stream=None):
        rows, cols = dst.shape
        self.call("msb_expr_case_f32", cid, _ptr(dst), _ptr(A), _ptr(B), _ptr(Cm), _ptr(bias), rows, cols,
                  _ld(dst), _ld(A), _ld(B), _ld(Cm), stream)
        return dst

    def reduce_keep_lowest(self, dst, src, scale=1.0, saver=0, reducer=0, stream=None, sink=None):
        """`sink`: a msb_peer_sink_t (ctypes structure) through which the results also reach the
        other GPUs of an exchange group."""
        rows, cols = src.shape
        if sink is not None:
            self.call("msb_reduce_keep_lowest_f32_sink", _ptr(dst), _ptr(src), rows, cols, _ld(src), scale, saver,
                      reducer, C.cast(C.pointer(sink), vp), stream)
            return dst
        self.call("msb_reduce_keep_lowest_f32", _ptr(dst), _ptr(src), rows, cols, _ld(src), scale, saver,
                  reducer, stream)
        return dst

    def reduce_keep_lowest_sum_noalloc(self, dst, src, scale=1.0, stream=None):
        """Column sum through the entry point that allocates nothing (fixed in-library scratch)."""
        rows, cols = src.shape
        self.call("msb_reduce_keep_lowest_sum_f32_noalloc", _ptr(dst), _ptr(src), rows, cols, _ld(src), scale,
                  stream)
        return dst

    def reduce_keep_highdim(self, dst, src, scale=1.0, saver=0, reducer=0, stream=None, sink=None):
        n, c, h, w = src.shape
        if sink is not None:
            self.call("msb_reduce_keep_highdim_f32_sink", _ptr(dst), _ptr(src), n, c, h, w, _ld(src), scale, saver,
                      reducer, C.cast(C.pointer(sink), vp), stream)
            return dst
        self.call("msb_reduce_keep_highdim_f32", _ptr(dst), _ptr(src), n, c, h, w, _ld(src), scale, saver,
                  reducer, stream)
        return dst

    def softmax(self, dst, src, stream=None):
        rows, cols = src.shape
        self.call("msb_softmax_f32", _ptr(dst), _ptr(src), rows, cols, _ld(dst), _ld(src), stream)
        return dst

    def softmax_grad(self, dst, src, label, mode=0, ignore_label=0.0, alpha=0.0, stream=None):
        rows, cols = src.shape
        self.call("msb_softmax_grad_f32", _ptr(dst), _ptr(src), _ptr(label), rows, cols, _ld(dst), _ld(src),
                  mode, ignore_label, alpha, stream)
        return dst

    def softmax_grad_fused(self, dst, logits, label, stream=None):
        rows, cols = logits.shape
        self.call("msb_softmax_grad_fused_f32", _ptr(dst), _ptr(logits), _ptr(label), rows, cols, _ld(dst),
                  _ld(logits), stream)
        return dst

    def pool(self, dst, src, ky, kx, sy, sx, reducer=1, stream=None):
        planes, h, w = src.shape
        self.call("msb_pool_f32", _ptr(dst), _ptr(src), planes, h, w, ky, kx, sy, sx, _ld(src), _ld(dst),
                  reducer, stream)
        return dst

    def unpool(self, dst, src, pooled, gpooled, ky, kx, sy, sx, reducer=1, stream=None):
        planes, h, w = src.shape
        _, ph, pw = pooled.shape
        assert _ld(pooled) == _ld(gpooled)
        self.call("msb_unpool_f32", _ptr(dst), _ptr(src), _ptr(pooled), _ptr(gpooled), planes, h, w, ph, pw,
                  ky, kx, sy, sx, _ld(src), _ld(pooled), _ld(dst), reducer, stream)
        return dst

    def chpool(self, dst, src, nsize, stride=1, pad=None, reducer=0, stream=None):
        n, c, h, w = src.shape
        pad = nsize // 2 if pad is None else pad
        self.call("msb_chpool_f32", _ptr(dst), _ptr(src), n, c, h, w, nsize, stride, pad, _ld(src), _ld(dst),
                  reducer, stream)
        return dst

    def ch_unpool(self, dst, src, pooled, gpooled, nsize, stride=1, pad=None, reducer=0, stream=None):
        n, c, h, w = src.shape
        pad = nsize // 2 if pad is None else pad
        assert _ld(pooled) == _ld(gpooled)
        self.call("msb_ch_unpool_f32", _ptr(dst), _ptr(src), _ptr(pooled), _ptr(gpooled), n, c, pooled.shape[1], h,
                  w, nsize, stride, pad, _ld(src), _ld(pooled), _ld(dst), reducer, stream)
        return dst

    def lrn_forward(self, out, norm, src, nsize, salpha, beta, knorm, power_kind=0, stream=None):
        """`norm` may be None (not kept)."""
        n, c, h, w = src.shape
        self.call("msb_lrn_forward_f32", _ptr(out), _ptr(norm) if norm is not None else None, _ptr(src), n, c, h, w,
                  nsize, salpha, beta, knorm, power_kind, stream)
        return out

    def lrn_backward(self, gsrc, gout, src, norm, nsize, salpha, beta, power_kind=0, stream=None):
        n, c, h, w = src.shape
        self.call("msb_lrn_backward_f32", _ptr(gsrc), _ptr(gout), _ptr(src), _ptr(norm), n, c, h, w, nsize, salpha,
                  beta, power_kind, stream)
        return gsrc

    def addtakegrad(self, dst, index, src, stream=None):
        k, d = dst.shape
        self.call("msb_addtakegrad_f32_i32", _ptr(dst), _ptr(index), _ptr(src), k, d, index.shape[0],
                  _ld(dst), _ld(src), stream)
        return dst

    def addtakegrad_largebatch(self, dst, sorted_, index, src, stream=None):
        k, d = dst.shape
        self.call("msb_addtakegrad_largebatch_f32_i32", _ptr(dst), _ptr(sorted_), _ptr(index), _ptr(src), k,
                  d, index.shape[0], stream)
        return dst

    def frequent_rows(self, rows_out, counts_out, sorted_, stream=None):
        self.call("msb_frequent_rows_i32", _ptr(rows_out), _ptr(counts_out), _ptr(sorted_), sorted_.shape[0],
                  rows_out.shape[0], stream)
        return rows_out, counts_out

    def run_index(self, run_of, run_keys, total, sorted_, stream=None):
        self.call("msb_run_index_i32", _ptr(run_of), _ptr(run_keys), _ptr(total), _ptr(sorted_), sorted_.shape[0], stream)
        return run_of, run_keys, total

    def run_bounds(self, first, run_keys, total, world, per_owner, stream=None):
        self.call("msb_run_bounds_i32", _ptr(first), _ptr(run_keys), _ptr(total), world, per_owner, stream)
        return first

    @staticmethod
    def _address_table(addresses):
        table = (C.c_void_p * len(addresses))(*[int(a) for a in addresses])
        return table

    def run_keys_to_owners(self, key_blocks, first, run_keys, world, per_owner, stream=None):
        """key_blocks: one device address per owner (ints; other GPUs' mapped memory allowed)."""
        self.call("msb_run_keys_to_owners_i32", self._address_table(key_blocks), _ptr(first), _ptr(run_keys),
                  run_keys.shape[0], world, per_owner, stream)

    def take_sum_to_owners(self, row_blocks, first, run_of, index, src, world, stream=None):
        """row_blocks: one device address per owner (ints; other GPUs' mapped memory allowed)."""
        self.call("msb_take_sum_to_owners_f32_i32", self._address_table(row_blocks), _ptr(first), _ptr(run_of),
                  _ptr(index), _ptr(src), src.shape[1], index.shape[0], world, stream)

    def route_cyclic_hot(self, keys_out, rows_out, totals, sorted_, index, hot, world, rank, src_begin, src_end,
                         hot_base, stream=None):
        self.call("msb_route_cyclic_hot_i32", _ptr(keys_out), _ptr(rows_out), _ptr(totals), _ptr(sorted_), _ptr(index),
                  sorted_.shape[0], _ptr(hot) if hot is not None else None, 0 if hot is None else hot.shape[0],
                  world, rank, src_begin, src_end, hot_base, stream)
        return keys_out, rows_out, totals

    def sort_by_key(self, keys, values, ascend=True, stream=None, bits=None):
        """bits: the keys are known to lie in [0, 2^bits) (ascending only): fewer passes."""
        if bits is not None:
            assert ascend
            self.call("msb_sort_by_key_lowbits_i32", _ptr(keys), _ptr(values), keys.shape[0], bits, stream)
        else:
            self.call("msb_sort_by_key_i32", _ptr(keys), _ptr(values), keys.shape[0], int(ascend), stream)
        return keys, values

    def remap_shape(self, cid, shape, p0=0, p1=0):
        out = (i64 * 4)()
        n, c, h, w = shape
        self.call("msb_remap_shape", cid, n, c, h, w, p0, p1, C.cast(out, vp))
        return tuple(int(v) for v in out)

    def remap_case(self, cid, dst, A, B, p0=0, p1=0, stream=None):
        n, c, h, w = A.shape
        self.call("msb_remap_case_f32", cid, _ptr(dst), _ptr(A), _ptr(B), n, c, h, w, p0, p1, stream)
        return dst

    def complex_case(self, cid, dst, A, B, stream=None):
        rows, cols = A.shape
        self.call("msb_complex_case_f32", cid, _ptr(dst), _ptr(A), _ptr(B), rows, cols, stream)
        return dst

    def axis_shape(self, cid, shape, p0=0, p1=1):
        out, ndim = (i64 * 4)(), C.c_int(0)
        n, c, h, w = shape
        self.call("msb_axis_shape", cid, n, c, h, w, p0, p1, C.cast(out, vp), C.cast(C.pointer(ndim), vp))
        return tuple(int(v) for v in out[:ndim.value])

    def axis_case(self, cid, dst, A, p0=0, p1=1, stream=None):
        n, c, h, w = A.shape
        self.call("msb_axis_case_f32", cid, _ptr(dst), _ptr(A), n, c, h, w, p0, p1, stream)
        return dst

    def select_case(self, cid, dst, A, B, idx_r, idx_c, p0=1, stream=None):
        rows, cols = A.shape
        self.call("msb_select_case_f32", cid, _ptr(dst), _ptr(A), _ptr(B), _ptr(idx_r), _ptr(idx_c), rows, cols, p0,
                  stream)
        return dst

    def unpack_patch2col(self, mat, img, psy, psx, sy, sx, dy=1, dx=1, stream=None):
        n, c, h, w = img.shape
        self.call("msb_unpack_patch2col_f32", _ptr(mat), _ptr(img), n, c, h, w, psy, psx, sy, sx, dy, dx, stream)
        return mat

    def pack_col2patch(self, img, mat, psy, psx, sy, sx, dy=1, dx=1, stream=None):
        n, c, h, w = img.shape
        self.call("msb_pack_col2patch_f32", _ptr(img), _ptr(mat), n, c, h, w, psy, psx, sy, sx, dy, dx, stream)
        return img

    def vectorized_sort(self, values, segments, stream=None):
        self.call("msb_vectorized_sort_f32_i32", _ptr(values), _ptr(segments), values.shape[0], stream)
        return values, segments

    def index_fill(self, dst, index, src, stream=None):
        k, d = dst.shape
        self.call("msb_index_fill_f32_i32", _ptr(dst), _ptr(index), _ptr(src), k, d, index.shape[0], stream)
        return dst

    def softmax3d(self, dst, src, stream=None):
        batch, classes, npos = src.shape
        self.call("msb_softmax3d_f32", _ptr(dst), _ptr(src), batch, classes, npos, _ld(dst), _ld(src), stream)
        return dst

    def softmax_grad3d(self, dst, src, label, mode=0, ignore_label=0.0, alpha=0.0, stream=None):
        batch, classes, npos = src.shape
        self.call("msb_softmax_grad3d_f32", _ptr(dst), _ptr(src), _ptr(label), batch, classes, npos, _ld(dst),
                  _ld(src), _ld(label), mode, ignore_label, alpha, stream)
        return dst


_lib = None


def load():
    """The process-wide Library instance."""
    global _lib
    if _lib is None:
        _lib = Library()
    return _lib
