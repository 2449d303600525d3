"""ctypes binding of libmshadow_b200_ps.so (include/mshadow_b200_ps.h): the multi-GPU
synchronisation model with the interface of dmlc/mshadow's mshadow-ps ISharedModel, one process
per GPU, sums by NCCL all-reduce.  Used by the tests and by multi-process examples; C++ users
include mshadow-ps/mshadow_ps.h instead.  There is no fallback when the library is missing.
"""
import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmshadow_b200_ps.so")
HEADER_PATH = os.path.join(os.path.dirname(HERE), "include", "mshadow_b200_ps.h")

vp, i64, cint = C.c_void_p, C.c_int64, C.c_int

_SIGNATURES = {
    "msb_ps_new_unique_id": [C.c_char_p, i64],
    "msb_ps_create": [cint, cint, C.c_char_p, cint, C.POINTER(vp)],
    "msb_ps_peer_create": [cint, cint, cint, i64, cint, cint, cint, C.POINTER(vp)],
    "msb_ps_pull_fence": [vp, cint, vp],
    "msb_ps_peer_handle": [vp, C.c_char_p, i64],
    "msb_ps_peer_connect": [vp, C.c_char_p],
    "msb_ps_peer_next_sink": [vp, cint, i64, i64, vp],
    "msb_ps_peer_reserve": [vp, i64, vp],
    "msb_ps_peer_window": [vp, cint, i64, vp],
    "msb_ps_destroy": [vp],
    "msb_ps_init_key": [vp, cint, i64, i64],
    "msb_ps_push": [vp, vp, i64, i64, i64, cint, vp],
    "msb_ps_pull_req": [vp, vp, i64, i64, i64, cint, vp],
    "msb_ps_pull_wait": [vp, cint],
    "msb_ps_set_weight": [vp, vp, i64, i64, i64, cint, vp],
    "msb_ps_check_weight": [vp, vp, i64, i64, i64, cint, vp],
}


def declared_symbols():
    text = open(HEADER_PATH).read()
    return sorted(set(re.findall(r"\b(msb_ps_[a-z0-9_]+)\s*\(", text)))


class PsError(RuntimeError):
    pass


class PeerSink(C.Structure):
    """msb_peer_sink_t of include/mshadow_b200_peer_sink.h."""
    _fields_ = [("row", C.c_void_p * 16), ("tag", C.c_uint32), ("count", C.c_uint32), ("world", C.c_int)]


_dll = None


def dll():
    global _dll
    if _dll is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError("%s not found: build it with `python -m mshadow_b200.build`" % LIB_PATH)
        _dll = C.CDLL(LIB_PATH)
        _dll.msb_ps_last_error.restype = C.c_char_p
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(_dll, name)
            fn.argtypes = argtypes
            fn.restype = cint
    return _dll


def _check(status):
    if status != 0:
        raise PsError(dll().msb_ps_last_error().decode("utf-8", "replace"))


def new_unique_id():
    """Group identifier for a new set of processes; create on one rank, hand to the others."""
    buf = C.create_string_buffer(300)
    _check(dll().msb_ps_new_unique_id(buf, 300))
    return buf.value.decode("ascii")


def _mat(t):
    """(pointer, rows, cols, leading dimension) of a tensor viewed as a matrix over its last axis."""
    assert t.dim() >= 1 and (t.stride(-1) == 1 or t.shape[-1] <= 1)
    cols = t.shape[-1]
    rows = t.numel() // cols if cols else 0
    ld = t.stride(-2) if t.dim() >= 2 else cols
    return vp(t.data_ptr()), rows, cols, ld


class SharedModel:
    """One process's handle on the model: mirrors ISharedModel (InitKey, Push, PullReq, PullWait,
    SetWeight, CheckWeight) for fp32 device tensors of the GPU it was created on."""

    def __init__(self, rank=0, world=1, unique_id=None, device=0):
        self.handle = vp()
        uid = unique_id.encode("ascii") if unique_id is not None else None
        _check(dll().msb_ps_create(rank, world, uid, device, C.byref(self.handle)))
        self._after_create()

    def _after_create(self):
        pass

    def close(self):
        if self.handle:
            _check(dll().msb_ps_destroy(self.handle))
            self.handle = vp()

    def init_key(self, key, shape):
        cols = shape[-1]
        rows = 1
        for s in shape[:-1]:
            rows *= s
        _check(dll().msb_ps_init_key(self.handle, key, rows, cols))

    def push(self, tensor, key, stream=None):
        p, rows, cols, ld = _mat(tensor)
        _check(dll().msb_ps_push(self.handle, p, rows, cols, ld, key, stream))

    def pull_req(self, tensor, key, stream=None):
        p, rows, cols, ld = _mat(tensor)
        _check(dll().msb_ps_pull_req(self.handle, p, rows, cols, ld, key, stream))

    def pull_wait(self, key):
        _check(dll().msb_ps_pull_wait(self.handle, key))

    def pull_fence(self, key, stream=None):
        """Later work on `stream` runs after the last pull of `key`; the host does not wait."""
        _check(dll().msb_ps_pull_fence(self.handle, key, stream))

    def set_weight(self, tensor, key, stream=None):
        p, rows, cols, ld = _mat(tensor)
        _check(dll().msb_ps_set_weight(self.handle, p, rows, cols, ld, key, stream))

    def check_weight(self, tensor, key, stream=None):
        p, rows, cols, ld = _mat(tensor)
        _check(dll().msb_ps_check_weight(self.handle, p, rows, cols, ld, key, stream))


class PeerModel(SharedModel):
    """The peer-store model (mshadow::ps::PeerModel): same calls as SharedModel; the sum of a small
    tensor is formed from direct stores into every GPU's window over NVLink, in rank order.

    Set-up takes two steps because the ranks must learn each other's windows: create the model on
    every rank, gather `handle()` of all ranks in rank order (any transport), `connect(handles)`."""

    def __init__(self, rank=0, world=1, device=0, window_bytes=0, depth=0, wait_limit_ms=0, own_stream=False):
        self.handle = vp()
        self.world = world
        _check(dll().msb_ps_peer_create(rank, world, device, window_bytes, depth, wait_limit_ms, int(own_stream),
                                        C.byref(self.handle)))

    def export_handle(self):
        buf = C.create_string_buffer(200)
        _check(dll().msb_ps_peer_handle(self.handle, buf, 200))
        return buf.value.decode("ascii")

    def connect(self, handles):
        """`handles`: the export_handle() strings of all ranks, in rank order."""
        assert len(handles) == self.world
        _check(dll().msb_ps_peer_connect(self.handle, "".join(handles).encode("ascii")))

    def reserve(self, nbytes):
        """Sets `nbytes` of every rank's window aside for the caller's own kernels; returns the offset
        (the same on all ranks when all make the same calls in the same order)."""
        off = C.c_int64(0)
        _check(dll().msb_ps_peer_reserve(self.handle, nbytes, C.byref(off)))
        return int(off.value)

    def window(self, rank, offset=0):
        """Address, in this process, of byte `offset` of rank `rank`'s window (after connect)."""
        ptr = vp()
        _check(dll().msb_ps_peer_window(self.handle, rank, offset, C.byref(ptr)))
        return int(ptr.value or 0)

    def next_sink(self, key, offset, count):
        """Sink for `count` results from element `offset` of the key's row in the step that the
        segment at offset 0 opens; hand it to Library.reduce_keep_*(..., sink=...)."""
        sink = PeerSink()
        _check(dll().msb_ps_peer_next_sink(self.handle, key, offset, count, C.byref(sink)))
        return sink
