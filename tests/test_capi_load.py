"""The C-ABI library loads without a GPU and exports everything the header declares."""
import ctypes as C
import os

import mshadow_b200
from mshadow_b200 import capi


def test_header_lists_expected_entry_points():
    names = capi.declared_symbols()
    for required in ["msb_expr_case_f32", "msb_reduce_keep_lowest_f32", "msb_reduce_keep_highdim_f32",
                     "msb_softmax_f32", "msb_softmax_grad_f32", "msb_pool_f32", "msb_unpool_f32",
                     "msb_chpool_f32", "msb_addtakegrad_f32_i32", "msb_addtakegrad_largebatch_f32_i32",
                     "msb_sort_by_key_i32", "msb_copy_2d", "msb_alloc_space", "msb_last_error"]:
        assert required in names


def test_library_exports_every_declared_symbol():
    assert os.path.exists(capi.LIB_PATH), "build the library first (python -m mshadow_b200.build)"
    dll = C.CDLL(capi.LIB_PATH)
    missing = [n for n in capi.declared_symbols() if not hasattr(dll, n)]
    assert not missing, missing


def test_binding_covers_every_status_returning_symbol():
    bound = set(capi._SIGNATURES) | {"msb_last_error", "msb_version", "msb_launch_count"}
    assert set(capi.declared_symbols()) <= bound


def test_version_and_argument_errors_need_no_gpu():
    lib = mshadow_b200.load()
    assert lib.dll.msb_version() >= 100
    # argument validation happens before any CUDA call
    st, msg = lib.status("msb_expr_case_f32", 42, None, None, None, None, None, 1, 1, 1, 1, 1, 1, None)
    assert st == 1 and "unknown expression id" in msg
    st, msg = lib.status("msb_softmax_f32", None, None, 4, 4, 2, 4, None)
    assert st == 2
    st, msg = lib.status("msb_copy_2d", None, 4, None, 4, 1, 4, 4, 7, None)
    assert st == 1
