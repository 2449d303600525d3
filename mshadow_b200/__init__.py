"""B200-native evaluation engine for the mshadow lazy-expression path.

The product is C++/CUDA: header-level templates under ``mshadow_b200/include/mshadow`` and the
C ABI of ``include/mshadow_b200.h`` built into ``libmshadow_b200.so``.  This Python package only
builds that library (``build.py``) and binds it (``capi.py``) for tests and benchmarks.
"""
from . import capi  # noqa: F401
from .capi import Library, MsbError, load  # noqa: F401
