"""thrust_b200 — Thrust's sort / scan / reduce_by_key hot path as hand-written sm_100a kernels.

The product is the C ABI in ``include/thrust_b200.h`` (``libthrust_b200.so``) and the
Thrust custom system in ``include/thrust_b200/system.h``. This Python package is the
test and benchmark driver: it binds the C ABI with ctypes and uses PyTorch only for
device memory, streams and ``torch.distributed``.

Attributes are resolved on first use so that ``python -m thrust_b200.build`` can run
before the shared library exists; touching any algorithm without the library raises
ImportError (there is no CPU or PyTorch fallback).
"""
import importlib

_ALGORITHMS = (
    "sort", "stable_sort", "sort_by_key", "stable_sort_by_key", "inclusive_scan", "exclusive_scan", "reduce",
    "inclusive_scan_by_key", "exclusive_scan_by_key",
    "reduce_by_key", "unique_by_key", "unique", "copy_flagged", "histogram_sorted", "dense_histogram", "tb200_dtype",
)
__all__ = ["Tb200Error", "_capi", "algorithms", "datagen", "sample_sort", *_ALGORITHMS]


def __getattr__(name):
    if name in _ALGORITHMS:
        return getattr(importlib.import_module(".algorithms", __name__), name)
    if name == "Tb200Error":
        return importlib.import_module("._capi", __name__).Tb200Error
    if name in ("_capi", "algorithms", "datagen", "sample_sort", "build"):
        return importlib.import_module("." + name, __name__)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
