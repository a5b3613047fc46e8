"""Loader of the native page-id pool.

The pool is C++ (``distie_b200/csrc/block_pool.cpp``) behind pybind11, like the
reference's ``distie_core.BlockPool`` (core/python/bindings.cpp:8-22) and its
loader (worker/src/inference/native.py:14-20): ``BlockPool(num_blocks)`` with
``allocate(count)``, ``free(ids)`` and the properties ``num_blocks``, ``num_free``,
``num_used``, ``utilization``.  It is compiled on first use.
"""

from __future__ import annotations

import importlib.util

_module = None


def native_module():
    global _module
    if _module is None:
        from ..csrc import build

        path = build.build_block_pool()
        spec = importlib.util.spec_from_file_location("distie_b200_core", path)
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        _module = module
    return _module


def BlockPool(num_blocks: int):
    """A new native pool of ``num_blocks`` page ids."""
    return native_module().BlockPool(int(num_blocks))
