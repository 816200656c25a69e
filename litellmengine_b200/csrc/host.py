"""ctypes access to the native host code (`host_core.cpp`): the records of the cache manager and the
packing of a step (the scheduler declares its own functions).

Needs no GPU.  The library is compiled in-tree on first use like the kernels' (by nvcc as plain
C++); a failed call raises what the Python classes document: `OutOfPages` for "nothing was taken",
`CacheError` for a misuse, with the library's message.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_int32, c_longlong, c_void_p

from . import build

_lib = None

_SIGNATURES = {
    "hc_last_error": ([], c_char_p),
    "hc_pool_new": ([c_int], c_void_p),
    "hc_pool_delete": ([c_void_p], None),
    "hc_pool_num_pages": ([c_void_p], c_int),
    "hc_pool_free_count": ([c_void_p], c_int),
    "hc_pool_take": ([c_void_p, c_int, c_void_p], c_int),
    "hc_pool_give": ([c_void_p, c_void_p, c_int], c_int),
    "hc_pool_used": ([c_void_p, c_void_p], c_int),
    "hc_cache_new": ([c_int, c_void_p, c_int, c_int, c_int, c_int, c_int], c_void_p),
    "hc_cache_delete": ([c_void_p], None),
    "hc_cache_pool": ([c_void_p, c_int], c_void_p),
    "hc_cache_table": ([c_void_p, c_int], POINTER(c_int32)),
    "hc_cache_first_held": ([c_void_p, c_int], POINTER(c_int32)),
    "hc_cache_num_logical": ([c_void_p, c_int], POINTER(c_int32)),
    "hc_cache_free_slots": ([c_void_p], c_int),
    "hc_cache_is_live": ([c_void_p, c_int], c_int),
    "hc_cache_admit": ([c_void_p, POINTER(c_int)], c_int),
    "hc_cache_length": ([c_void_p, c_int, POINTER(c_longlong)], c_int),
    "hc_cache_release": ([c_void_p, c_int], c_int),
    "hc_cache_pages_missing": ([c_void_p, c_int, c_longlong, c_void_p], c_int),
    "hc_cache_can_hold": ([c_void_p, c_int, c_void_p, c_void_p, POINTER(c_int)], c_int),
    "hc_cache_reserve": ([c_void_p, c_void_p, c_int, c_longlong, c_void_p, POINTER(c_int)], c_int),
    "hc_cache_ensure": ([c_void_p, c_int, c_longlong], c_int),
    "hc_cache_commit": ([c_void_p, c_int, c_longlong, POINTER(c_int)], c_int),
    "hc_cache_pending": ([c_void_p, c_int], c_int),
    "hc_cache_drain": ([c_void_p, c_int, c_void_p, c_void_p], None),
    "hc_cache_check": ([c_void_p], c_int),
    "hc_cache_lengths": ([c_void_p, c_int, c_void_p, c_void_p], c_int),
    "hc_cache_ensure_all": ([c_void_p, c_int, c_void_p, c_void_p], c_int),
    "hc_cache_commit_all": ([c_void_p, c_int, c_void_p, c_void_p, POINTER(c_int)], c_int),
    "hc_pack_step": ([c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                      c_void_p], c_int),
}


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        l = ctypes.CDLL(build.ensure_built("host_core"))
        for name, (argtypes, restype) in _SIGNATURES.items():
            f = getattr(l, name)
            f.argtypes, f.restype = argtypes, restype
        _lib = l
    return _lib


def last_error() -> str:
    return lib().hc_last_error().decode()
