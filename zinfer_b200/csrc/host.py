"""The native host runtime (``host_runtime.cpp``: page pools, the cache manager's
bookkeeping, the step builder) as ctypes functions.  It is part of the kernel library
but touches no GPU, so it loads and runs on a machine without one (only nvcc is needed,
to build the library at first use)."""
from __future__ import annotations

import ctypes

from . import build as _build

_LIB = None

# negative return codes of the native functions
OUT_OF_PAGES, NOT_LIVE, ALREADY_LIVE, BAD_PAGE, RELEASED, CHECK, ARGUMENT, NAMED_TWICE = -2, -3, -4, -5, -6, -7, -8, -9

_P, _I, _LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
_SIGNATURES = {
    "zi_pool_create": (_P, [_I]),
    "zi_pool_destroy": (None, [_P]),
    "zi_pool_alloc": (_I, [_P, _I, _P]),
    "zi_pool_free": (_I, [_P, _P, _I, _P]),
    "zi_pool_stats": (None, [_P, _P]),
    "zi_pool_check": (_I, [_P]),
    "zi_cache_create": (_P, [_I, _P, _P, _I, _I]),
    "zi_cache_destroy": (None, [_P]),
    "zi_cache_add": (_I, [_P, _LL]),
    "zi_cache_free": (_I, [_P, _LL, _P, _I]),
    "zi_cache_has": (_I, [_P, _LL]),
    "zi_cache_length": (_LL, [_P, _LL]),
    "zi_cache_slot": (_I, [_P, _LL]),
    "zi_cache_num_requests": (_I, [_P]),
    "zi_cache_pages_needed": (_I, [_P, _LL, _LL, _P]),
    "zi_cache_can_reserve": (_I, [_P, _LL, _LL]),
    "zi_cache_reserve": (_I, [_P, _LL, _LL, _P]),
    "zi_cache_reserve_all": (_I, [_P, _I, _P, _P, _P]),
    "zi_cache_commit": (_I, [_P, _LL, _LL, _P, _I]),
    "zi_cache_table_len": (_I, [_P, _LL, _I]),
    "zi_cache_table": (_I, [_P, _LL, _I, _P, _I]),
    "zi_cache_slots_for": (_I, [_P, _LL, _I, _LL, _I, _P]),
    "zi_cache_pool_stats": (_I, [_P, _I, _P]),
    "zi_cache_check": (_I, [_P]),
    "zi_step_build": (_LL, [_P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _LL, _P]),
}


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        handle = ctypes.CDLL(_build.library_path())
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        handle.zi_last_error.restype = ctypes.c_char_p
        _LIB = handle
    return _LIB


def last_error() -> str:
    return lib().zi_last_error().decode("utf-8", "replace")
