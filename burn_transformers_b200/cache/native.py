"""The host library (csrc/host/page_book.cpp): the cache's books and the packing of a step's integers, in C++.

Loaded with ctypes and built on first use with the system's C++ compiler; it has no CUDA in it."""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_longlong, c_void_p

from ..errors import CacheError

_LIB = None


def library() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        from ..csrc.build import build_host
        path = build_host()
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as error:
            raise CacheError(f"cannot load the host library {path}: {error}") from None
        lib.bth_last_error.restype = c_char_p
        lib.bth_pool_create.restype = c_void_p
        lib.bth_pool_create.argtypes = [c_int, c_char_p]
        lib.bth_book_create.restype = c_void_p
        lib.bth_book_create.argtypes = [c_int, c_int, c_longlong, c_int, c_void_p, c_void_p]
        lib.bth_book_tokens_held.restype = c_longlong
        for name in ("bth_pool_destroy", "bth_pool_take", "bth_pool_free", "bth_pool_check", "bth_book_destroy",
                     "bth_book_acquire", "bth_book_free_slots", "bth_book_tokens_held", "bth_book_check"):
            getattr(lib, name).argtypes = [c_void_p]
        for name in ("bth_pool_give_back", "bth_pool_is_held", "bth_book_release", "bth_book_length",
                     "bth_book_slot_is_held", "bth_book_free_pages"):
            getattr(lib, name).argtypes = [c_void_p, c_int]
        lib.bth_book_commit.argtypes = [c_void_p, c_int, c_int]
        lib.bth_book_reserve.argtypes = [c_void_p, c_int, c_void_p, c_void_p]
        lib.bth_book_table_row.argtypes = [c_void_p, c_int, c_int, c_void_p, c_int]
        lib.bth_book_pack_step.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                           c_void_p, c_void_p, c_void_p]
        if lib.bth_abi_version() != 1:
            raise CacheError(f"{path} has an unexpected interface version")
        _LIB = lib
    return _LIB


def error() -> CacheError:
    """The library's last error as an exception to raise."""
    return CacheError(library().bth_last_error().decode(errors="replace"))
