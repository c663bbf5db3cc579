"""The host runtime library (``include/iian_b200/c_api.h``) through ``ctypes``.

Block pool, cache manager, scheduler and the packing of a decode step are C++ (``iian_b200/csrc/host``); the
classes in ``block_pool.py``, ``manager.py`` and ``engine/scheduler.py`` are thin handles on them.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_double, c_int, c_int32, c_longlong, c_uint64, c_void_p

from ..csrc import build as _build


class PoolError(RuntimeError):
    """Out of pages, a page freed twice, a token in a page that was given back."""


_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    L = _build.load_host()
    I32P, IP, U64P, LLP, VPP = POINTER(c_int32), POINTER(c_int), POINTER(c_uint64), POINTER(c_longlong), POINTER(c_void_p)

    def sig(name, res, *args):
        f = getattr(L, name)
        f.restype = res
        f.argtypes = list(args)

    sig("iian_host_last_error", ctypes.c_char_p)
    sig("iian_hash_block", c_uint64, c_uint64, I32P, c_int, c_uint64)
    sig("iian_pool_new", c_void_p, c_int, c_int, c_int)
    sig("iian_pool_delete", None, c_void_p)
    sig("iian_pool_get", c_longlong, c_void_p, c_int, c_int)
    sig("iian_pool_hash", c_uint64, c_void_p, c_int)
    sig("iian_pool_free_list", c_int, c_void_p, IP, c_int)
    sig("iian_pool_get_cached_block", c_int, c_void_p, c_uint64, I32P, c_int)
    sig("iian_pool_cache_block", c_int, c_void_p, c_int, c_uint64, I32P, c_int)
    sig("iian_pool_reset_prefix_cache", c_int, c_void_p)
    sig("iian_pool_touch", c_int, c_void_p, c_int)
    sig("iian_pool_get_new_blocks", c_int, c_void_p, c_int, IP)
    sig("iian_pool_free_blocks", c_int, c_void_p, IP, c_int)
    sig("iian_pool_check", c_int, c_void_p)
    sig("iian_cache_new", c_void_p, IP, IP, c_int, c_int, c_int, c_int)
    sig("iian_cache_delete", None, c_void_p)
    sig("iian_cache_pool", c_void_p, c_void_p, c_int)
    sig("iian_cache_slots", c_int, c_void_p, c_int, c_int, IP)
    sig("iian_cache_counter", c_longlong, c_void_p, c_int, c_longlong)
    sig("iian_rc_new", c_void_p, c_void_p)
    sig("iian_rc_delete", None, c_void_p)
    sig("iian_rc_get", c_int, c_void_p, c_int, c_int)
    sig("iian_rc_set_state_fresh", None, c_void_p, c_int)
    sig("iian_rc_table", IP, c_void_p, c_int)
    sig("iian_rc_hashes", U64P, c_void_p)
    sig("iian_cache_allot_state", c_int, c_void_p, c_void_p)
    sig("iian_cache_first_needed_block", c_int, c_void_p, c_int, c_int)
    sig("iian_cache_update_hashes", c_int, c_void_p, c_void_p, I32P, c_int, c_uint64)
    sig("iian_cache_find_prefix", c_int, c_void_p, I32P, c_int, U64P, c_int, IP, IP, c_int)
    sig("iian_cache_commit", c_int, c_void_p, c_void_p, I32P, c_int, c_int)
    sig("iian_cache_release_passed", c_int, c_void_p, c_void_p, c_int, IP)
    sig("iian_cache_allocate", c_int, c_void_p, c_void_p, c_int, c_int, IP, IP, c_int, IP)
    sig("iian_cache_free", c_int, c_void_p, c_void_p)
    sig("iian_cache_slot_of", c_int, c_void_p, c_void_p, c_int, c_int, LLP)
    sig("iian_cache_usage", c_double, c_void_p)
    sig("iian_cache_check", c_int, c_void_p)
    sig("iian_req_new", c_void_p, c_longlong, I32P, c_int, c_int, c_double, c_uint64)
    sig("iian_req_delete", None, c_void_p)
    sig("iian_req_get", c_int, c_void_p, c_int)
    sig("iian_req_set", None, c_void_p, c_int, c_int)
    sig("iian_req_append", None, c_void_p, I32P, c_int)
    sig("iian_req_cache", c_void_p, c_void_p)
    sig("iian_req_adopt_cache", None, c_void_p, c_void_p)
    sig("iian_sched_new", c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int)
    sig("iian_sched_delete", None, c_void_p)
    sig("iian_sched_add", c_int, c_void_p, c_void_p)
    sig("iian_sched_finish", c_int, c_void_p, c_void_p, c_int)
    sig("iian_sched_schedule", c_int, c_void_p, VPP, IP, IP, c_int, IP, VPP, IP, IP)
    sig("iian_sched_update", c_int, c_void_p)
    sig("iian_sched_queue", c_int, c_void_p, c_int, VPP, c_int)
    sig("iian_sched_num_preemptions", c_longlong, c_void_p)
    sig("iian_pack_decode_step", c_int, c_void_p, VPP, I32P, I32P, c_int, c_int, c_int, c_void_p, c_void_p, c_int, IP)
    _lib = L
    return L


def check(code: int) -> None:
    """Raise what the library reported: 1 is a pool error, anything else a ValueError."""
    if code == 0:
        return
    msg = lib().iian_host_last_error().decode("utf-8", "replace")
    if code == 1:
        raise PoolError(msg)
    raise ValueError(msg)


def i32_array(values):
    n = len(values)
    return (c_int32 * n)(*values), n


def int_array(values):
    n = len(values)
    return (c_int * n)(*values), n
