"""Loads ``libhl_b200.so`` (the C ABI of ``include/hl_b200.h``) and declares its signatures.

There is no fallback: if the library is missing or a symbol is absent, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libhl_b200.so")

OK = 0
ERR_ARG, ERR_OOM, ERR_DEVICE, ERR_TIMEOUT, ERR_MISMATCH, ERR_ZERO, ERR_UNSUPPORTED = -1, -2, -3, -4, -5, -6, -7


class Stats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("commits", "folds", "gathers", "merkles", "round_batches", "kernel_launches",
                                          "bytes_h2d", "bytes_d2h", "declines", "generated_rounds")]


_vp, _u32, _u64, _sz, _int = C.c_void_p, C.c_uint32, C.c_uint64, C.c_size_t, C.c_int
_pp = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); every entry point the header declares
SIGNATURES = {
    "hl_b200_init": (_int, [_int, _pp]),
    "hl_b200_shutdown": (None, [_vp]),
    "hl_b200_label": (C.c_char_p, [_vp]),
    "hl_b200_last_error": (C.c_char_p, [_vp]),
    "hl_b200_set_stream": (_int, [_vp, _vp]),
    "hl_b200_sync": (_int, [_vp]),
    "hl_b200_set_encoder": (_int, [_vp, _int]),
    "hl_b200_set_slot_kernels": (_int, [_vp, _int]),
    "hl_b200_probe_field": (_int, [_vp, _vp, _vp, _sz, _vp]),
    "hl_b200_commit": (_int, [_vp, _u32, _u32, _vp, _sz, _u32, _vp, _pp, _vp]),
    "hl_b200_commit_zk": (_int, [_vp, _u32, _u32, _vp, _sz, _vp, _sz, _vp, _u32, _vp, _pp, _vp]),
    "hl_b200_commit_zk_dev": (_int, [_vp, _u32, _u32, _vp, _sz, _vp, _sz, _vp, _vp, _pp, _vp]),
    "hl_b200_merkle": (_int, [_vp, _vp, _vp, _sz, _vp, _vp, _vp]),
    "hl_b200_store_merkle": (_int, [_vp, _vp, _vp, _vp, _vp]),
    "hl_b200_store_merkle_dev": (_int, [_vp, _vp, _vp, _vp, _vp]),
    "hl_b200_store_fold": (_int, [_vp, _vp, _sz, _int, _vp]),
    "hl_b200_store_columns": (_int, [_vp, _vp, _sz, _vp]),
    "hl_b200_store_shape": (_int, [_vp, C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_sz)]),
    "hl_b200_store_encoded_dev": (_vp, [_vp]),
    "hl_b200_store_leaves_dev": (_vp, [_vp]),
    "hl_b200_store_free": (None, [_vp]),
    "hl_b200_stats": (_int, [_vp, C.POINTER(Stats)]),
}

class FsState(C.Structure):
    _fields_ = [("state", C.c_uint8 * 32), ("counter", C.c_uint64), ("key", C.c_uint8 * 32), ("keyed", C.c_int32),
                ("recover_one", C.c_int32), ("have_claim", C.c_int32), ("reserved", C.c_int32), ("claim", C.c_uint64 * 2)]


SIGNATURES.update({
    "hl_b200_rounds_new": (_int, [_vp, _int, _sz, _u32, _u32, _vp, _vp, _sz, _pp]),
    "hl_b200_rounds_new_ir": (_int, [_vp, _sz, _u32, _u32, _vp, _vp, _sz, _u32, _u32, _vp, _sz, _pp]),
    "hl_b200_witness_product": (_int, [_vp, _sz, _vp, _sz, _sz, _vp, _sz, _sz, _sz, _sz, _sz, _int, _vp, _vp]),
    "hl_b200_witness_product_dev": (_int, [_vp, _sz, _vp, _sz, _sz, _vp, _sz, _sz, _sz, _sz, _sz, _int, _vp, _vp]),
    "hl_b200_act_histogram": (_int, [_vp, _vp, _vp, _sz, _sz, _sz, _sz, _vp, _vp, _sz, _vp, _vp]),
    "hl_b200_act_helpers": (_int, [_vp, _vp, _vp, _sz, _sz, _sz, _sz, _vp, _vp, _vp, _vp, _vp]),
    "hl_b200_act_table": (_int, [_vp, _vp, _sz, _sz, _vp, _vp, _vp, _vp, _vp, _vp]),
    "hl_b200_commit_zk_tree": (_int, [_vp, _u32, _u32, _vp, _sz, _vp, _sz, _vp, _u32, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "hl_b200_commit_zk_packed": (_int, [_vp, _u32, _u32, _vp, _vp, _sz, _vp, _sz, _vp, _u32, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "hl_b200_set_dependent_launch": (_int, [_int]),
    "hl_b200_verify_opening": (_int, [_vp, _u32, _u32, _sz, _vp, _vp, _sz, _vp, _sz, _sz, _vp, _vp, _vp, _u32, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "hl_b200_verify_columns": (_int, [_vp, _vp, _sz, _sz, _vp, _vp, _vp, _u32, _vp, _vp, _vp, _vp, _vp, _sz, _vp, _vp, _vp, _vp]),
    "hl_b200_mask_commit": (_int, [_vp, _u32, _u32, _vp, _sz, _vp, _sz, _vp, _vp, _vp, _vp, _vp]),
    "hl_b200_mask_open_q": (_int, [_vp, _sz, _vp, _vp]),
    "hl_b200_lookup_inverse_table": (_int, [_vp, _vp, _vp, _u32, _vp]),
    "hl_b200_lookup_helpers_dev": (_int, [_vp, _vp, _vp, _u32, _vp, _vp, _vp, _u32, _vp, _vp, _sz, _vp, _vp]),
    "hl_b200_rng_fill": (_int, [_vp, _vp, _u64, _u64, _int, _vp]),
    "hl_b200_rng_fill_dev": (_int, [_vp, _vp, _u64, _u64, _int, _vp]),
    "hl_b200_tables_new": (_int, [_vp, _sz, _u32, _pp]),
    "hl_b200_tables_put": (_int, [_vp, _sz, _vp]),
    "hl_b200_tables_eq": (_int, [_vp, _sz, _u32, _u32, _vp, _vp, _int]),
    "hl_b200_tables_plane": (_int, [_vp, _sz, _vp, _vp, _sz, _u64, _u32, _vp, _vp, _vp, _u32, _vp, _vp, _u32, _int]),
    "hl_b200_tables_flush": (_int, [_vp]),
    "hl_b200_tables_read": (_int, [_vp, _sz, _vp]),
    "hl_b200_tables_free": (None, [_vp]),
    "hl_b200_rounds_from_tables": (_int, [_vp, _int, _u32, _vp, _vp, _sz, _pp]),
    "hl_b200_rounds_from_tables_ir": (_int, [_vp, _u32, _vp, _vp, _sz, _u32, _u32, _vp, _sz, _pp]),
    "hl_b200_rounds_round": (_int, [_vp, _u32, _int, _vp]),
    "hl_b200_rounds_fold": (_int, [_vp, _vp]),
    "hl_b200_rounds_finals": (_int, [_vp, _vp]),
    "hl_b200_rounds_free": (None, [_vp]),
    "hl_b200_rounds_batched": (_int, [_vp, _u32, C.POINTER(FsState), _vp, _u32, _vp, _vp]),
})

SIGNATURES["hl_b200_hash_columns_static"] = (_int, [_vp, _sz, _sz, _vp, _vp, _vp])

SIGNATURES.update({
    "hl_b200_logup_histogram": (_int, [_vp, _vp, _sz, _sz, _vp]),
    "hl_b200_logup_helpers": (_int, [_vp, _vp, _vp, _sz, _vp, _vp, _vp, C.c_int64, _vp, _vp]),
    "hl_b200_fold_rows_i8": (_int, [_vp, _vp, _sz, _sz, _vp, _vp]),
    "hl_b200_fold_cols_i8": (_int, [_vp, _vp, _sz, _sz, _vp, _vp]),
})

SIGNATURES["hl_b200_butterfly_peak"] = (_int, [_vp, _u32, C.POINTER(C.c_double)])
SIGNATURES["hl_b200_compress_peak"] = (_int, [_vp, _u32, C.POINTER(C.c_double)])

SIGNATURES["hl_b200_set_alloc_cap"] = (_int, [_vp, _sz])

T_NAMES = ("encode", "hash", "merkle", "fold", "gather", "rounds", "logup", "tables", "witness")


class Timing(C.Structure):
    _fields_ = [("ms", C.c_double * 9), ("spans", C.c_uint64 * 9)]


SIGNATURES["hl_b200_timing_enable"] = (_int, [_vp, _int])
SIGNATURES["hl_b200_timing_read"] = (_int, [_vp, C.POINTER(Timing), _int])

_lib = None


def load() -> C.CDLL:
    """The loaded library; raises if it was not built (``python -m intelligenceregulation_b200.build``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m intelligenceregulation_b200.build`; "
                               "this backend has no CPU path")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the symbol is absent
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib
