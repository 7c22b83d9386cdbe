"""ctypes binding of libsphkv_b200.so (declarations mirror include/sphkv.h).

The library is the only compute path of this package: if it cannot be loaded the import
of any op raises, there is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libsphkv_b200.so")

F32, BF16, F16 = 0, 1, 2
RADIUS_I8, RADIUS_F16 = 0, 1
MAX_TIER_SLOTS = 4
MAX_GQA = 8
ST_BAD_POSITION, ST_BAD_BLOCK, ST_BAD_SLOT, ST_TIMEOUT, ST_INTERNAL = 1, 2, 4, 8, 16

_I4 = C.c_int32 * MAX_TIER_SLOTS


class Tiers(C.Structure):
    _fields_ = [("n_slots", C.c_int32), ("G_max", C.c_int32), ("C_max", C.c_int32),
                ("g_max", C.c_int32), ("g", _I4), ("bits", _I4), ("tier_id", _I4)]


class EncodeParams(C.Structure):
    _fields_ = [
        ("k_src", C.c_void_p), ("v_src", C.c_void_p), ("src_index", C.c_void_p),
        ("bundles", C.c_void_p), ("page_head", C.c_void_p), ("page_slot", C.c_void_p),
        ("ptable", C.c_void_p), ("codebooks", C.c_void_p), ("k_pages", C.c_void_p),
        ("v_pool", C.c_void_p), ("scratch", C.c_void_p), ("scratch_bytes", C.c_int64),
        ("k_row_stride", C.c_int64), ("k_head_stride", C.c_int64),
        ("v_row_stride", C.c_int64), ("v_head_stride", C.c_int64),
        ("code_r", C.c_void_p * MAX_TIER_SLOTS), ("code_theta", C.c_void_p * MAX_TIER_SLOTS),
        ("code_rows", C.c_int64),
        ("n_bundles", C.c_int32), ("n_pages", C.c_int32), ("page_size", C.c_int32),
        ("dh", C.c_int32), ("Hkv", C.c_int32),
        ("k_dtype", C.c_int32), ("v_src_dtype", C.c_int32), ("v_pool_dtype", C.c_int32),
        ("radius_fmt", C.c_int32), ("tiers", Tiers),
    ]


class DecodeParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k_pages", C.c_void_p), ("ptable", C.c_void_p),
        ("v_pool", C.c_void_p), ("positions", C.c_void_p), ("block_table", C.c_void_p),
        ("bits_table", C.c_void_p), ("num_blocks", C.c_void_p), ("codebooks", C.c_void_p),
        ("rope_table", C.c_void_p), ("out", C.c_void_p), ("out_partial", C.c_void_p),
        ("page_ml", C.c_void_p), ("logits_out", C.c_void_p), ("scratch", C.c_void_p), ("scratch_bytes", C.c_int64),
        ("status", C.c_void_p), ("omega", C.c_void_p),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("dh", C.c_int32),
        ("page_size", C.c_int32), ("max_blocks", C.c_int32), ("n_pages", C.c_int32),
        ("max_pos", C.c_int32),
        ("q_dtype", C.c_int32), ("v_dtype", C.c_int32), ("out_dtype", C.c_int32),
        ("radius_fmt", C.c_int32), ("n_ctas", C.c_int32), ("sm_scale", C.c_float),
        ("ema_beta", C.c_float), ("tiers", Tiers),
        ("xchg_recv", C.c_void_p), ("xchg_seq", C.c_void_p),
        ("xchg_timeout_cycles", C.c_int64), ("xchg_rank", C.c_int32), ("xchg_world", C.c_int32),
    ]


# name -> (restype, argtypes); every symbol include/sphkv.h declares
SIGNATURES = {
    "sphkv_abi_version": (C.c_int, []),
    "sphkv_last_error": (C.c_char_p, []),
    "sphkv_sm_count": (C.c_int, []),
    "sphkv_struct_size": (C.c_int, [C.c_int]),
    "sphkv_rope_table_build": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "sphkv_encode_pages": (C.c_int, [C.POINTER(EncodeParams), C.c_void_p]),
    "sphkv_pages_from_codes": (C.c_int, [C.POINTER(EncodeParams), C.c_void_p]),
    "sphkv_encode_codes": (C.c_int, [C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_int32,
                                     C.c_void_p, C.POINTER(Tiers), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                     C.c_void_p]),
    "sphkv_encode_scratch_bytes": (C.c_int64, [C.c_int32, C.c_int32, C.c_int32]),
    "sphkv_decode_scratch_bytes": (C.c_int64, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "sphkv_decode_paged": (C.c_int, [C.POINTER(DecodeParams), C.c_void_p]),
    "sphkv_decode_paged_static": (C.c_int, [C.POINTER(DecodeParams), C.c_void_p]),
    "sphkv_merge_partials": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                       C.c_int32, C.c_void_p]),
    "sphkv_xchg_alloc": (C.c_int, [C.c_int64, C.POINTER(C.c_void_p), C.c_char_p]),
    "sphkv_xchg_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "sphkv_xchg_close": (C.c_int, [C.c_void_p]),
    "sphkv_xchg_free": (C.c_int, [C.c_void_p]),
    "sphkv_pool_decode": (C.c_int, [C.c_void_p] * 13 + [C.c_int32] * 10 + [C.c_float, C.c_int32,
                                                                            C.c_void_p]),
    "sphkv_pool_encode_append": (C.c_int, [C.c_void_p] * 8 + [C.c_int32] * 9 + [C.c_void_p]),
    "sphkv_qlut_logits": (C.c_int, [C.c_void_p] * 8 + [C.c_int32] * 8 + [C.c_float, C.c_int32,
                                                                        C.c_void_p]),
    "sphkv_omega_ema": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                  C.c_float, C.c_void_p]),
    "sphkv_ragged_logits": (C.c_int, [C.c_void_p] * 9 + [C.c_int32] * 12 + [C.c_void_p]),
    "sphkv_pool_build_pages": (C.c_int, [C.c_void_p] * 3 + [C.c_int32, C.c_int64, C.c_int64, C.c_void_p,
                                         C.c_int32] + [C.c_void_p] * 4 + [C.c_int32] * 3 + [C.c_void_p]),
    "sphkv_kmeans_assign": (C.c_int, [C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_int32] + [C.c_void_p] * 5),
    "sphkv_pool_append_step": (C.c_int, [C.c_void_p] * 12 + [C.c_int32] * 10 + [C.c_void_p]),
}

_lib = None


class SphKVError(RuntimeError):
    pass


def load() -> C.CDLL:
    """Loads the shared library once; raises if it is missing (no fallback exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise SphKVError(
            f"{LIB_PATH} is missing: build it with `python -c \"import __graft_entry__ as g; "
            f"g.build()\"` (needs nvcc); this package has no CPU or PyTorch fallback")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    ver = lib.sphkv_abi_version()
    if ver != 4:
        raise SphKVError(f"libsphkv_b200.so ABI version {ver}, expected 4")
    for which, st in enumerate((Tiers, EncodeParams, DecodeParams)):
        if lib.sphkv_struct_size(which) != C.sizeof(st):
            raise SphKVError(f"struct layout mismatch for {st.__name__}: library "
                             f"{lib.sphkv_struct_size(which)} B, binding {C.sizeof(st)} B")
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().sphkv_last_error().decode(errors="replace")
        raise SphKVError(f"{what} failed (code {rc}): {msg}")
