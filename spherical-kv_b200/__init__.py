"""B200-native kernels for the Spherical-KV hot path: spherical encode into bit-packed
pages and angle-domain decode attention over them.

The directory name is not a Python identifier; import it with
``importlib.import_module("spherical-kv_b200")`` (the repository root on sys.path).

All compute goes through libsphkv_b200.so (C ABI in include/sphkv.h).  There is no CPU or
PyTorch fallback: ops raise if the library is missing.
"""
from . import _lib, pages, synth  # noqa: F401
from ._lib import SphKVError, RADIUS_F16, RADIUS_I8  # noqa: F401
from .pages import (PagedCache, PageLists, REFERENCE_TIERS, TierSet, TierSpec,  # noqa: F401
                    build_page_lists, shard_block_lists)
from . import split_kv  # noqa: F401
from .ops import (CodeCache, check_status, decode_paged, decode_scratch, encode_codes, encode_pages,  # noqa: F401
                  hf_inv_freq, merge_partials, omega_ema, pages_from_codes, rope_table)
from .kmeans import kmeans_assign, spherical_kmeans  # noqa: F401

__all__ = ["SphKVError", "RADIUS_F16", "RADIUS_I8", "PagedCache", "PageLists", "REFERENCE_TIERS",
           "TierSet", "TierSpec", "build_page_lists", "shard_block_lists", "check_status", "decode_paged", "decode_scratch",
           "encode_pages", "hf_inv_freq", "merge_partials", "omega_ema", "rope_table", "kmeans_assign", "CodeCache", "encode_codes", "pages_from_codes",
           "spherical_kmeans"]
