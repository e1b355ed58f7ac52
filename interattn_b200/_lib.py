"""ctypes binding of libinterattn_b200.so (the C ABI in include/interattn_b200.h).

There is no fallback: if the shared library is missing or a symbol cannot be
resolved, importing the operators raises, and every operator refuses
non-CUDA tensors.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libinterattn_b200.so")

IA_OK = 0
IA_ERR_BAD_ARG = -1
IA_ERR_UNSUPPORTED = -2
IA_ERR_LAUNCH = -3

IA_F32, IA_BF16 = 0, 1
IA_SELECT_TOPK, IA_SELECT_EPS = 0, 1
IA_SELECT_TERM1_MASS_EXP = 0x100   # OR-ed into the mode
IA_GEOM_KBAR_BF16 = 1              # ia_geom.reserved flag: k_bar stored in bf16
IA_GEOM_DIAG_ELL = 2               # ia_geom.reserved flag: the selection uses the (w, rho) bound
IA_GEOM_PACKED_BOUNDS = 4          # ia_geom.reserved flag: k_max holds (k_max[d], k_min[d]) pairs, k_min is unused
IA_REP_SPARSE_ONLY, IA_REP_HYBRID = 0, 1
ABI_VERSION = 3
# masks of the device status word (ia_read_device_status)
IA_DEV_STATUS_SELECT_WAIT, IA_DEV_STATUS_GEMM_WAIT, IA_DEV_STATUS_PEER_WAIT, IA_DEV_STATUS_BAD_INDEX = 1, 2, 4, 8


class Geom(Structure):
    _fields_ = [
        ("batch", c_int32), ("n_kv_heads", c_int32), ("group_size", c_int32), ("head_dim", c_int32),
        ("page_size", c_int32), ("block_size", c_int32), ("max_pages", c_int32), ("max_blocks", c_int32),
        ("dtype", c_int32), ("reserved", c_int32), ("n_pool_pages", c_int32), ("reserved2", c_int32),
        ("pool_page_stride", c_int64), ("pool_head_stride", c_int64),
    ]


class Summaries(Structure):
    _fields_ = [("k_bar", c_void_p), ("k_max", c_void_p), ("k_min", c_void_p), ("v_bar", c_void_p),
                ("v_norm_max", c_void_p), ("w", c_void_p), ("rho", c_void_p)]


class SelectAux(Structure):
    _fields_ = [("score", c_void_p), ("z", c_void_p), ("s", c_void_p), ("delta", c_void_p),
                ("globals", c_void_p)]


class PeerExchange(Structure):
    _fields_ = [("n_ranks", c_int32), ("my_rank", c_int32), ("gather", c_void_p * 8), ("flags", c_void_p * 8),
                ("chunk_floats", c_int64), ("lse_offset", c_int64), ("step_counter", c_void_p),
                ("grid_counter", c_void_p)]


class SelectExchange(Structure):
    _fields_ = [("n_ranks", c_int32), ("my_rank", c_int32), ("norm", c_void_p * 8), ("cand", c_void_p * 8),
                ("flags", c_void_p * 8), ("step_counter", c_void_p), ("grid_counter", c_void_p)]


# name -> (restype, argtypes); mirrors include/interattn_b200.h one to one
SIGNATURES = {
    "ia_abi_version": (c_int, []),
    "ia_last_decode_fused": (c_int, []),
    "ia_set_fused_step": (c_int, [c_int]),
    "ia_last_step_phases": (c_int, [POINTER(ctypes.c_double), POINTER(ctypes.c_double)]),
    "ia_last_error_string": (c_char_p, []),
    "ia_read_device_status": (c_int, [POINTER(c_int)]),
    "ia_build_summaries": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, POINTER(Geom), POINTER(Summaries), c_void_p]),
    "ia_update_summaries": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, POINTER(Geom), POINTER(Summaries),
                                    c_void_p]),
    "ia_select": (c_int, [c_void_p, POINTER(Summaries), c_void_p, POINTER(Geom), c_int, c_int, c_float, c_int,
                          c_void_p, c_void_p, POINTER(SelectAux), c_void_p]),
    "ia_select_split": (c_int, [c_void_p, POINTER(Summaries), c_void_p, POINTER(Geom), c_int, c_int, c_int, c_int,
                                c_void_p, c_void_p, POINTER(SelectAux), POINTER(SelectExchange), c_void_p]),
    "ia_sparse_decode": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_int, POINTER(Summaries), c_void_p, POINTER(Geom), c_int, c_int, c_int, c_int,
                                 c_int, c_void_p, c_void_p, c_void_p]),
    "ia_finalize": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p]),
    "ia_workspace_bytes": (c_int64, [POINTER(Geom), c_int, c_int, c_int]),
    "ia_suggest_splits": (c_int, [POINTER(Geom), c_int]),
    "ia_decode_attention": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, POINTER(Summaries),
                                    POINTER(Geom), c_int, c_int, c_float, c_int, c_int, c_int, c_void_p, c_int64,
                                    c_void_p, c_void_p, c_void_p, c_void_p]),
    "ia_decode_attention_timed": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          POINTER(Summaries), POINTER(Geom), c_int, c_int, c_float, c_int, c_int,
                                          c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                                          POINTER(c_void_p), c_void_p]),
    "ia_decode_attention_host": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         POINTER(Summaries), POINTER(Geom), c_int, c_int, c_float, c_int, c_int,
                                         c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "ia_noalloc_scratch_bytes": (c_int64, []),
    "ia_decode_attention_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                            POINTER(Summaries), POINTER(Geom), c_int, c_int, c_float, c_int, c_int,
                                            c_int, c_void_p, c_void_p]),
    "ia_sparse_decode_exchange": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_int, POINTER(Summaries), c_void_p, POINTER(Geom), c_int, c_int,
                                          c_int, c_int, c_int, POINTER(PeerExchange), c_void_p]),
    "ia_finalize_exchange": (c_int, [POINTER(PeerExchange), c_int, c_int, c_int, c_void_p, c_int, c_void_p]),
    "ia_finalize_gathered": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_int, c_void_p, c_int, c_void_p]),
    "ia_llama_add_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "ia_llama_rope_append": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int64,
                                     c_int64, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "ia_llama_silu_mul": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "ia_llama_argmax": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "ia_llama_gemm_packed_bytes": (c_int64, [c_int, c_int]),
    "ia_llama_gemm_pack": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "ia_llama_gemm_workspace_bytes": (c_int64, [c_int]),
    "ia_llama_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int64, c_void_p]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library (once) and bind every declared symbol."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m interattn_b200.build` "
            "(there is no CPU or PyTorch fallback for these operators)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    got = lib.ia_abi_version()
    if got != ABI_VERSION:
        raise ImportError(f"libinterattn_b200.so has ABI {got}, this package expects {ABI_VERSION}")
    _lib = lib
    return lib


def check(status: int) -> None:
    """Turn a non-zero status into the exception the reference would raise:
    ValueError for argument / shape problems, RuntimeError for CUDA failures."""
    if status == IA_OK:
        return
    msg = load().ia_last_error_string().decode("utf-8", "replace")
    if status in (IA_ERR_BAD_ARG, IA_ERR_UNSUPPORTED):
        raise ValueError(f"interattn_b200: {msg}")
    raise RuntimeError(f"interattn_b200: {msg} (status {status})")
