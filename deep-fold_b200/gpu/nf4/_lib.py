"""ctypes binding of ``libchr_nf4.so`` (the C ABI declared in ``include/chr_gpu.h``).

There is no fallback: if the library is missing or an entry point is absent the
import of any op fails loudly. Build it with ``python deep-fold_b200/csrc/build.py``.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_void_p
from pathlib import Path

_DIR = Path(__file__).resolve().parent
#: ``CHR_NF4_LIB`` points at another build of the same C ABI (A/B of kernel variants).
LIB_PATH = Path(os.environ.get("CHR_NF4_LIB") or _DIR / "libchr_nf4.so")


class ChrNf4Dev(Structure):
    """Mirror of ``chr_nf4_dev_t``; field order is frozen."""

    _fields_ = [
        ("M", c_int32),
        ("K", c_int32),
        ("K_pad", c_int32),
        ("packed", c_void_p),
        ("scale", c_void_p),
    ]


class ChrNf4Plan(Structure):
    """Mirror of ``chr_nf4_plan_t``."""

    _fields_ = [
        ("path", c_int32),
        ("grid_x", c_int32),
        ("grid_y", c_int32),
        ("block", c_int32),
        ("bm", c_int32),
        ("bk", c_int32),
        ("n_ktiles", c_int32),
        ("tiles_per_split", c_int32),
        ("ctas", c_int32),
        ("smem_bytes", c_int32),
        ("ws_floats", c_int64),
    ]


AR_MAX_RANKS = 8
AR_MAX_CTAS = 256


class ChrNf4Peers(Structure):
    """Mirror of ``chr_nf4_peers_t``."""

    _fields_ = [("rank", c_int32), ("world", c_int32), ("shape_k_pad", c_int32),
                ("capacity", c_int32), ("recv", c_void_p * AR_MAX_RANKS),
                ("flags", c_void_p * AR_MAX_RANKS), ("epoch", c_void_p), ("status", c_void_p)]


_DEV = POINTER(ChrNf4Dev)

# name -> (restype, argtypes); every symbol include/chr_gpu.h declares.
SIGNATURES = {
    "chr_nf4_gemm": (c_int, [_DEV, c_void_p, c_void_p, c_int32, c_void_p]),
    "chr_nf4_gemm_plan": (c_int, [_DEV, c_int32, c_int32, POINTER(ChrNf4Plan)]),
    "chr_nf4_gemm_ws": (c_int, [_DEV, c_void_p, c_void_p, c_int32, c_void_p, c_int64, c_void_p]),
    "chr_nf4_gemm_ws_max": (
        c_int,
        [_DEV, c_void_p, c_void_p, c_int32, c_void_p, c_int64, c_void_p, c_int32],
    ),
    "chr_nf4_set_tuning": (None, [c_int32, c_int32, c_int32]),
    "chr_nf4_gemv": (c_int, [_DEV, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float]),
    "chr_nf4_gemv_f32": (c_int, [_DEV, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float]),
    "chr_nf4_gemv_shape": (c_int, [c_int32, c_int32, c_int32, POINTER(c_int32)]),
    "chr_nf4_gemv_status": (c_int, []),
    "chr_nf4_gemv_n_ws": (c_int64, [_DEV, c_int32]),
    "chr_nf4_gemv_n": (
        c_int, [_DEV, c_void_p, c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]
    ),
    "chr_nf4_set_peer_polls": (None, [ctypes.c_uint32]),
    "chr_nf4_gemv_allreduce": (
        c_int, [_DEV, c_void_p, c_void_p, POINTER(ChrNf4Peers), c_void_p, c_void_p]
    ),
    "chr_nf4_gemv_qkv": (
        c_int,
        [_DEV, _DEV, _DEV, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_void_p, c_float],
    ),
    "chr_nf4_gemv_swiglu": (
        c_int, [_DEV, _DEV, c_void_p, c_void_p, c_void_p, c_void_p, c_float]
    ),
    "chr_nf4_rope_kv": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_int32, c_int32, c_int32, c_int32, c_void_p],
    ),
    "chr_nf4_attn": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32,
         c_int32, c_int32, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_int32],
    ),
    "chr_nf4_attn_batch": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32,
         c_int32, c_int32, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_int32],
    ),
    "chr_nf4_attn_noalloc": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32,
         c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32],
    ),
    "chr_nf4_rms": (c_int, [c_void_p, c_void_p, c_void_p, c_int32, c_float, c_void_p]),
    "chr_nf4_version": (c_char_p, []),
    "chr_nf4_gemm_status": (c_int, []),
    "chr_nf4_set_pdl": (None, [c_int32]),
    "chr_nf4_gemm_rows_ws": (c_int64, [_DEV, c_int32]),
    "chr_nf4_gemm_rows": (
        c_int, [_DEV, c_void_p, c_void_p, c_int32, c_void_p, c_int64, c_void_p]
    ),
    "chr_nf4_gemm_rows_add": (
        c_int, [_DEV, c_void_p, c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]
    ),
    "chr_nf4_embed_rows": (
        c_int, [_DEV, c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
    ),
    "chr_nf4_pick_commit": (
        c_int,
        [c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p],
    ),
    "chr_nf4_pick_commit_batch": (
        c_int,
        [c_void_p, c_int64, c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
         c_void_p, c_void_p],
    ),
    "chr_nf4_pick_commit_tp": (
        c_int,
        [c_void_p, c_int32, c_int32, POINTER(ChrNf4Peers), c_void_p, c_void_p, c_void_p, c_void_p,
         c_int64, c_void_p, c_void_p],
    ),
    "chr_nf4_rms_rows": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int32, c_int32, c_float,
                                 c_void_p]),
    "chr_nf4_rope_kv_rows": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_void_p],
    ),
    "chr_nf4_attn_prefill": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_int32,
         c_int32, c_float, c_void_p],
    ),
    "chr_nf4_silu_mul": (c_int, [c_void_p, c_void_p, c_int32, c_int32, c_void_p]),
    "chr_nf4_encode_f32": (c_int, [c_void_p, c_int32, c_int32, c_void_p, c_void_p, c_int32]),
    "chr_nf4_decode_f32": (c_int, [c_void_p, c_void_p, c_int32, c_int32, c_void_p, c_int32]),
    "chr_nf4_encode_dev": (
        c_int, [c_void_p, c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p]
    ),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the library once and type every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.is_file():
        raise RuntimeError(
            f"{LIB_PATH} is missing: the NF4 ops have no fallback. "
            "Build it with `python deep-fold_b200/csrc/build.py`."
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise RuntimeError(f"{LIB_PATH.name} does not export {name}") from exc
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


_RC_TEXT = {
    0: "ok",
    -1: "null pointer",
    -2: "N out of range (live 1..32, plan 1..64)",
    -3: "invalid M/K or null packed/scale",
    -4: "K_pad != 64*ceil(K/64)",
    -5: "packed or x not 16-byte aligned",
    -6: "CUDA launch / func attribute failed",
    -7: "split-K workspace smaller than the plan asked for",
    -8: "non-finite value in encoder input",
}


def rc_text(rc: int) -> str:
    return _RC_TEXT.get(int(rc), "unknown error")


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed ({rc}): {rc_text(rc)}")
