"""Host-side NF4 group-64 encode/decode through the library's C++ codec.

Bit-exact with the reference writer (internal/nf4/nf4.go:46-121) and its Python
restatement (gpu/tests/nf4_oracle.py:119-187); multi-threaded, so a random-init
model of billions of weights quantizes in seconds. Arrays are numpy, on the host.
"""

from __future__ import annotations

import ctypes

import numpy as np

from gpu.nf4 import _lib
from gpu.nf4.plan import GROUP_SIZE, k_pad

__all__ = ["encode_nf4", "decode_nf4", "encode_nf4_device"]


def encode_nf4(w: np.ndarray, *, threads: int = 0) -> tuple[np.ndarray, np.ndarray]:
    """float32 ``[M, K]`` -> (packed uint8 ``[M, K_pad/2]``, scale float16 ``[M, K_pad/64]``)."""
    if w.dtype != np.float32 or w.ndim != 2:
        raise TypeError(f"encode wants float32 [M, K], got {w.dtype} {w.shape}")
    w = np.ascontiguousarray(w)
    m, k = w.shape
    kp = k_pad(k)
    packed = np.empty((m, kp // 2), dtype=np.uint8)
    scale = np.empty((m, kp // GROUP_SIZE), dtype=np.uint16)
    rc = _lib.load().chr_nf4_encode_f32(
        w.ctypes.data_as(ctypes.c_void_p), m, k, packed.ctypes.data_as(ctypes.c_void_p),
        scale.ctypes.data_as(ctypes.c_void_p), int(threads),
    )
    if rc == -8:
        raise ValueError("NaN/Inf in encode input")
    _lib.check(rc, "chr_nf4_encode_f32")
    return packed, scale.view(np.float16)


def decode_nf4(packed: np.ndarray, scale: np.ndarray, m: int, k: int, *, threads: int = 0) -> np.ndarray:
    """Packed blobs -> float32 ``[M, K]`` (pad columns dropped)."""
    kp = k_pad(k)
    if packed.dtype != np.uint8 or packed.shape != (m, kp // 2):
        raise ValueError(f"packed must be uint8 {(m, kp // 2)}, got {packed.dtype} {packed.shape}")
    if scale.dtype != np.float16 or scale.shape != (m, kp // GROUP_SIZE):
        raise ValueError(f"scale must be float16 {(m, kp // GROUP_SIZE)}")
    packed = np.ascontiguousarray(packed)
    scale = np.ascontiguousarray(scale)
    out = np.empty((m, k), dtype=np.float32)
    rc = _lib.load().chr_nf4_decode_f32(
        packed.ctypes.data_as(ctypes.c_void_p), scale.ctypes.data_as(ctypes.c_void_p), m, k,
        out.ctypes.data_as(ctypes.c_void_p), int(threads),
    )
    _lib.check(rc, "chr_nf4_decode_f32")
    return out


def encode_nf4_device(w):
    """CUDA float32 ``[M, K]`` -> (packed uint8, scale float16) on the same device.

    One warp per group; bit-identical to :func:`encode_nf4`.
    """
    import torch

    if not w.is_cuda or w.dtype is not torch.float32 or w.dim() != 2:
        raise TypeError("encode_nf4_device wants a CUDA float32 [M, K] tensor")
    w = w.contiguous()
    m, k = int(w.shape[0]), int(w.shape[1])
    kp = k_pad(k)
    packed = torch.empty((m, kp // 2), dtype=torch.uint8, device=w.device)
    scale = torch.empty((m, kp // GROUP_SIZE), dtype=torch.float16, device=w.device)
    status = torch.zeros((), dtype=torch.int32, device=w.device)
    rc = _lib.load().chr_nf4_encode_dev(
        ctypes.c_void_p(w.data_ptr()), m, k, ctypes.c_void_p(packed.data_ptr()),
        ctypes.c_void_p(scale.data_ptr()), ctypes.c_void_p(status.data_ptr()),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
    )
    _lib.check(rc, "chr_nf4_encode_dev")
    if int(status.item()) != 0:
        raise ValueError("NaN/Inf in encode input")
    return packed, scale
