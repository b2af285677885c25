"""NF4 fused-dequant ops for B200 behind deep-fold's ``gpu.nf4`` surface.

Same function names, argument order and meaning as the reference module
(gpu/nf4/__init__.py:151-372); the implementation is a ctypes call into
``libchr_nf4.so`` (C ABI, ``include/chr_gpu.h``) on torch's current stream.
Argument validation mirrors the reference binding (gpu/nf4/bindings.cpp:35-503):
wrong device / dtype, undersized blobs, K_pad mismatch and short outputs are
rejected before anything is launched. Torch supplies device memory and the
stream only; every workspace is a caller-visible tensor.

There is no CPU path and no fallback kernel library.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import ChrNf4Dev, ChrNf4Plan
from .plan import LIVE_MAX_N, PLAN_MAX_N, k_pad as _k_pad

__all__ = [
    "ATTN_SPLIT",
    "LIVE_MAX_N",
    "PLAN_MAX_N",
    "nf4_attn",
    "nf4_embed_rows",
    "nf4_gemm",
    "nf4_gemm_rows",
    "nf4_gemm_status",
    "nf4_gemv",
    "nf4_gemv_allreduce",
    "nf4_gemv_f32",
    "nf4_gemv_n",
    "nf4_attn_batch",
    "GEMV_MAX_N",
    "nf4_pick_commit",
    "nf4_pick_commit_tp",
    "nf4_plan",
    "nf4_qkv",
    "nf4_rms",
    "nf4_rms_rows",
    "nf4_rope_kv_rows",
    "nf4_silu_mul",
    "nf4_attn_prefill",
    "nf4_pick_commit_batch",
    "nf4_rope_kv",
    "nf4_set_pdl",
    "nf4_set_tuning",
    "nf4_swiglu",
    "nf4_version",
]

GEMV_MAX_N = 8
ATTN_SPLIT = 32


# --------------------------------------------------------------------------- #
# checks shared by the ops
# --------------------------------------------------------------------------- #
def _fail(msg: str):
    raise RuntimeError(msg)


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _matrix(packed: torch.Tensor, scale: torch.Tensor, M: int, K: int, K_pad: int, name: str = ""):
    """Validate one packed matrix and return (struct, keep-alive tensors)."""
    tag = f"{name} " if name else ""
    if not (packed.is_cuda and scale.is_cuda):
        _fail(f"{tag}packed and scale must be CUDA tensors")
    if packed.dtype is not torch.uint8:
        _fail(f"{tag}packed must be uint8")
    if scale.dtype is not torch.float16:
        _fail(f"{tag}scale must be float16")
    M, K, K_pad = int(M), int(K), int(K_pad)
    if M < 1 or K < 1:
        _fail("M and K must be >= 1")
    want = _k_pad(K)
    if K_pad != want:
        _fail(f"{tag}K_pad must be 64*ceil(K/64) = {want}, got {K_pad}")
    packed = packed.contiguous()
    scale = scale.contiguous()
    if packed.numel() < M * (K_pad // 2):
        _fail(f"{tag}packed has {packed.numel()} bytes, the kernel reads M*K_pad/2 = {M * (K_pad // 2)}")
    if scale.numel() < M * (K_pad // 64):
        _fail(f"{tag}scale has {scale.numel()} elements, the kernel reads M*K_pad/64 = {M * (K_pad // 64)}")
    dev = ChrNf4Dev(M, K, K_pad, packed.data_ptr(), scale.data_ptr())
    return dev, (packed, scale)


def _kvec(x: torch.Tensor, K: int) -> torch.Tensor:
    if not x.is_cuda or x.dtype is not torch.bfloat16:
        _fail("x must be CUDA bfloat16")
    x = x.contiguous()
    if x.dim() == 1 and x.size(0) == K:
        return x
    if x.dim() == 2 and tuple(x.shape) in ((K, 1), (1, K)):
        return x.view(K)
    _fail("x must be [K], [K,1], or [1,K]")


def _out_vec(out: torch.Tensor, M: int, what: str = "out") -> torch.Tensor:
    if out is None:
        _fail(f"{what} must be defined")
    if not out.is_cuda or out.dtype is not torch.bfloat16:
        _fail(f"{what} must be CUDA bfloat16")
    if not out.is_contiguous():
        _fail(f"{what} must be contiguous")
    if out.numel() < M:
        _fail(f"{what} too small")
    return out


def _opt_bf16(t: torch.Tensor | None, n: int, what: str, exact: bool) -> torch.Tensor | None:
    if t is None or t.numel() == 0:
        return None
    if not t.is_cuda:
        _fail(f"{what} must be CUDA")
    if exact and t.numel() != n:
        _fail(f"{what} numel must equal {n}")
    if not exact and t.numel() < n:
        _fail(f"{what} too small")
    t = t.contiguous()
    return t if t.dtype is torch.bfloat16 else t.to(torch.bfloat16)


# --------------------------------------------------------------------------- #
# GEMM (prefill)
# --------------------------------------------------------------------------- #
def nf4_gemm(
    packed: torch.Tensor,
    scale: torch.Tensor,
    x: torch.Tensor,
    M: int,  # noqa: N803
    K: int,  # noqa: N803
    K_pad: int,  # noqa: N803
    max_n: int = LIVE_MAX_N,
) -> torch.Tensor:
    """``y[M,N] = dequant(W) @ x`` with ``x`` bf16 ``[K, N]`` or ``[K]``; returns bf16 ``[M, N]``."""
    n = 1 if x.dim() == 1 else int(x.size(-1))
    cap = int(max_n)
    if cap < 1 or cap > PLAN_MAX_N:
        _fail(f"chr_nf4_gemm: max_n={cap} not in 1..{PLAN_MAX_N}")
    if n < 1 or n > cap:
        _fail(f"chr_nf4_gemm: N={n} not in 1..{cap} (host must chunk N>{LIVE_MAX_N})")
    if not x.is_cuda:
        _fail("packed, scale, and x must be CUDA tensors")
    if x.dtype is not torch.bfloat16:
        _fail("x must be bfloat16")
    dev, keep = _matrix(packed, scale, M, K, K_pad)
    x = x.contiguous()
    if x.dim() == 1:
        x = x.unsqueeze(1)
    if x.dim() != 2:
        _fail("x must be [K, N] or [K]")
    if x.size(0) != int(K):
        _fail("x.size(0) must equal K")
    lib = _lib.load()
    y = torch.empty((int(M), n), dtype=torch.bfloat16, device=x.device)
    pl = ChrNf4Plan()
    _lib.check(lib.chr_nf4_gemm_plan(ctypes.byref(dev), n, 1, ctypes.byref(pl)), "chr_nf4_gemm_plan")
    ws = None
    if pl.ws_floats > 0:
        ws = torch.empty(int(pl.ws_floats), dtype=torch.float32, device=x.device)
    rc = lib.chr_nf4_gemm_ws_max(
        ctypes.byref(dev), _ptr(x), _ptr(y), n, _ptr(ws), int(pl.ws_floats), _stream(), cap
    )
    _lib.check(rc, "chr_nf4_gemm")
    del keep
    return y


def nf4_gemm_rows(
    packed: torch.Tensor,
    scale: torch.Tensor,
    x_rows: torch.Tensor,
    M: int,  # noqa: N803
    K: int,  # noqa: N803
    K_pad: int,  # noqa: N803
    out: torch.Tensor | None = None,
    bias: torch.Tensor | None = None,
    add: torch.Tensor | None = None,
) -> torch.Tensor:
    """``y[N, M] = x_rows[N, K] @ dequant(W).T (+ bias[M]) (+ add[N, M])`` on the tensor
    cores, any ``N >= 1``; bias and residual join the FP32 sum before its one rounding.

    Activations keep their natural ``[tokens, features]`` layout on both sides; ``add``
    may alias ``out``. Needs ``K % 8 == 0`` (TMA row pitch); other shapes go through
    :func:`nf4_gemm`.
    """
    if not x_rows.is_cuda or x_rows.dtype is not torch.bfloat16:
        _fail("x_rows must be CUDA bfloat16")
    if x_rows.dim() != 2 or x_rows.size(1) != int(K):
        _fail("x_rows must be [N, K]")
    if int(K) % 8:
        _fail("nf4_gemm_rows needs K % 8 == 0")
    dev, keep = _matrix(packed, scale, M, K, K_pad)
    x_rows = x_rows.contiguous()
    n = int(x_rows.size(0))
    if n < 1:
        _fail("x_rows must be non-empty")
    if out is None:
        out = torch.empty((n, int(M)), dtype=torch.bfloat16, device=x_rows.device)
    else:
        _out_vec(out, n * int(M))
    lib = _lib.load()
    need = int(lib.chr_nf4_gemm_rows_ws(ctypes.byref(dev), n))
    ws = torch.empty(need, dtype=torch.float32, device=x_rows.device) if need > 0 else None
    bias_t = _opt_bf16(bias, int(M), "bias", exact=True)
    add_t = None
    if add is not None:
        if (not add.is_cuda or add.dtype is not torch.bfloat16 or not add.is_contiguous()
                or add.numel() != n * int(M)):
            _fail("add must be contiguous CUDA bfloat16 [N, M]")
        add_t = add
    rc = lib.chr_nf4_gemm_rows_add(ctypes.byref(dev), _ptr(x_rows), _ptr(out), n, _ptr(bias_t),
                                   _ptr(add_t), _ptr(ws), need, _stream())
    _lib.check(rc, "chr_nf4_gemm_rows_add")
    del keep
    return out


def nf4_plan(
    M: int,  # noqa: N803
    K: int,  # noqa: N803
    N: int = 1,  # noqa: N803
    *,
    K_pad: int | None = None,  # noqa: N803
    have_ws: bool = True,
) -> dict:
    """The grid ``chr_nf4_gemm`` would launch, from the library's planner. No launch."""
    kp = _k_pad(K) if K_pad is None else int(K_pad)
    dev = ChrNf4Dev(int(M), int(K), kp, None, None)
    pl = ChrNf4Plan()
    rc = _lib.load().chr_nf4_gemm_plan(ctypes.byref(dev), int(N), 1 if have_ws else 0, ctypes.byref(pl))
    _lib.check(rc, "chr_nf4_gemm_plan")
    return {name: int(getattr(pl, name)) for name, _ in ChrNf4Plan._fields_}


def nf4_set_tuning(path: int = 0, split_k: int = 0, one_wave: int = 0) -> None:
    """Planner override for one process: ``path`` 0 auto / 1 tensor-core / 2 SIMT,
    ``split_k`` 0 auto or forced, ``one_wave`` 0 = this GPU's SM count."""
    _lib.load().chr_nf4_set_tuning(int(path), int(split_k), int(one_wave))


def nf4_set_pdl(on: bool = True) -> None:
    """Programmatic dependent launch for the decode-chain kernels (default on)."""
    _lib.load().chr_nf4_set_pdl(1 if on else 0)


def nf4_gemm_status() -> int:
    """Read and clear the tensor-core GEMM's status word (0 = healthy). Synchronises."""
    return int(_lib.load().chr_nf4_gemm_status())


def nf4_version() -> str:
    return _lib.load().chr_nf4_version().decode()


# --------------------------------------------------------------------------- #
# GEMV family (decode)
# --------------------------------------------------------------------------- #
def nf4_gemv(
    packed: torch.Tensor,
    scale: torch.Tensor,
    x: torch.Tensor,
    M: int,  # noqa: N803
    K: int,  # noqa: N803
    K_pad: int,  # noqa: N803
    out: torch.Tensor | None = None,
    add: torch.Tensor | None = None,
    rms_w: torch.Tensor | None = None,
    rms_eps: float = 1e-6,
) -> torch.Tensor:
    """N=1 GEMV: ``y[M] = dequant(W) @ x (+ add)``; ``out`` and ``add`` may alias."""
    n = 1 if x.dim() == 1 else int(x.size(-1))
    if x.dim() == 2 and x.size(0) == 1 and x.size(1) == int(K):
        n = 1
    if n != 1:
        _fail(f"chr_nf4_gemv is N=1 only, got N={n}")
    dev, keep = _matrix(packed, scale, M, K, K_pad)
    xk = _kvec(x, int(K))
    if out is not None:
        y = _out_vec(out, int(M))
    else:
        y = torch.empty((int(M), 1), dtype=torch.bfloat16, device=x.device)
    add_t = _opt_bf16(add, int(M), "add", exact=False)
    rms_t = _opt_bf16(rms_w, int(K), "rms_w", exact=True)
    rc = _lib.load().chr_nf4_gemv(
        ctypes.byref(dev), _ptr(xk), _ptr(y), _stream(), _ptr(add_t), _ptr(rms_t), float(rms_eps)
    )
    _lib.check(rc, "chr_nf4_gemv")
    del keep
    return y


_GEMV_N_WS: dict = {}


def nf4_gemv_n(
    packed: torch.Tensor,
    scale: torch.Tensor,
    x_rows: torch.Tensor,
    M: int,  # noqa: N803
    K: int,  # noqa: N803
    K_pad: int,  # noqa: N803
    out: torch.Tensor | None = None,
    add: torch.Tensor | None = None,
    bias: torch.Tensor | None = None,
) -> torch.Tensor:
    """``y[N, M] = x_rows[N, K] @ dequant(W).T (+ bias) (+ add)`` for ``N`` in 1..8 on the
    CUDA cores, with the GEMV's numerics (FP32 weights). ``out`` and ``add`` may alias.
    The FP32 split-K workspace large K needs is kept per (device, size) and reused."""
    if not x_rows.is_cuda or x_rows.dtype is not torch.bfloat16:
        _fail("x_rows must be CUDA bfloat16")
    if x_rows.dim() != 2 or x_rows.size(1) != int(K):
        _fail("x_rows must be [N, K]")
    n = int(x_rows.size(0))
    if not 1 <= n <= GEMV_MAX_N:
        _fail(f"nf4_gemv_n takes 1..{GEMV_MAX_N} rows, got {n}")
    dev, keep = _matrix(packed, scale, M, K, K_pad)
    x_rows = x_rows.contiguous()
    if out is None:
        out = torch.empty((n, int(M)), dtype=torch.bfloat16, device=x_rows.device)
    else:
        _out_vec(out, n * int(M))
    add_t = _opt_bf16(add, n * int(M), "add", exact=False)
    bias_t = _opt_bf16(bias, int(M), "bias", exact=True)
    lib = _lib.load()
    need = int(lib.chr_nf4_gemv_n_ws(ctypes.byref(dev), n))
    ws = None
    if need:
        key = (x_rows.device, need)
        ws = _GEMV_N_WS.get(key)
        if ws is None:
            ws = _GEMV_N_WS[key] = torch.empty(need, dtype=torch.float32, device=x_rows.device)
    rc = lib.chr_nf4_gemv_n(ctypes.byref(dev), _ptr(x_rows), _ptr(out), n, _ptr(add_t), _ptr(bias_t),
                            _ptr(ws), need, _stream())
    _lib.check(rc, "chr_nf4_gemv_n")
    del keep
    return out


def nf4_gemv_f32(
    packed: torch.Tensor,
    scale: torch.Tensor,
    x: torch.Tensor,
    M: int,  # noqa: N803
    K: int,  # noqa: N803
    K_pad: int,  # noqa: N803
    out: torch.Tensor,
    add: torch.Tensor | None = None,
    rms_w: torch.Tensor | None = None,
    rms_eps: float = 1e-6,
) -> torch.Tensor:
    """:func:`nf4_gemv` with the FP32 sum kept unrounded in ``out`` (float32, numel >= M)."""
    dev, keep = _matrix(packed, scale, M, K, K_pad)
    xk = _kvec(x, int(K))
    if not out.is_cuda or out.dtype is not torch.float32 or not out.is_contiguous():
        _fail("out must be contiguous CUDA float32")
    if out.numel() < int(M):
        _fail("out too small")
    add_t = _opt_bf16(add, int(M), "add", exact=False)
    rms_t = _opt_bf16(rms_w, int(K), "rms_w", exact=True)
    rc = _lib.load().chr_nf4_gemv_f32(
        ctypes.byref(dev), _ptr(xk), _ptr(out), _stream(), _ptr(add_t), _ptr(rms_t), float(rms_eps)
    )
    _lib.check(rc, "chr_nf4_gemv_f32")
    del keep
    return out


def nf4_gemv_allreduce(
    packed: torch.Tensor,
    scale: torch.Tensor,
    x: torch.Tensor,
    M: int,  # noqa: N803
    K: int,  # noqa: N803
    K_pad: int,  # noqa: N803
    y: torch.Tensor,
    peers,
    add: torch.Tensor | None = None,
) -> torch.Tensor:
    """Row-split shard: ``y += sum over ranks of (W_shard @ x_shard)`` in one launch per rank.

    ``peers`` is a ``ChrNf4Peers`` whose buffers are mapped on every rank (see
    ``gpu.decodev2.tp.PeerExchange``); ``y`` is the bf16 residual, updated in place and
    identical on all ranks afterwards; ``add`` an optional bf16 bias (pass it on one rank)."""
    dev, keep = _matrix(packed, scale, M, K, K_pad)
    xk = _kvec(x, int(K))
    _out_vec(y, int(M))
    add_t = _opt_bf16(add, int(M), "add", exact=False)
    rc = _lib.load().chr_nf4_gemv_allreduce(
        ctypes.byref(dev), _ptr(xk), _ptr(y), ctypes.byref(peers), _ptr(add_t), _stream()
    )
    _lib.check(rc, "chr_nf4_gemv_allreduce")
    del keep
    return y


def nf4_qkv(
    q_packed: torch.Tensor,
    q_scale: torch.Tensor,
    k_packed: torch.Tensor,
    k_scale: torch.Tensor,
    v_packed: torch.Tensor,
    v_scale: torch.Tensor,
    x: torch.Tensor,
    Mq: int,  # noqa: N803
    Mk: int,  # noqa: N803
    Mv: int,  # noqa: N803
    K: int,  # noqa: N803
    K_pad: int,  # noqa: N803
    out_q: torch.Tensor,
    out_k: torch.Tensor,
    out_v: torch.Tensor,
    q_bias: torch.Tensor | None = None,
    k_bias: torch.Tensor | None = None,
    v_bias: torch.Tensor | None = None,
    rms_w: torch.Tensor | None = None,
    rms_eps: float = 1e-6,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """One launch: q/k/v GEMVs sharing ``x`` (+ bias each). Writes ``out_*``."""
    dq, kq = _matrix(q_packed, q_scale, Mq, K, K_pad, "q")
    dk, kk = _matrix(k_packed, k_scale, Mk, K, K_pad, "k")
    dv, kv = _matrix(v_packed, v_scale, Mv, K, K_pad, "v")
    xk = _kvec(x, int(K))
    yq = _out_vec(out_q, int(Mq), "out_q")
    yk = _out_vec(out_k, int(Mk), "out_k")
    yv = _out_vec(out_v, int(Mv), "out_v")
    bq = _opt_bf16(q_bias, int(Mq), "bias", exact=True)
    bk = _opt_bf16(k_bias, int(Mk), "bias", exact=True)
    bv = _opt_bf16(v_bias, int(Mv), "bias", exact=True)
    rms_t = _opt_bf16(rms_w, int(K), "rms_w", exact=True)
    rc = _lib.load().chr_nf4_gemv_qkv(
        ctypes.byref(dq), ctypes.byref(dk), ctypes.byref(dv), _ptr(xk), _ptr(yq), _ptr(yk),
        _ptr(yv), _ptr(bq), _ptr(bk), _ptr(bv), _stream(), _ptr(rms_t), float(rms_eps),
    )
    _lib.check(rc, "chr_nf4_gemv_qkv")
    del kq, kk, kv
    return yq, yk, yv


def nf4_swiglu(
    g_packed: torch.Tensor,
    g_scale: torch.Tensor,
    u_packed: torch.Tensor,
    u_scale: torch.Tensor,
    x: torch.Tensor,
    M: int,  # noqa: N803
    K: int,  # noqa: N803
    K_pad: int,  # noqa: N803
    out: torch.Tensor,
    rms_w: torch.Tensor | None = None,
    rms_eps: float = 1e-6,
) -> torch.Tensor:
    """One launch: ``silu(gate @ x) * (up @ x)`` into ``out``."""
    dg, kg = _matrix(g_packed, g_scale, M, K, K_pad, "gate")
    du, ku = _matrix(u_packed, u_scale, M, K, K_pad, "up")
    xk = _kvec(x, int(K))
    y = _out_vec(out, int(M))
    rms_t = _opt_bf16(rms_w, int(K), "rms_w", exact=True)
    rc = _lib.load().chr_nf4_gemv_swiglu(
        ctypes.byref(dg), ctypes.byref(du), _ptr(xk), _ptr(y), _stream(), _ptr(rms_t), float(rms_eps)
    )
    _lib.check(rc, "chr_nf4_gemv_swiglu")
    del kg, ku
    return y


# --------------------------------------------------------------------------- #
# RoPE / attention / RMSNorm
# --------------------------------------------------------------------------- #
def _heads(q: torch.Tensor, hd: int, what: str) -> int:
    if q.dim() == 3:
        if q.size(0) != 1:
            _fail(f"{what} batch must be 1")
        if q.size(2) != hd:
            _fail(f"{what} head_dim")
        return int(q.size(1))
    if q.dim() != 2:
        _fail(f"{what} must be [n,hd] or [1,n,hd]")
    if q.size(1) != hd:
        _fail(f"{what} head_dim")
    return int(q.size(0))


def _cache_dims(k: torch.Tensor, v: torch.Tensor) -> tuple[int, int, int]:
    if k.dim() != 3 or v.dim() != 3:
        _fail("cache must be [max_seq,n_kv,hd]")
    if tuple(k.shape) != tuple(v.shape):
        _fail("v cache shape mismatch")
    if not (k.is_contiguous() and v.is_contiguous()):
        _fail("cache must be contiguous")
    return int(k.size(0)), int(k.size(1)), int(k.size(2))


def _position(position: torch.Tensor) -> torch.Tensor:
    if not position.is_cuda or position.numel() != 1 or position.dtype is not torch.int64:
        _fail("position must be a CUDA int64 scalar")
    return position.contiguous()


def nf4_rope_kv(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    cos: torch.Tensor,
    sin: torch.Tensor,
    position: torch.Tensor,
) -> None:
    """In-place RoPE on q, k; write k, v into the cache at device ``position``."""
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        _fail("q/k/v must be CUDA")
    if q.dtype is not torch.bfloat16 or k.dtype is not torch.bfloat16 or v.dtype is not torch.bfloat16:
        _fail("q/k/v must be bf16")
    if not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()):
        _fail("q/k/v must be contiguous (rotated in place)")
    max_seq, n_kv, hd = _cache_dims(k_cache, v_cache)
    if tuple(cos.shape) != (max_seq, hd) or tuple(sin.shape) != (max_seq, hd):
        _fail("cos/sin shape")
    n_q = _heads(q, hd, "q")
    if _heads(k, hd, "k") != n_kv or _heads(v, hd, "v") != n_kv:
        _fail("k/v heads")
    pos = _position(position)
    rc = _lib.load().chr_nf4_rope_kv(
        _ptr(q), _ptr(k), _ptr(v), _ptr(k_cache), _ptr(v_cache), _ptr(cos.contiguous()),
        _ptr(sin.contiguous()), _ptr(pos), n_q, n_kv, hd, max_seq, _stream(),
    )
    _lib.check(rc, "chr_nf4_rope_kv")


def nf4_attn_batch(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out: torch.Tensor,
    valid_len: torch.Tensor,
    scale: float,
    ws: torch.Tensor,
    n_split: int,
    k_act: torch.Tensor,
    v_act: torch.Tensor,
    cos: torch.Tensor,
    sin: torch.Tensor,
    position: torch.Tensor,
) -> None:
    """``nf4_attn`` for ``B`` independent sequences in one launch: ``q [B, n_q, hd]``,
    ``k``/``v`` caches ``[B, max_seq, n_kv, hd]``, ``k_act``/``v_act [B, n_kv, hd]``,
    ``out [B, n_q*hd]``, ``valid_len`` int32 ``[B]``, ``position`` int64 ``[B]``."""
    for t, what in ((q, "q"), (k, "k"), (v, "v"), (out, "out"), (k_act, "k_act"), (v_act, "v_act"),
                    (cos, "cos"), (sin, "sin")):
        if not t.is_cuda or t.dtype is not torch.bfloat16 or not t.is_contiguous():
            _fail(f"{what} must be a contiguous CUDA bf16 tensor")
    if k.dim() != 4 or k.shape != v.shape:
        _fail("caches must be [B, max_seq, n_kv, hd]")
    b, max_seq, n_kv, hd = (int(d) for d in k.shape)
    if q.dim() != 3 or int(q.size(0)) != b or int(q.size(2)) != hd:
        _fail("q must be [B, n_q, hd]")
    n_q = int(q.size(1))
    if out.numel() < b * n_q * hd or k_act.numel() != b * n_kv * hd or v_act.numel() != b * n_kv * hd:
        _fail("out / k_act / v_act sizes")
    if tuple(cos.shape) != (max_seq, hd) or tuple(sin.shape) != (max_seq, hd):
        _fail("cos / sin shape")
    if valid_len.dtype is not torch.int32 or valid_len.numel() != b or not valid_len.is_cuda:
        _fail("valid_len must be CUDA int32 [B]")
    if position.dtype is not torch.int64 or position.numel() != b or not position.is_cuda:
        _fail("position must be CUDA int64 [B]")
    n_split = int(n_split)
    if not 1 <= n_split <= 64:
        _fail("n_split must be 1..64")
    if ws.dtype is not torch.float32 or not ws.is_cuda or ws.numel() < b * n_q * min(n_split, 32) * (hd + 2):
        _fail("attn workspace too small")
    rc = _lib.load().chr_nf4_attn_batch(
        _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(valid_len), _ptr(ws), b, n_q, n_kv, hd, n_split,
        float(scale), _stream(), _ptr(k_act), _ptr(v_act), _ptr(cos), _ptr(sin), _ptr(position),
        max_seq)
    _lib.check(rc, "chr_nf4_attn_batch")


def nf4_attn(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out: torch.Tensor,
    valid_len: torch.Tensor,
    scale: float,
    ws: torch.Tensor | None = None,
    n_split: int = ATTN_SPLIT,
    k_act: torch.Tensor | None = None,
    v_act: torch.Tensor | None = None,
    cos: torch.Tensor | None = None,
    sin: torch.Tensor | None = None,
    position: torch.Tensor | None = None,
) -> None:
    """GQA decode attention over cache rows ``t < valid_len``; see ``chr_nf4_attn``."""
    if not (q.is_cuda and k.is_cuda and v.is_cuda and out.is_cuda):
        _fail("q/k/v/out must be CUDA")
    if q.dtype is not torch.bfloat16:
        _fail("q must be bf16")
    if k.dtype is not torch.bfloat16 or v.dtype is not torch.bfloat16:
        _fail("cache must be bf16")
    q = q.contiguous()
    max_seq, n_kv, hd = _cache_dims(k, v)
    n_q = _heads(q, hd, "q")
    if not out.is_contiguous() or out.dtype is not torch.bfloat16:
        _fail("out must be contiguous bf16")
    if out.numel() < n_q * hd:
        _fail("out too small")
    if not valid_len.is_cuda or valid_len.numel() != 1 or valid_len.dtype is not torch.int32:
        _fail("valid_len must be a CUDA int32 scalar")
    n_split = int(n_split)
    if not 1 <= n_split <= 64:
        _fail("n_split must be 1..64")
    need = n_q * n_split * (hd + 2)
    if ws is None:
        ws = torch.empty(need, device=q.device, dtype=torch.float32)
    if not ws.is_cuda or ws.dtype is not torch.float32 or not ws.is_contiguous():
        _fail("ws must be contiguous CUDA fp32")
    if ws.numel() < need:
        _fail("attn workspace too small")

    def opt(t, what):
        if t is None or t.numel() == 0:
            return None
        if not t.is_cuda or t.dtype is not torch.bfloat16:
            _fail(f"{what} must be CUDA bf16")
        return t.contiguous()

    ka, va = opt(k_act, "k_act"), opt(v_act, "v_act")
    cs, sn = opt(cos, "cos"), opt(sin, "sin")
    for t, what in ((cs, "cos"), (sn, "sin")):
        if t is not None and tuple(t.shape) != (max_seq, hd):
            _fail(f"{what} shape")
    for t, what in ((ka, "k_act"), (va, "v_act")):
        if t is not None and t.numel() != n_kv * hd:
            _fail(f"{what} numel")
    pos = None
    if position is not None and position.numel() == 1:
        pos = _position(position)
    rc = _lib.load().chr_nf4_attn(
        _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(valid_len), _ptr(ws), n_q, n_kv, hd, n_split,
        float(scale), _stream(), _ptr(ka), _ptr(va), _ptr(cs), _ptr(sn), _ptr(pos), max_seq,
    )
    _lib.check(rc, "chr_nf4_attn")


def nf4_rms(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, eps: float) -> None:
    """``y = w * x * rsqrt(mean(x^2)+eps)``; all three bf16 with equal numel."""
    if not (x.is_cuda and w.is_cuda and y.is_cuda):
        _fail("x/w/y must be CUDA")
    if x.dtype is not torch.bfloat16 or w.dtype is not torch.bfloat16:
        _fail("x and w must be bf16")
    if not y.is_contiguous() or y.dtype is not torch.bfloat16:
        _fail("y must be contiguous bf16")
    x = x.contiguous()
    w = w.contiguous()
    n = x.numel()
    if w.numel() != n or y.numel() != n:
        _fail("rms numel mismatch")
    _lib.check(_lib.load().chr_nf4_rms(_ptr(x), _ptr(w), _ptr(y), n, float(eps), _stream()), "chr_nf4_rms")


# --------------------------------------------------------------------------- #
# additive ops
# --------------------------------------------------------------------------- #
def nf4_embed_rows(
    packed: torch.Tensor,
    scale: torch.Tensor,
    ids: torch.Tensor,
    M: int,  # noqa: N803
    K: int,  # noqa: N803
    K_pad: int,  # noqa: N803
    out: torch.Tensor | None = None,
    status: torch.Tensor | None = None,
    position: torch.Tensor | None = None,
    valid_len: torch.Tensor | None = None,
) -> torch.Tensor:
    """Decode rows ``ids`` (CUDA int64) of an NF4 table to bf16 ``[n, K]``."""
    dev, keep = _matrix(packed, scale, M, K, K_pad)
    if not ids.is_cuda or ids.dtype is not torch.int64:
        _fail("ids must be CUDA int64")
    ids = ids.contiguous().view(-1)
    n = int(ids.numel())
    if n < 1:
        _fail("ids must be non-empty")
    if out is None:
        out = torch.empty((n, int(K)), dtype=torch.bfloat16, device=ids.device)
    else:
        _out_vec(out, n * int(K))
    if status is not None and (not status.is_cuda or status.dtype is not torch.int32):
        _fail("status must be CUDA int32")
    if (position is None) != (valid_len is None):
        _fail("position and valid_len go together")
    if position is not None:
        position = _position(position)
        if not valid_len.is_cuda or valid_len.dtype is not torch.int32 or valid_len.numel() != 1:
            _fail("valid_len must be a CUDA int32 scalar")
    rc = _lib.load().chr_nf4_embed_rows(
        ctypes.byref(dev), _ptr(ids), n, _ptr(out), _ptr(status), _ptr(position), _ptr(valid_len),
        _stream(),
    )
    _lib.check(rc, "chr_nf4_embed_rows")
    del keep
    return out


def nf4_pick_commit(
    logits: torch.Tensor,
    next_token: torch.Tensor,
    scratch: torch.Tensor,
    token: torch.Tensor | None = None,
    position: torch.Tensor | None = None,
    finished: torch.Tensor | None = None,
    eos: int = -1,
) -> None:
    """``next_token = argmax(logits)`` and, when given, the greedy commit
    (``token = next``, ``position += 1``, ``finished |= next == eos``) in one launch.
    ``scratch`` is 16 zeroed device bytes (uint8) that stay zero after the call."""
    if not logits.is_cuda or logits.dtype is not torch.bfloat16 or not logits.is_contiguous():
        _fail("logits must be contiguous CUDA bf16")
    if not next_token.is_cuda or next_token.dtype is not torch.int64 or next_token.numel() != 1:
        _fail("next_token must be a CUDA int64 scalar")
    if not scratch.is_cuda or scratch.numel() * scratch.element_size() < 16:
        _fail("scratch must hold 16 device bytes")
    for t, dt, what in ((token, torch.int64, "token"), (position, torch.int64, "position"),
                        (finished, torch.uint8, "finished")):
        if t is not None and (not t.is_cuda or t.dtype is not dt or t.numel() != 1):
            _fail(f"{what} must be a CUDA {dt} scalar")
    rc = _lib.load().chr_nf4_pick_commit(
        _ptr(logits), int(logits.numel()), _ptr(next_token), _ptr(token), _ptr(position),
        _ptr(finished), int(eos), _ptr(scratch), _stream(),
    )
    _lib.check(rc, "chr_nf4_pick_commit")


# --------------------------------------------------------------------------- #
# row-wise helpers of the chunked prefill
# --------------------------------------------------------------------------- #
def _rows_view(t: torch.Tensor, what: str) -> tuple[int, int]:
    """(rows, row stride in elements) of a CUDA bf16 2-D view whose rows are contiguous."""
    if not t.is_cuda or t.dtype is not torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
        _fail(f"{what} must be a CUDA bfloat16 [N, F] view with contiguous rows")
    return int(t.size(0)), int(t.stride(0))


def nf4_pick_commit_batch(logits: torch.Tensor, next_token: torch.Tensor, scratch: torch.Tensor,
                          token: torch.Tensor | None = None, position: torch.Tensor | None = None,
                          finished: torch.Tensor | None = None, eos: int = -1) -> None:
    """Greedy pick + commit for every row of ``logits`` ``[B, n]`` in one launch; per-sequence
    ``next_token`` / ``token`` / ``position`` (int64 ``[B]``), ``finished`` (uint8 ``[B]``),
    ``scratch`` uint8 ``[B, 16]`` zeroed once. See ``chr_nf4_pick_commit_batch``."""
    if not logits.is_cuda or logits.dtype is not torch.bfloat16 or logits.dim() != 2 or logits.stride(1) != 1:
        _fail("logits must be a CUDA bfloat16 [B, n] view with contiguous rows")
    b, n = int(logits.size(0)), int(logits.size(1))
    for t, what, dt in ((next_token, "next_token", torch.int64), (token, "token", torch.int64),
                        (position, "position", torch.int64), (finished, "finished", torch.uint8)):
        if t is None:
            continue
        if not t.is_cuda or t.dtype is not dt or not t.is_contiguous() or t.numel() != b:
            _fail(f"{what} must be a contiguous CUDA {dt} tensor of {b} elements")
    if (not scratch.is_cuda or scratch.dtype is not torch.uint8 or not scratch.is_contiguous()
            or scratch.numel() < 16 * b):
        _fail("scratch must be contiguous CUDA uint8 with 16 bytes per sequence")
    rc = _lib.load().chr_nf4_pick_commit_batch(_ptr(logits), int(logits.stride(0)), n, b, _ptr(next_token),
                                               _ptr(token), _ptr(position), _ptr(finished), int(eos),
                                               _ptr(scratch), _stream())
    _lib.check(rc, "chr_nf4_pick_commit_batch")


def nf4_pick_commit_tp(
    logits_local: torch.Tensor,
    index_offset: int,
    peers,
    next_token: torch.Tensor,
    scratch: torch.Tensor,
    token: torch.Tensor | None = None,
    position: torch.Tensor | None = None,
    finished: torch.Tensor | None = None,
    eos: int = -1,
) -> None:
    """Greedy pick over a vocabulary split across ranks: local argmax, one (value, id) pair
    exchanged per rank over peer memory, the same commit on every rank."""
    if not logits_local.is_cuda or logits_local.dtype is not torch.bfloat16 or not logits_local.is_contiguous():
        _fail("logits_local must be contiguous CUDA bf16")
    rc = _lib.load().chr_nf4_pick_commit_tp(
        _ptr(logits_local), int(logits_local.numel()), int(index_offset), ctypes.byref(peers),
        _ptr(next_token), _ptr(token), _ptr(position), _ptr(finished), int(eos), _ptr(scratch),
        _stream())
    _lib.check(rc, "chr_nf4_pick_commit_tp")


def nf4_rms_rows(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm of every row of ``x`` ``[N, K]`` (rows may be strided) -> contiguous ``[N, K]``."""
    n, stride = _rows_view(x, "x")
    k = int(x.size(1))
    wv = _opt_bf16(w, k, "w", exact=True)
    y = torch.empty((n, k), dtype=torch.bfloat16, device=x.device)
    rc = _lib.load().chr_nf4_rms_rows(_ptr(x), stride, _ptr(wv), _ptr(y), n, k, float(eps), _stream())
    _lib.check(rc, "chr_nf4_rms_rows")
    return y


def nf4_rope_kv_rows(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor,
                     v_cache: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, start: int,
                     n_q: int, n_kv: int, hd: int) -> torch.Tensor:
    """RoPE for positions ``start..start+N-1``: rotated q ``[N, n_q, hd]`` (new tensor); k rotated
    and v copied into cache rows ``start..`` of ``k_cache`` / ``v_cache`` ``[max_seq, n_kv, hd]``."""
    n, qs = _rows_view(q, "q")
    nk, ks = _rows_view(k, "k")
    nv, vs = _rows_view(v, "v")
    if nk != n or nv != n or q.size(1) != n_q * hd or k.size(1) != n_kv * hd or v.size(1) != n_kv * hd:
        _fail("q / k / v rows do not match N, n_q, n_kv, hd")
    for t, what in ((k_cache, "k_cache"), (v_cache, "v_cache"), (cos, "cos"), (sin, "sin")):
        if not t.is_cuda or t.dtype is not torch.bfloat16 or not t.is_contiguous():
            _fail(f"{what} must be contiguous CUDA bfloat16")
    max_seq = int(k_cache.size(0))
    if tuple(k_cache.shape) != (max_seq, n_kv, hd) or tuple(v_cache.shape) != (max_seq, n_kv, hd):
        _fail("caches must be [max_seq, n_kv, hd]")
    if cos.size(0) < int(start) + n or cos.size(-1) != hd or sin.shape != cos.shape:
        _fail("cos / sin must cover the positions with hd columns")
    q_out = torch.empty((n, n_q, hd), dtype=torch.bfloat16, device=q.device)
    rc = _lib.load().chr_nf4_rope_kv_rows(
        _ptr(q), qs, _ptr(k), ks, _ptr(v), vs, _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _ptr(cos),
        _ptr(sin), int(start), n, int(n_q), int(n_kv), int(hd), max_seq, _stream())
    _lib.check(rc, "chr_nf4_rope_kv_rows")
    return q_out


def nf4_attn_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, start: int,
                     scale: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """Causal GQA attention of a prefill chunk: query row ``i`` (position ``start + i``) over cache
    rows ``t <= start + i``; ``q`` ``[n, n_q, hd]`` (or ``[n, n_q*hd]`` rows with a stride), caches
    ``[max_seq, n_kv, hd]`` -> ``[n, n_q*hd]``. See ``chr_nf4_attn_prefill``."""
    for t, what in ((k_cache, "k_cache"), (v_cache, "v_cache")):
        if not t.is_cuda or t.dtype is not torch.bfloat16 or not t.is_contiguous() or t.dim() != 3:
            _fail(f"{what} must be contiguous CUDA bfloat16 [max_seq, n_kv, hd]")
    max_seq, n_kv, hd = (int(v) for v in k_cache.shape)
    if tuple(v_cache.shape) != (max_seq, n_kv, hd):
        _fail("k_cache and v_cache differ in shape")
    if q.dim() == 3:
        if q.stride(2) != 1 or q.stride(1) != q.size(2) or q.size(2) != hd:
            _fail("q must be [n, n_q, hd] with contiguous heads")
        q2 = q.as_strided((q.size(0), q.size(1) * q.size(2)), (q.stride(0), 1))
    else:
        q2 = q
    n, qs = _rows_view(q2, "q")
    width = int(q2.size(1))
    if width % hd != 0 or (width // hd) % n_kv != 0:
        _fail("q width must be n_q * hd with n_q a multiple of n_kv")
    n_q = width // hd
    if out is None:
        out = torch.empty((n, width), dtype=torch.bfloat16, device=q.device)
    elif (not out.is_cuda or out.dtype is not torch.bfloat16 or not out.is_contiguous()
          or out.numel() != n * width):
        _fail("out must be contiguous CUDA bfloat16 [n, n_q*hd]")
    rc = _lib.load().chr_nf4_attn_prefill(_ptr(q2), qs, _ptr(k_cache), _ptr(v_cache), _ptr(out), n,
                                          int(start), n_q, n_kv, hd, max_seq, float(scale), _stream())
    _lib.check(rc, "chr_nf4_attn_prefill")
    return out


def nf4_silu_mul(gate_up: torch.Tensor, inter: int) -> torch.Tensor:
    """``silu(gate_up[:, :I]) * gate_up[:, I:]`` with bf16 rounding after each op -> ``[N, I]``."""
    if (not gate_up.is_cuda or gate_up.dtype is not torch.bfloat16 or gate_up.dim() != 2
            or not gate_up.is_contiguous() or gate_up.size(1) != 2 * int(inter)):
        _fail("gate_up must be contiguous CUDA bfloat16 [N, 2*I]")
    n = int(gate_up.size(0))
    out = torch.empty((n, int(inter)), dtype=torch.bfloat16, device=gate_up.device)
    rc = _lib.load().chr_nf4_silu_mul(_ptr(gate_up), _ptr(out), n, int(inter), _stream())
    _lib.check(rc, "chr_nf4_silu_mul")
    return out
