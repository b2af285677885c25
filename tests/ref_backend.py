"""The reference's own CUDA kernels as a GPU-side checker (tests only).

``oracle/_ref/libchr_nf4_ref.so`` is built by ``oracle/build.py`` from the
reference checkout's ``gpu/nf4/nf4_gemv.cu`` and ``gpu/nf4/nf4_gemm.cu``. This
module binds its C ABI (the same ``chr_gpu.h`` entry points the product library
exports) with ctypes and offers op functions with the product's Python
signatures, so a test can run the same inputs, or the same executor, through
either library. It is never imported by the package.
"""

from __future__ import annotations

import contextlib
import ctypes
from pathlib import Path

import torch

from gpu.nf4 import _lib as product_lib
from gpu.nf4._lib import ChrNf4Dev, ChrNf4Plan

REF_LIB = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "libchr_nf4_ref.so"
KEPT = ("chr_nf4_gemm", "chr_nf4_gemm_plan", "chr_nf4_gemm_ws", "chr_nf4_gemm_ws_max",
        "chr_nf4_set_tuning", "chr_nf4_gemv", "chr_nf4_gemv_qkv", "chr_nf4_gemv_swiglu",
        "chr_nf4_rope_kv", "chr_nf4_attn", "chr_nf4_rms")

_ref = None


def available() -> bool:
    return REF_LIB.is_file()


def load() -> ctypes.CDLL:
    global _ref
    if _ref is None:
        lib = ctypes.CDLL(str(REF_LIB))
        for name in KEPT:
            restype, argtypes = product_lib.SIGNATURES[name]
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = restype, argtypes
        _ref = lib
    return _ref


def _s():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _dev(packed, scale, m, k, kp):
    return ChrNf4Dev(int(m), int(k), int(kp), packed.data_ptr(), scale.data_ptr())


def _ok(rc, what):
    if rc != 0:
        raise RuntimeError(f"reference {what} failed ({rc})")


def nf4_gemv(packed, scale, x, M, K, K_pad, out=None, add=None, rms_w=None, rms_eps=1e-6):
    y = out if out is not None else torch.empty((M, 1), dtype=torch.bfloat16, device=x.device)
    d = _dev(packed, scale, M, K, K_pad)
    _ok(load().chr_nf4_gemv(ctypes.byref(d), _p(x.contiguous()), _p(y), _s(), _p(add), _p(rms_w),
                            float(rms_eps)), "gemv")
    return y


def nf4_qkv(qp, qs, kp_, ks, vp, vs, x, Mq, Mk, Mv, K, K_pad, oq, ok, ov, bq=None, bk=None, bv=None,
            rms_w=None, rms_eps=1e-6):
    dq, dk, dv = _dev(qp, qs, Mq, K, K_pad), _dev(kp_, ks, Mk, K, K_pad), _dev(vp, vs, Mv, K, K_pad)
    _ok(load().chr_nf4_gemv_qkv(ctypes.byref(dq), ctypes.byref(dk), ctypes.byref(dv),
                                _p(x.contiguous()), _p(oq), _p(ok), _p(ov), _p(bq), _p(bk), _p(bv),
                                _s(), _p(rms_w), float(rms_eps)), "qkv")
    return oq, ok, ov


def nf4_swiglu(gp, gs, up, us, x, M, K, K_pad, out, rms_w=None, rms_eps=1e-6):
    dg, du = _dev(gp, gs, M, K, K_pad), _dev(up, us, M, K, K_pad)
    _ok(load().chr_nf4_gemv_swiglu(ctypes.byref(dg), ctypes.byref(du), _p(x.contiguous()), _p(out),
                                   _s(), _p(rms_w), float(rms_eps)), "swiglu")
    return out


def nf4_rms(x, w, y, eps):
    _ok(load().chr_nf4_rms(_p(x), _p(w), _p(y), int(x.numel()), float(eps), _s()), "rms")


def nf4_attn(q, k, v, out, valid_len, scale, ws=None, n_split=32, k_act=None, v_act=None, cos=None,
             sin=None, position=None):
    max_seq, n_kv, hd = k.shape
    n_q = q.numel() // hd
    if ws is None:
        ws = torch.empty(n_q * n_split * (hd + 2), dtype=torch.float32, device=q.device)
    _ok(load().chr_nf4_attn(_p(q), _p(k), _p(v), _p(out), _p(valid_len), _p(ws), n_q, n_kv, hd,
                            int(n_split), float(scale), _s(), _p(k_act), _p(v_act), _p(cos), _p(sin),
                            _p(position), max_seq), "attn")


def nf4_gemm(packed, scale, x, M, K, K_pad, max_n=32):
    x = x.contiguous()
    if x.dim() == 1:
        x = x.unsqueeze(1)
    n = int(x.size(1))
    y = torch.empty((M, n), dtype=torch.bfloat16, device=x.device)
    d = _dev(packed, scale, M, K, K_pad)
    pl = ChrNf4Plan()
    _ok(load().chr_nf4_gemm_plan(ctypes.byref(d), n, 1, ctypes.byref(pl)), "plan")
    ws = torch.empty(max(1, int(pl.ws_floats)), dtype=torch.float32, device=x.device)
    _ok(load().chr_nf4_gemm_ws_max(ctypes.byref(d), _p(x), _p(y), n, _p(ws), int(pl.ws_floats), _s(),
                                   int(max_n)), "gemm")
    return y


def nf4_pick_commit(logits, next_token, scratch, token=None, position=None, finished=None, eos=-1):
    """The reference's torch-op form of argmax + commit (gpu/decodev2/step.py:182, state.py:98-103)."""
    next_token.copy_(logits.view(-1).argmax(dim=-1).reshape(()).to(torch.int64))
    if token is not None:
        token.copy_(next_token)
    if position is not None:
        position.add_(1)
    if finished is not None:
        finished.bitwise_or_((next_token == eos).to(torch.uint8))


@contextlib.contextmanager
def reference_kernels():
    """Run this repository's executor on the reference's kernels: the step and
    prefill modules' op bindings are swapped for the duration of the block, and
    RMSNorm runs as its own launch as in the reference's decode path."""
    import gpu.decodev2.linear as lin
    import gpu.decodev2.step as step

    here = globals()
    saved_step = {n: getattr(step, n) for n in ("nf4_attn", "nf4_gemv", "nf4_qkv", "nf4_rms",
                                                "nf4_swiglu", "nf4_pick_commit")}
    saved_lin = {n: getattr(lin, n) for n in ("nf4_gemm", "nf4_gemv")}
    fused = step.fuse_rms()
    try:
        for n in saved_step:
            setattr(step, n, here[n])
        for n in saved_lin:
            setattr(lin, n, here[n])
        step.set_fuse_rms(False)
        yield
    finally:
        for n, f in saved_step.items():
            setattr(step, n, f)
        for n, f in saved_lin.items():
            setattr(lin, n, f)
        step.set_fuse_rms(fused)
