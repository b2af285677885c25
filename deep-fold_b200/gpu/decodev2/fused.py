"""The greedy step as ONE persistent launch (``chr_nf4_decode_step``).

Same operations and the same bits as :func:`step.greedy_decode`, which issues one
launch per operation (reference sequence: gpu/decodev2/step.py:162-187); here the
whole step is a cooperative kernel with grid-wide barriers between operations.
``FusedStep`` binds a ``DecodeState`` and its ``DeviceWeights`` once: it lays the
per-layer descriptors out once and keeps the call structure, so a step
is one C call with no Python work per layer.
"""

from __future__ import annotations

import ctypes

import torch

from gpu.nf4 import _lib
from gpu.nf4._lib import STEP_SYNC_BYTES, ChrNf4Dev, ChrNf4Step, ChrNf4StepLayer
from gpu.nf4.plan import k_pad

from .embed import PackedEmbed
from .linear import DeviceLinear, DeviceWeights
from .state import ATTN_SPLIT, DecodeState

__all__ = ["FusedStep", "fused_step_supported"]


def _dev(mat: DeviceLinear | None) -> ChrNf4Dev:
    if mat is None:
        return ChrNf4Dev(0, 0, 0, None, None)
    return ChrNf4Dev(int(mat.M), int(mat.K), int(mat.K_pad), mat.packed.data_ptr(), mat.scale.data_ptr())


def _p(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def fused_step_supported(state: DecodeState, weights: DeviceWeights) -> str | None:
    """``None`` when the persistent step covers this model, else the reason it does not."""
    spec = state.spec
    if spec.tp != 1:
        return "tensor-parallel shards exchange partial sums between operations"
    if spec.hidden % 8:
        return "hidden is not a multiple of 8"
    for ly in weights.layers:
        if ly.o.bias is not None or ly.down.bias is not None:
            return "bias on a row-split projection"
        if ly.gate.bias is not None or ly.up.bias is not None:
            return "bias on gate / up"
    if weights.lm_head.bias is not None:
        return "bias on lm_head"
    return None


class FusedStep:
    """Callable ``(state, weights) -> None`` with the signature of ``greedy_decode``."""

    def __init__(self, state: DecodeState, weights: DeviceWeights, *, commit: bool = True) -> None:
        why = fused_step_supported(state, weights)
        if why is not None:
            raise RuntimeError(f"persistent step not available: {why}")
        self.state, self.weights = state, weights
        spec, ar = state.spec, state.arena
        dev = state.device
        fused_qkv = weights.layers[0].wqkv is not None
        rows = (ChrNf4StepLayer * len(weights.layers))()
        for li, ly in enumerate(weights.layers):
            r = rows[li]
            if fused_qkv:
                r.q, r.k, r.v = _dev(ly.wqkv), _dev(None), _dev(None)
                r.bq, r.bk, r.bv = _p(ly.wqkv.bias), None, None
            else:
                r.q, r.k, r.v = _dev(ly.q), _dev(ly.k), _dev(ly.v)
                r.bq, r.bk, r.bv = _p(ly.q.bias), _p(ly.k.bias), _p(ly.v.bias)
            r.o, r.gate, r.up, r.down = _dev(ly.o), _dev(ly.gate), _dev(ly.up), _dev(ly.down)
            r.norm1, r.norm2 = _p(ly.norm1), _p(ly.norm2)
            r.k_cache, r.v_cache = state.kv.k[li].data_ptr(), state.kv.v[li].data_ptr()
        self._layers = rows  # host array, read by the library at every call
        self._sync = torch.zeros(STEP_SYNC_BYTES, dtype=torch.uint8, device=dev)
        s = ChrNf4Step()
        s.n_layers, s.hidden, s.intermediate = spec.n_layers, spec.hidden, spec.intermediate
        s.n_q, s.n_kv, s.head_dim = spec.n_q, spec.n_kv, spec.head_dim
        s.max_seq, s.vocab, s.n_split = spec.max_seq, spec.vocab, ATTN_SPLIT
        s.fused_qkv, s.commit = int(fused_qkv), int(bool(commit))
        s.rms_eps, s.attn_scale, s.eos = float(spec.rms_eps), float(spec.attn_scale), int(spec.eos_id)
        if isinstance(weights.embed, PackedEmbed):
            e = weights.embed
            s.embed = ChrNf4Dev(int(e.vocab), int(e.hidden), int(k_pad(e.hidden)),
                                e.packed.data_ptr(), e.scale.data_ptr())
            s.embed_dense = None
        else:
            s.embed = ChrNf4Dev(0, 0, 0, None, None)
            s.embed_dense = weights.embed.data_ptr()
        s.lm_head = _dev(weights.lm_head)
        s.final_norm, s.cos, s.sin = _p(weights.final_norm), _p(state.cos), _p(state.sin)
        s.token, s.position, s.next_token = _p(state.token), _p(state.position), _p(state.next_token)
        s.valid_len, s.finished = _p(state.valid_len), _p(state.finished)
        s.x, s.q, s.k, s.v, s.qkv = _p(ar.x), _p(ar.q), _p(ar.k), _p(ar.v), _p(ar.qkv)
        s.attn, s.down_in, s.logits = _p(ar.attn), _p(ar.down_in), _p(ar.logits)
        s.attn_ws, s.layers, s.sync = _p(ar.attn_ws), ctypes.addressof(self._layers), self._sync.data_ptr()
        self._step = s
        self._call = _lib.load().chr_nf4_decode_step

    def __call__(self, state: DecodeState, weights: DeviceWeights) -> None:
        if state is not self.state or weights is not self.weights:
            raise RuntimeError("FusedStep is bound to the state and weights it was built from")
        rc = self._call(ctypes.byref(self._step),
                        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        _lib.check(rc, "chr_nf4_decode_step")

    def timeline_us(self) -> list[float]:
        """Per-operation durations (microseconds) of the last step as seen by CTA 0:
        entry n-1 is the time between the barriers before operations n and n+1
        (operation 1 is layer 0's q/k/v; then attention, o, gate/up, down per layer;
        then lm_head and the pick). Synchronises the device."""
        torch.cuda.synchronize()
        n_ops = 5 * self.state.spec.n_layers + 2
        stamps = self._sync[4160:4160 + 8 * (n_ops + 1)].view(torch.int64).tolist()
        return [(b - a) / 1e3 for a, b in zip(stamps[1:], stamps[2:])]

    def status(self) -> int:
        """0, the index of the operation whose barrier wait gave up, 1000 for a token id
        outside the embedding table, or 2000 when a replayed launch found another model's
        operation table on the device; synchronises the device and clears the word."""
        return int(_lib.load().chr_nf4_decode_step_status(ctypes.c_void_p(self._sync.data_ptr())))
