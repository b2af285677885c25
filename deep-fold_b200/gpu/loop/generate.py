"""``TokenLoop``: greedy generation where every N=1 linear runs the tensor-core GEMM.

The reference keeps two executors (gpu/loop/generate.py:559-758 and
gpu/decodev2): TokenLoop drives the MMA kernel at N=1 with the weight operand
rounded to bf16 and captures its GEMM groups in CUDA graphs; Decode V2 drives the
CUDA-core GEMV and captures the whole step. Here TokenLoop keeps the first
numerics (``nf4_gemm`` at N=1, separate RMSNorm launches, residual adds in bf16)
and the same request API (``generate``, ``prefill_from``, ``decode_from_logits``,
``step``, ``warmup``, ``capture_graphs``, ``Generation``), on the resident state
and KV cache of Decode V2; its graph mode captures the whole step at once, which
subsumes the reference's per-group graphs without their static-input copies.
"""

from __future__ import annotations

import torch

from gpu.decodev2.embed import PackedEmbed
from gpu.decodev2.linear import DeviceLinear, DeviceWeights
from gpu.decodev2.session import DecodeV2Loop, Generation
from gpu.decodev2.state import DecodeState
from gpu.decodev2.graph import capture_greedy
from gpu.nf4 import ATTN_SPLIT, nf4_attn, nf4_gemm, nf4_pick_commit, nf4_rms

__all__ = ["Generation", "TokenLoop", "mma_decode"]


def _mma(mat: DeviceLinear, vec: torch.Tensor) -> torch.Tensor:
    """``W @ vec`` through the tensor-core kernel at N=1 (+ bias); returns bf16 ``[M]``."""
    y = nf4_gemm(mat.packed, mat.scale, vec.reshape(mat.K), mat.M, mat.K, mat.K_pad).view(mat.M)
    return y if mat.bias is None else y + mat.bias


def mma_decode(state: DecodeState, weights: DeviceWeights) -> None:
    """One greedy token on the MMA path; commits token / position / finished on the device."""
    spec, ar = state.spec, state.arena
    if spec.tp != 1:
        raise RuntimeError("TokenLoop is single-GPU; tensor parallelism runs through Decode V2")
    if isinstance(weights.embed, PackedEmbed):
        weights.embed.gather(state.token.reshape(1), out=ar.x, status=ar.status,
                             position=state.position, valid_len=state.valid_len)
    else:
        torch.index_select(weights.embed, 0, state.token.reshape(1), out=ar.x)
        state.kv.mark_written(state.position)
    x = ar.x.view(-1)
    for li, layer in enumerate(weights.layers):
        nf4_rms(x, layer.norm1.view(-1), ar.h.view(-1), spec.rms_eps)
        if layer.wqkv is not None:
            grouped = _mma(layer.wqkv, ar.h).view(spec.n_kv, spec.n_rep + 2, spec.head_dim)
            ar.q.view(spec.n_kv, spec.n_rep, spec.head_dim).copy_(grouped[:, : spec.n_rep])
            ar.k.view(spec.n_kv, spec.head_dim).copy_(grouped[:, -2])
            ar.v.view(spec.n_kv, spec.head_dim).copy_(grouped[:, -1])
        else:
            ar.q.view(-1).copy_(_mma(layer.q, ar.h))
            ar.k.view(-1).copy_(_mma(layer.k, ar.h))
            ar.v.view(-1).copy_(_mma(layer.v, ar.h))
        nf4_attn(ar.q, state.kv.k[li], state.kv.v[li], ar.attn, state.valid_len, spec.attn_scale,
                 ar.attn_ws, ATTN_SPLIT, ar.k, ar.v, state.cos, state.sin, state.position)
        x.add_(_mma(layer.o, ar.attn))
        nf4_rms(x, layer.norm2.view(-1), ar.h.view(-1), spec.rms_eps)
        gate, up = _mma(layer.gate, ar.h), _mma(layer.up, ar.h)
        ar.down_in.view(-1).copy_(torch.nn.functional.silu(gate) * up)
        x.add_(_mma(layer.down, ar.down_in))
    nf4_rms(x, weights.final_norm.view(-1), ar.h.view(-1), spec.rms_eps)
    ar.logits.view(-1).copy_(_mma(weights.lm_head, ar.h))
    nf4_pick_commit(ar.logits.view(-1), state.next_token, ar.pick_scratch, state.token,
                    state.position, state.finished, int(spec.eos_id))


class TokenLoop(DecodeV2Loop):
    """Request API of :class:`DecodeV2Loop`, decode steps on the MMA path."""

    def _step(self):
        return self._graph if self._graph is not None else mma_decode

    def step(self) -> int:
        """One decode step; returns the committed token id (host read)."""
        self._step()(self.state, self.weights)
        return int(self.state.token.item())

    def capture_graphs(self) -> str:
        try:
            self.reset()
            self._graph = capture_greedy(self.state, self.weights, warmup=2, step=mma_decode)
            self.graph_mode = "tokenloop"
            self.graph_error = None
        except Exception as exc:  # noqa: BLE001 - reported, not swallowed
            self._graph = None
            self.graph_mode = "off"
            self.graph_error = f"{type(exc).__name__}: {exc}"
        self.reset()
        return self.graph_mode
