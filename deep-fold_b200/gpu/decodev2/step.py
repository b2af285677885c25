"""One resident greedy decode step: no Python sequence length, no host sync.

Same operation sequence as the reference's CUDA GEMV path
(gpu/decodev2/step.py:162-187): embed row -> per layer [RMSNorm, fused q/k/v
GEMV (+bias), attention with fused RoPE and KV write over the valid prefix,
o-proj GEMV with fused residual, RMSNorm, fused SwiGLU GEMV, down-proj GEMV with
fused residual] -> final RMSNorm -> lm_head GEMV -> greedy pick -> commit.
Differences are launch-count only: RMSNorm rides inside the following GEMV
(``rms_w``), the packed embedding row and ``valid_len = position + 1`` are one
kernel, argmax + commit are one kernel.
"""

from __future__ import annotations

import torch

from gpu.nf4 import (ATTN_SPLIT, nf4_attn, nf4_gemv, nf4_gemv_allreduce, nf4_gemv_f32,
                     nf4_pick_commit, nf4_pick_commit_tp, nf4_qkv, nf4_rms, nf4_swiglu)

from .embed import PackedEmbed
from .linear import DeviceLayer, DeviceLinear, DeviceWeights
from .state import DecodeState

__all__ = ["forward_decode", "greedy_decode", "teacher_force_token", "set_fuse_rms", "fuse_rms"]

_FUSE_RMS = True


def fuse_rms() -> bool:
    return _FUSE_RMS


def set_fuse_rms(on: bool) -> None:
    """``True`` (default): RMSNorm runs inside the GEMV that consumes it."""
    global _FUSE_RMS
    _FUSE_RMS = bool(on)


def _embed_into(state: DecodeState, weights: DeviceWeights) -> None:
    ar = state.arena
    if isinstance(weights.embed, PackedEmbed):
        weights.embed.gather(state.token.reshape(1), out=ar.x, status=ar.status,
                             position=state.position, valid_len=state.valid_len)
    else:
        torch.index_select(weights.embed, 0, state.token.reshape(1), out=ar.x)
        state.kv.mark_written(state.position)


def _normed(state: DecodeState, w: torch.Tensor):
    """(x to feed the next GEMV, rms_w to hand it)."""
    ar = state.arena
    if _FUSE_RMS:
        return ar.x, w
    nf4_rms(ar.x.view(-1), w.view(-1), ar.h.view(-1), state.spec.rms_eps)
    return ar.h, None


def _qkv(state: DecodeState, layer: DeviceLayer) -> None:
    spec, ar = state.spec, state.arena
    x, rms_w = _normed(state, layer.norm1)
    if layer.wqkv is None:
        q, k, v = layer.q, layer.k, layer.v
        nf4_qkv(q.packed, q.scale, k.packed, k.scale, v.packed, v.scale, x, q.M, k.M, v.M,
                q.K, q.K_pad, ar.q.view(-1), ar.k.view(-1), ar.v.view(-1), q.bias, k.bias, v.bias,
                rms_w, spec.rms_eps)
        return
    m = layer.wqkv
    nf4_gemv(m.packed, m.scale, x, m.M, m.K, m.K_pad, ar.qkv.view(-1), m.bias, rms_w, spec.rms_eps)
    grouped = ar.qkv.view(spec.n_kv, spec.n_rep + 2, spec.head_dim)
    ar.q.view(spec.n_kv, spec.n_rep, spec.head_dim).copy_(grouped[:, : spec.n_rep])
    ar.k.view(spec.n_kv, spec.head_dim).copy_(grouped[:, -2])
    ar.v.view(spec.n_kv, spec.head_dim).copy_(grouped[:, -1])


def _accumulate(state: DecodeState, mat: DeviceLinear, src: torch.Tensor, dest: torch.Tensor) -> None:
    """``dest += W @ src``. Single GPU: one launch, residual fused into the GEMV
    epilogue. Row-split shard: FP32 partial -> sum over ranks -> one rounded add, either as
    one launch that exchanges the partials over peer memory (``state.peers``) or as GEMV +
    NCCL all-reduce + add."""
    if state.spec.tp == 1:
        nf4_gemv(mat.packed, mat.scale, src.reshape(mat.K), mat.M, mat.K, mat.K_pad,
                 dest.view(-1), dest.view(-1))
        if mat.bias is not None:
            dest.view(-1).add_(mat.bias.to(dtype=dest.dtype))
        return
    if state.peers is not None:  # partial, exchange over peer memory and sum in one launch
        nf4_gemv_allreduce(mat.packed, mat.scale, src.reshape(mat.K), mat.M, mat.K, mat.K_pad,
                           dest.view(-1), state.peers.for_matrix(mat), mat.bias)
        return
    part = state.arena.partial
    nf4_gemv_f32(mat.packed, mat.scale, src.reshape(mat.K), mat.M, mat.K, mat.K_pad, part, mat.bias)
    state.comm.all_reduce_sum(part)
    dest.view(-1).add_(part)


def forward_decode(state: DecodeState, weights: DeviceWeights, *, gather_logits: bool = True) -> None:
    """``gather_logits=False`` (tensor parallel only) leaves each rank with its slice in
    ``arena.logits_local``: the greedy pick then exchanges one pair per rank instead."""
    spec, ar = state.spec, state.arena
    _embed_into(state, weights)
    for li, layer in enumerate(weights.layers):
        _qkv(state, layer)
        nf4_attn(ar.q, state.kv.k[li], state.kv.v[li], ar.attn, state.valid_len, spec.attn_scale,
                 ar.attn_ws, ATTN_SPLIT, ar.k, ar.v, state.cos, state.sin, state.position)
        _accumulate(state, layer.o, ar.attn, ar.x)
        x, rms_w = _normed(state, layer.norm2)
        g, u = layer.gate, layer.up
        nf4_swiglu(g.packed, g.scale, u.packed, u.scale, x, g.M, g.K, g.K_pad,
                   ar.down_in.view(-1), rms_w, spec.rms_eps)
        _accumulate(state, layer.down, ar.down_in, ar.x)
    x, rms_w = _normed(state, weights.final_norm)
    head = weights.lm_head
    if spec.tp == 1:
        nf4_gemv(head.packed, head.scale, x, head.M, head.K, head.K_pad, ar.logits.view(-1),
                 head.bias, rms_w, spec.rms_eps)
    else:  # vocabulary slice per rank, gathered in rank order into the full logits
        nf4_gemv(head.packed, head.scale, x, head.M, head.K, head.K_pad,
                 ar.logits_local.view(-1), head.bias, rms_w, spec.rms_eps)
        if gather_logits:
            state.comm.all_gather_into(ar.logits.view(-1), ar.logits_local.view(-1))


def greedy_decode(state: DecodeState, weights: DeviceWeights) -> None:
    """Forward + pick + commit: ``token``/``position``/``finished`` advance on the device."""
    if state.spec.tp > 1 and state.pick_peers is not None:
        forward_decode(state, weights, gather_logits=False)
        local = state.arena.logits_local.view(-1)
        nf4_pick_commit_tp(local, state.comm.rank * local.numel(), state.pick_peers.peers,
                           state.next_token, state.arena.pick_scratch, state.token, state.position,
                           state.finished, int(state.spec.eos_id))
        return
    forward_decode(state, weights)
    nf4_pick_commit(state.arena.logits.view(-1), state.next_token, state.arena.pick_scratch,
                    state.token, state.position, state.finished, int(state.spec.eos_id))


def teacher_force_token(state: DecodeState, weights: DeviceWeights, token_id: int) -> None:
    """Feed a given token: logits + ``next_token`` are produced, nothing is committed
    except the position."""
    state.load_token(token_id)
    forward_decode(state, weights)
    nf4_pick_commit(state.arena.logits.view(-1), state.next_token, state.arena.pick_scratch)
    state.position.add_(1)
