"""Chunked prompt prefill: tensor-core NF4 GEMM for the linears, eager (not captured).

Follows the reference (gpu/decodev2/prefill.py:26-141): chunks of positions, RMSNorm /
RoPE / causal GQA attention in the cache dtype, KV rows written per chunk, lm_head only
on the last chunk. The attention of a chunk over the cache prefix is this library's
``chr_nf4_attn_prefill`` kernel (the reference calls torch's
``scaled_dot_product_attention`` with a boolean mask there, prefill.py:50-92).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from gpu.nf4 import LIVE_MAX_N, nf4_attn_prefill, nf4_rms_rows, nf4_rope_kv_rows, nf4_silu_mul

from .arch import ArchSpec
from .embed import gather_embed
from .linear import DeviceLayer, DeviceWeights, nf4_linear
from .rope import apply_rope_torch
from .state import DecodeState

__all__ = ["forward_prefill", "prefill_chunk_width", "set_fused_rows", "fused_rows"]

_FUSED_ROWS = True


def fused_rows() -> bool:
    return _FUSED_ROWS


def set_fused_rows(on: bool) -> None:
    """``True`` (default): RMSNorm, RoPE + cache write and SiLU*up of a chunk run as one
    launch each; ``False``: as the reference's torch ops (same bits for RoPE and SiLU*up)."""
    global _FUSED_ROWS
    _FUSED_ROWS = bool(on)


#: positions per prefill chunk when the caller does not say; the wide GEMM has no
#: 32-column ceiling, so a chunk is bounded by attention-mask memory, not by the kernel.
PREFILL_CHUNK = 512


def prefill_chunk_width(state: DecodeState, chunk: int | None = None) -> int:
    """Positions per chunk. ``chunk=LIVE_MAX_N`` (32) reproduces the reference's chunking."""
    cap = min(int(PREFILL_CHUNK), int(state.spec.max_seq))
    return cap if chunk is None else max(1, min(int(chunk), cap))


def _split_qkv(layer: DeviceLayer, h: torch.Tensor, spec: ArchSpec):
    n = int(h.shape[0])
    if spec.family == "internlm_gqa":
        y = nf4_linear(layer.wqkv, h).view(n, spec.n_kv, spec.n_rep + 2, spec.head_dim)
        q = y[:, :, : spec.n_rep].reshape(n, spec.n_q, spec.head_dim)
        return q, y[:, :, -2], y[:, :, -1]
    if layer.qkv_rows is not None:  # q, k, v stacked in memory: one pass over the activations
        y = nf4_linear(layer.qkv_rows, h)
        mq, mk = layer.q.M, layer.k.M
        return (y[:, :mq].reshape(n, spec.n_q, spec.head_dim),
                y[:, mq:mq + mk].reshape(n, -1, spec.head_dim),
                y[:, mq + mk:].reshape(n, -1, spec.head_dim))
    return (
        nf4_linear(layer.q, h).view(n, spec.n_q, spec.head_dim),
        nf4_linear(layer.k, h).view(n, spec.n_kv, spec.head_dim),
        nf4_linear(layer.v, h).view(n, spec.n_kv, spec.head_dim),
    )


ATTN_HEAD_DIMS = (16, 32, 64, 128)


def _attend(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, spec: ArchSpec,
            start: int) -> torch.Tensor:
    """``q`` [n, n_q, hd] (rotated) against cache rows ``0 .. start+n-1`` of one layer
    (``[max_seq, n_kv, hd]``, the chunk's rows already written) -> ``[n, q_dim]``."""
    if q.dtype is not torch.bfloat16 or spec.head_dim not in ATTN_HEAD_DIMS:
        raise RuntimeError(f"prefill attention covers bfloat16 caches with head_dim in {ATTN_HEAD_DIMS}; "
                           f"got {q.dtype}, head_dim={spec.head_dim}")
    return nf4_attn_prefill(q, k_cache, v_cache, start, spec.attn_scale)


def _reduced(state: DecodeState, partial: torch.Tensor) -> torch.Tensor:
    """Sum a row-split linear's output over the tensor-parallel ranks (FP32 on the wire)."""
    if state.spec.tp == 1:
        return partial
    acc = partial.float()
    state.comm.all_reduce_sum(acc)
    return acc.to(partial.dtype)


def forward_prefill(state: DecodeState, weights: DeviceWeights, token_ids: torch.Tensor,
                    start: int, *, logits: bool = True) -> None:
    """Teacher-force ``token_ids`` into KV slots ``start..start+n-1``."""
    spec = state.spec
    ids = token_ids.reshape(-1).to(device=state.device, dtype=torch.long)
    n = int(ids.numel())
    if n < 1:
        raise ValueError("prefill chunk must be non-empty")
    start = int(start)
    seq = start + n
    if seq > spec.max_seq:
        raise ValueError(f"prefill {start}..{seq} exceeds max_seq={spec.max_seq}")
    dtype = state.arena.x.dtype
    x = gather_embed(weights.embed, ids, dtype=dtype)
    cos, sin = state.cos[start:seq], state.sin[start:seq]
    fused = _FUSED_ROWS and x.dtype is torch.bfloat16 and spec.hidden % 8 == 0
    for li, layer in enumerate(weights.layers):
        if fused:
            h = nf4_rms_rows(x, layer.norm1, spec.rms_eps)
        else:
            h = F.rms_norm(x, layer.norm1.shape, layer.norm1, spec.rms_eps)
        q, k, v = _split_qkv(layer, h, spec)
        if fused and layer.wqkv is None:
            q = nf4_rope_kv_rows(q.flatten(1), k.flatten(1), v.flatten(1), state.kv.k[li],
                                 state.kv.v[li], state.cos, state.sin, start, q.shape[1],
                                 k.shape[1], spec.head_dim)
        else:
            q = apply_rope_torch(q, cos, sin)
            k = apply_rope_torch(k, cos, sin)
            state.kv.write_range(li, start, k, v)
        attn = _attend(q.contiguous(), state.kv.k[li], state.kv.v[li], spec, start)
        if spec.tp == 1:
            x = nf4_linear(layer.o, attn, add=x)      # residual folded into the GEMM epilogue
        else:
            x = x + _reduced(state, nf4_linear(layer.o, attn))
        if fused:
            h = nf4_rms_rows(x, layer.norm2, spec.rms_eps)
        else:
            h = F.rms_norm(x, layer.norm2.shape, layer.norm2, spec.rms_eps)
        if layer.gate_up is not None:
            gu = nf4_linear(layer.gate_up, h)
            act = (nf4_silu_mul(gu, layer.gate.M) if fused
                   else F.silu(gu[:, : layer.gate.M]) * gu[:, layer.gate.M:])
        else:
            act = F.silu(nf4_linear(layer.gate, h)) * nf4_linear(layer.up, h)
        if spec.tp == 1:
            x = nf4_linear(layer.down, act, add=x)
        else:
            x = x + _reduced(state, nf4_linear(layer.down, act))
    state.position.fill_(seq)
    state.valid_len.fill_(seq)
    if not logits:
        return
    hidden = F.rms_norm(x[-1:], weights.final_norm.shape, weights.final_norm, spec.rms_eps)
    out = nf4_linear(weights.lm_head, hidden)
    if spec.tp > 1:
        state.comm.all_gather_into(state.arena.logits.view(-1), out.reshape(-1).contiguous())
        out = state.arena.logits
    else:
        state.arena.logits[0].copy_(out.reshape(-1))
    state.next_token.copy_(out.reshape(-1).argmax(dim=-1).reshape(()).to(dtype=torch.int64))
