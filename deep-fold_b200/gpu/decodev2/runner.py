"""Greedy runner: chunked GEMM prefill, then decode steps that stay on the GPU
(reference: gpu/decodev2/runner.py:17-81)."""

from __future__ import annotations

from collections.abc import Sequence

import torch

from .linear import DeviceWeights
from .prefill import forward_prefill, prefill_chunk_width
from .state import DecodeState
from .step import greedy_decode

__all__ = ["consume_prompt", "generate"]


def consume_prompt(state: DecodeState, weights: DeviceWeights, token_ids: Sequence[int], *,
                   chunk: int | None = None, start: int = 0) -> None:
    """Fill KV for ``token_ids`` starting at slot ``start`` (0 = cold prompt after ``reset``)."""
    if not len(token_ids):
        raise ValueError("prompt must be non-empty")
    ids = [int(t) for t in token_ids]
    pos = int(start)
    if pos < 0:
        raise ValueError(f"start {pos} is negative")
    if pos + len(ids) > state.spec.max_seq:
        raise ValueError(f"prompt {pos}+{len(ids)} exceeds max_seq={state.spec.max_seq}")
    width = prefill_chunk_width(state, chunk)
    buf = torch.tensor(ids, dtype=torch.long, device=state.device)
    for lo in range(0, len(ids), width):
        hi = min(lo + width, len(ids))
        forward_prefill(state, weights, buf[lo:hi], start=pos + lo, logits=(hi == len(ids)))


def generate(state: DecodeState, weights: DeviceWeights, prompt_ids: Sequence[int], n_new: int, *,
             step=None, ignore_eos: bool = False, chunk: int | None = None) -> list[int]:
    """Host list of ``n_new`` greedy ids (shorter if EOS is hit and not ignored)."""
    consume_prompt(state, weights, prompt_ids, chunk=chunk)
    decode = greedy_decode if step is None else step
    out = [int(state.next_token.item())]
    if not ignore_eos:
        state.finished.bitwise_or_((state.next_token == state.eos_id).to(torch.uint8))
        if int(state.finished.item()) == 1:
            return out
    state.token.copy_(state.next_token)
    for _ in range(max(0, int(n_new) - 1)):
        decode(state, weights)
        out.append(int(state.token.item()))
        if not ignore_eos and int(state.finished.item()) == 1:
            break
    return out
