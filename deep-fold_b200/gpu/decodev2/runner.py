"""Greedy runner: chunked GEMM prefill, then decode steps that stay on the GPU
(reference: gpu/decodev2/runner.py:17-81)."""

from __future__ import annotations

from collections.abc import Sequence

import torch

from .graph import capture_on_side_stream
from .linear import DeviceWeights
from .prefill import forward_prefill, prefill_chunk_width
from .state import DecodeState
from .step import greedy_decode

__all__ = ["PrefillGraphs", "consume_prompt", "generate"]


class PrefillGraphs:
    """Prefill chunks as CUDA graphs, keyed by (start slot, length, logits wanted).

    A prefill chunk is ~30 small launches per layer around the GEMMs, issued from
    Python; for a prompt shape that comes back (same length bucket, same start) the
    whole chunk replays as one graph instead. The first time a shape is seen it runs
    eagerly (which also warms every kernel) and is then captured for the next time;
    the token ids live in a static device buffer the replay reads. At most
    ``max_entries`` shapes are kept (least recently used goes first). Under tensor
    parallelism the chunk's NCCL all-reduces are captured with it, so every rank must see
    the same sequence of prompt shapes, and the graphs have to be dropped before the
    process group is destroyed (``Comm.shutdown`` does).
    """

    def __init__(self, state: DecodeState, weights: DeviceWeights, max_entries: int = 4) -> None:
        self.state, self.weights, self.max_entries = state, weights, int(max_entries)
        self._cache: dict = {}
        self.replays = 0

    def run(self, ids: torch.Tensor, start: int, logits: bool) -> None:
        key = (int(start), int(ids.numel()), bool(logits))
        entry = self._cache.pop(key, None)
        if entry is not None:
            static_ids, graph = entry
            static_ids.copy_(ids)
            graph.replay()
            self.replays += 1
            self._cache[key] = entry  # most recently used last
            return
        forward_prefill(self.state, self.weights, ids, start=start, logits=logits)
        static_ids = ids.clone()
        graph = capture_on_side_stream(
            lambda: forward_prefill(self.state, self.weights, static_ids, start=start, logits=logits))
        while len(self._cache) >= self.max_entries:
            self._cache.pop(next(iter(self._cache)))
        self._cache[key] = (static_ids, graph)


def consume_prompt(state: DecodeState, weights: DeviceWeights, token_ids: Sequence[int], *,
                   chunk: int | None = None, start: int = 0,
                   graphs: PrefillGraphs | None = None) -> None:
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
        if graphs is not None:
            graphs.run(buf[lo:hi], pos + lo, hi == len(ids))
        else:
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
