"""``DecodeV2Loop``: the request-level API over the resident executor.

Keeps the reference's surface (gpu/decodev2/session.py:135-417 and the
``Generation`` record of gpu/loop/generate.py:254-294): ``generate``,
``prefill_from``, ``decode_from_logits``, ``seal_last``, ``warmup``,
``capture_graphs``, ``reset``. Prefill and decode are timed apart; graph capture
is never inside a timed window. ``generate_device_window`` is additive: it runs
the decode steps back to back with no per-token host read and returns the ids
afterwards, which is how the device-window tokens/s is measured.
"""

from __future__ import annotations

import time
from collections.abc import Callable, Sequence
from dataclasses import dataclass, field

import torch

from .graph import capture_greedy
from .linear import DeviceWeights
from .prefill import prefill_chunk_width
from .runner import PrefillGraphs, consume_prompt
from .state import DecodeState
from .step import greedy_decode, teacher_force_token

__all__ = ["DecodeV2Loop", "Generation"]


@dataclass
class Generation:
    """One greedy request; prefill and decode times are never averaged together."""

    prompt_len: int
    tokens: list[int] = field(default_factory=list)
    prefill_ms: float = 0.0
    decode_ms: float = 0.0
    decode_steps: int = 0
    stop_token: int | None = None
    interrupted: bool = False
    prefill_chunk: int = 1
    graph: str = "off"

    @property
    def decode_tok_s(self) -> float:
        """Steps after the first token over the decode window."""
        return self.decode_steps / (self.decode_ms / 1000.0) if self.decode_ms > 0 else 0.0

    @property
    def eval_tok_s(self) -> float:
        return len(self.tokens) / (self.decode_ms / 1000.0) if self.decode_ms > 0 else 0.0

    @property
    def prefill_tok_s(self) -> float:
        return self.prompt_len / (self.prefill_ms / 1000.0) if self.prefill_ms > 0 else 0.0

    @property
    def ms_per_token(self) -> float:
        return self.decode_ms / self.decode_steps if self.decode_steps else 0.0


class DecodeV2Loop:
    def __init__(self, state: DecodeState, weights: DeviceWeights) -> None:
        self.state = state
        self.weights = weights
        self.max_seq = int(state.spec.max_seq)
        self.prefill_chunk = prefill_chunk_width(state)
        self.graph_mode = "off"
        self.graph_error: str | None = None
        self._graph = None
        self._prefill_graphs: PrefillGraphs | None = None

    @classmethod
    def from_weights(cls, weights: DeviceWeights, *, dtype: torch.dtype = torch.bfloat16,
                     comm=None) -> "DecodeV2Loop":
        """``weights`` may be a tensor-parallel shard (``weights.spec.tp > 1``) with its ``comm``."""
        return cls(DecodeState.allocate(weights.spec, weights.embed, dtype=dtype, comm=comm), weights)

    @property
    def device(self) -> torch.device:
        return self.state.device

    @property
    def weight_bytes(self) -> int:
        return self.weights.nbytes

    def reset(self) -> None:
        self.state.reset()

    @staticmethod
    def _ids(prompt_ids) -> list[int]:
        if hasattr(prompt_ids, "reshape"):
            return [int(t) for t in prompt_ids.reshape(-1).tolist()]
        return [int(t) for t in prompt_ids]

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill_from(self, ids, start_pos: int, *, chunk: int | None = None) -> torch.Tensor:
        seq = self._ids(ids)
        pos = int(start_pos)
        if not seq:
            raise ValueError("empty prompt")
        if pos < 0 or pos + len(seq) > self.max_seq:
            raise ValueError(f"position {pos}+{len(seq)} past max_seq={self.max_seq}")
        consume_prompt(self.state, self.weights, seq, start=pos, chunk=chunk,
                       graphs=self._prefill_graphs)
        return self.state.arena.logits[0]

    forward = prefill_from

    @torch.no_grad()
    def seal_last(self, token_id: int) -> None:
        if int(self.state.valid_len.item()) >= self.max_seq:
            return
        teacher_force_token(self.state, self.weights, int(token_id))

    # ------------------------------------------------------------------- decode
    def check_exchange(self) -> None:
        """Raise if a bounded wait for a peer GPU ran out since the last check (tensor
        parallel with the peer-memory exchange): the ids produced since then are not to
        be trusted. One host read per exchange set; called after every decode window."""
        for px in (self.state.peers, self.state.pick_peers):
            if px is not None and px.timed_out():
                raise RuntimeError("a wait for a peer GPU ran out of polls during decode; "
                                   "the tensor-parallel sums since the last check are incomplete")

    def _step(self):
        return self._graph if self._graph is not None else greedy_decode

    def enable_prefill_graphs(self, on: bool = True, max_entries: int = 4) -> None:
        """Replay prefill chunks whose (start, length) has been seen before as CUDA graphs."""
        self._prefill_graphs = PrefillGraphs(self.state, self.weights, max_entries) if on else None

    @torch.no_grad()
    def decode_from_logits(self, logits, max_new_tokens: int, *, prompt_len: int,
                           stop: Sequence[int] = (),
                           on_token: Callable[[int], None] | None = None,
                           should_stop: Callable[[], bool] | None = None,
                           prefill_ms: float = 0.0) -> Generation:
        """Greedy decode after a prefill; the host reads one id per step."""
        del logits
        stop_set = frozenset(int(s) for s in stop)
        out = Generation(prompt_len=int(prompt_len), prefill_chunk=self.prefill_chunk,
                         graph=self.graph_mode, prefill_ms=float(prefill_ms))
        token = int(self.state.next_token.item())
        seq = int(self.state.valid_len.item())
        step = self._step()
        self.state.token.copy_(self.state.next_token)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        limit = max(0, int(max_new_tokens))
        for i in range(limit):
            if should_stop is not None and should_stop():
                out.interrupted = True
                break
            out.tokens.append(token)
            if on_token is not None:
                on_token(token)
            if token in stop_set:
                out.stop_token = token
                break
            if i + 1 == limit or seq >= self.max_seq:
                break
            step(self.state, self.weights)
            out.decode_steps += 1
            token = int(self.state.token.item())
            seq += 1
        torch.cuda.synchronize()
        out.decode_ms = (time.perf_counter() - t1) * 1000.0
        self.check_exchange()
        return out

    @torch.no_grad()
    def generate(self, prompt_ids, max_new_tokens: int = 64, *, stop: Sequence[int] = (),
                 on_token: Callable[[int], None] | None = None,
                 should_stop: Callable[[], bool] | None = None,
                 chunk: int | None = None) -> Generation:
        self.reset()
        ids = self._ids(prompt_ids)
        if not ids:
            raise ValueError("empty prompt")
        if len(ids) > self.max_seq:
            raise ValueError(f"prompt {len(ids)} exceeds max_seq={self.max_seq}")
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        logits = self.prefill_from(ids, 0, chunk=chunk)
        torch.cuda.synchronize()
        prefill_ms = (time.perf_counter() - t0) * 1000.0
        return self.decode_from_logits(logits, max_new_tokens, prompt_len=len(ids), stop=stop,
                                       on_token=on_token, should_stop=should_stop,
                                       prefill_ms=prefill_ms)

    @torch.no_grad()
    def generate_device_window(self, prompt_ids, max_new_tokens: int = 64, *,
                               chunk: int | None = None) -> Generation:
        """Same tokens as ``generate(..., stop=())`` with EOS ignored, but the decode
        steps are enqueued back to back and timed with CUDA events; ids are copied
        into a device buffer per step and read once at the end."""
        self.reset()
        ids = self._ids(prompt_ids)
        if not ids or len(ids) > self.max_seq:
            raise ValueError("prompt length out of range")
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        ev[0].record()
        self.prefill_from(ids, 0, chunk=chunk)
        ev[1].record()
        limit = max(1, min(int(max_new_tokens), self.max_seq - len(ids) + 1))
        trace = torch.zeros(limit, dtype=torch.int64, device=self.device)
        trace[0].copy_(self.state.next_token)
        self.state.token.copy_(self.state.next_token)
        step = self._step()
        ev[2].record()
        for i in range(1, limit):
            step(self.state, self.weights)
            trace[i].copy_(self.state.token)
        ev[3].record()
        torch.cuda.synchronize()
        out = Generation(prompt_len=len(ids), prefill_chunk=self.prefill_chunk, graph=self.graph_mode)
        out.tokens = [int(t) for t in trace.tolist()]
        out.prefill_ms = ev[0].elapsed_time(ev[1])
        out.decode_ms = ev[2].elapsed_time(ev[3])
        out.decode_steps = limit - 1
        self.check_exchange()
        return out

    # ------------------------------------------------------------ warm-up/graph
    def warmup(self, *, prompt: int = 8, tokens: int = 8) -> float:
        n = max(1, min(int(prompt), self.max_seq - 2))
        self.reset()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        consume_prompt(self.state, self.weights, [1] * n)
        self.state.token.copy_(self.state.next_token)
        for _ in range(max(0, min(int(tokens), 8, self.max_seq - n - 1))):
            greedy_decode(self.state, self.weights)
        torch.cuda.synchronize()
        self.reset()
        return (time.perf_counter() - t0) * 1000.0

    def capture_graphs(self) -> str:
        """Capture the greedy step once; on failure stay eager and keep the reason."""
        try:
            self.reset()
            self._graph = capture_greedy(self.state, self.weights, warmup=2)
            self.graph_mode = "decodev2"
            self.graph_error = None
        except Exception as exc:  # noqa: BLE001 - reported, not swallowed
            self._graph = None
            self.graph_mode = "off"
            self.graph_error = f"{type(exc).__name__}: {exc}"
        self.reset()
        return self.graph_mode
