"""CUDA-graph holders of the executor.

``capture_on_side_stream`` is the one place a graph is recorded: the decode step
(``capture_greedy`` / ``GreedyGraph``, the names of gpu/decodev2/graph.py:16-55)
and the prefill chunks (``runner.PrefillGraphs``) both go through it. Position,
valid length and token live in device buffers, so a captured step replays for
every token.
"""

from __future__ import annotations

from collections.abc import Callable

import torch

from .linear import DeviceWeights
from .state import DecodeState
from .step import greedy_decode

__all__ = ["GreedyGraph", "capture_greedy", "capture_on_side_stream"]


def capture_on_side_stream(body: Callable[[], None], *, warm_runs: int = 0) -> torch.cuda.CUDAGraph:
    """Record ``body`` into a fresh graph on a stream of its own.

    ``warm_runs`` eager executions come first on that same stream: the library sets
    kernel attributes and looks up device symbols on first use, which must not
    happen while a capture is open. The caller's stream waits for the side stream
    before this returns."""
    caller = torch.cuda.current_stream()
    lane = torch.cuda.Stream()
    lane.wait_stream(caller)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(lane):
        for _ in range(warm_runs):
            body()
        if warm_runs:
            lane.synchronize()
        with torch.cuda.graph(graph, stream=lane):
            body()
    caller.wait_stream(lane)
    return graph


class GreedyGraph:
    """One captured greedy step, callable like the eager step it stands for."""

    def __init__(self, graph: torch.cuda.CUDAGraph, state: DecodeState, weights: DeviceWeights):
        self.graph, self.state, self.weights = graph, state, weights

    def replay(self) -> None:
        self.graph.replay()

    def __call__(self, state: DecodeState, weights: DeviceWeights) -> None:
        if state is not self.state or weights is not self.weights:
            raise RuntimeError("this graph replays the state and weights it was captured with, "
                               "not the ones passed")
        self.graph.replay()


def capture_greedy(state: DecodeState, weights: DeviceWeights, *, warmup: int = 3,
                   step=greedy_decode) -> GreedyGraph:
    """Capture one ``step(state, weights)``. The warm-up runs and the capture advance
    the device registers; callers reset or restore them (``DecodeV2Loop`` does)."""
    if state.device.type != "cuda":
        raise RuntimeError("a decode graph needs the state on a CUDA device")
    graph = capture_on_side_stream(lambda: step(state, weights), warm_runs=max(1, int(warmup)))
    return GreedyGraph(graph, state, weights)
