"""One CUDA graph per greedy step; position / valid_len / token are device buffers,
so the same graph replays for every token (reference: gpu/decodev2/graph.py:16-55)."""

from __future__ import annotations

import gc

import torch

from .linear import DeviceWeights
from .state import DecodeState
from .step import greedy_decode

__all__ = ["GreedyGraph", "capture_greedy"]


class GreedyGraph:
    def __init__(self, graph: torch.cuda.CUDAGraph, state: DecodeState, weights: DeviceWeights):
        self.graph = graph
        self.state = state
        self.weights = weights

    def replay(self) -> None:
        self.graph.replay()

    def __call__(self, state: DecodeState, weights: DeviceWeights) -> None:
        if state is not self.state or weights is not self.weights:
            raise RuntimeError("replay is bound to the captured state/weights")
        self.graph.replay()


def capture_greedy(state: DecodeState, weights: DeviceWeights, *, warmup: int = 3,
                   step=greedy_decode) -> GreedyGraph:
    """Warm up eagerly on a side stream (first launches set function attributes),
    then capture one step. Warm-up and capture advance the device registers;
    callers snapshot/restore them (``DecodeV2Loop`` does)."""
    if state.device.type != "cuda":
        raise RuntimeError("greedy graph is CUDA-only")
    main = torch.cuda.current_stream()
    side = torch.cuda.Stream()
    side.wait_stream(main)
    with torch.cuda.stream(side):
        for _ in range(max(1, int(warmup))):
            step(state, weights)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step(state, weights)
    main.wait_stream(side)
    gc.collect()
    return GreedyGraph(graph, state, weights)
