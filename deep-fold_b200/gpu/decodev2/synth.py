"""Seeded random-init NF4 decoders: no checkpoints, no CHR file.

``build(spec, seed)`` reproduces the reference's toy models draw for draw
(gpu/decodev2/synth.py:50-99: one numpy Generator, standard normal, scale 0.05
for matrices and 0.5 for vectors, in layer order q k v | wqkv, norm1, norm2, o,
gate, up, down, then embed, final norm, lm_head), so its published
(spec, seed, prompt) greedy ids apply to this repository's executors as well.

``build_device(spec, seed, device)`` makes the checkpoint-sized configurations:
weights ``0.02 * randn`` drawn and quantized on the GPU, q/k/v bias ``0.02 *
randn`` where the architecture has one, norm weights of ones, and an NF4 packed
embedding table (shared with lm_head when the architecture ties them).
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from gpu.host.codec import encode_nf4
from gpu.nf4.plan import k_pad

from .arch import ArchSpec

__all__ = ["Nf4Matrix", "SynthLayer", "SynthModel", "build"]


@dataclass
class Nf4Matrix:
    packed: np.ndarray
    scale: np.ndarray
    M: int
    K: int
    K_pad: int
    bias: np.ndarray | None = None


@dataclass
class SynthLayer:
    norm1: np.ndarray
    norm2: np.ndarray
    q: Nf4Matrix | None
    k: Nf4Matrix | None
    v: Nf4Matrix | None
    wqkv: Nf4Matrix | None
    o: Nf4Matrix
    gate: Nf4Matrix
    up: Nf4Matrix
    down: Nf4Matrix


@dataclass
class SynthModel:
    spec: ArchSpec
    seed: int
    embed: np.ndarray
    final_norm: np.ndarray
    lm_head: Nf4Matrix
    layers: list[SynthLayer]


def _mat(rng: np.random.Generator, m: int, k: int, std: float) -> Nf4Matrix:
    w = rng.standard_normal((m, k), dtype=np.float32) * np.float32(std)
    packed, scale = encode_nf4(w)
    return Nf4Matrix(packed, scale, m, k, k_pad(k))


def _vec(rng: np.random.Generator, n: int, std: float) -> np.ndarray:
    return rng.standard_normal(n, dtype=np.float32) * np.float32(std)


def build(spec: ArchSpec, seed: int) -> SynthModel:
    rng = np.random.default_rng(int(seed))
    h, kv, inter = spec.hidden, spec.kv_dim, spec.intermediate
    layers: list[SynthLayer] = []
    for _ in range(spec.n_layers):
        q = k = v = wqkv = None
        if spec.family == "llama_swiglu":
            q = _mat(rng, h, h, 0.05)
            k = _mat(rng, kv, h, 0.05)
            v = _mat(rng, kv, h, 0.05)
        else:
            wqkv = _mat(rng, spec.wqkv_out, h, 0.05)
        norm1 = _vec(rng, h, 0.5)
        norm2 = _vec(rng, h, 0.5)
        o = _mat(rng, h, h, 0.05)
        gate = _mat(rng, inter, h, 0.05)
        up = _mat(rng, inter, h, 0.05)
        down = _mat(rng, h, inter, 0.05)
        layers.append(SynthLayer(norm1, norm2, q, k, v, wqkv, o, gate, up, down))
    embed = _vec(rng, spec.vocab * h, 0.5).reshape(spec.vocab, h)
    final_norm = _vec(rng, h, 0.5)
    lm_head = _mat(rng, spec.vocab, h, 0.05)
    return SynthModel(spec, int(seed), embed, final_norm, lm_head, layers)
