"""Resident greedy executor (Decode V2) on the B200 NF4 kernels."""

from __future__ import annotations

from .arch import (CONFIGS, INTERNLM25_20B, MEDIUM_LLAMA, QWEN25_3B, QWEN25_14B, QWEN25_32B,
                   TINY_INTERNLM, TINY_LLAMA, ArchSpec, shard_spec, with_max_seq)
from .chrfile import load_weights, save_synth, tensor_names
from .embed import PackedEmbed, bind_embed, gather_embed
from .graph import GreedyGraph, capture_greedy
from .linear import (DeviceLayer, DeviceLinear, DeviceWeights, linear_backend, nf4_linear,
                     set_linear_backend)
from .prefill import forward_prefill, prefill_chunk_width
from .rope import apply_rope_torch, rope_tables_numpy, rope_tables_torch
from .runner import PrefillGraphs, consume_prompt, generate
from .session import DecodeV2Loop, Generation
from .state import Arena, DecodeState, GraphSafeKV
from .step import forward_decode, greedy_decode, set_fuse_rms, teacher_force_token
from .synth import Nf4Matrix, SynthLayer, SynthModel, build
from .tp import Comm, shard_weights

__all__ = [
    "load_weights",
    "save_synth",
    "tensor_names",
    "PrefillGraphs",
    "ArchSpec", "Arena", "CONFIGS", "DecodeState", "DecodeV2Loop", "DeviceLayer", "DeviceLinear",
    "DeviceWeights", "Generation", "GraphSafeKV", "GreedyGraph", "INTERNLM25_20B", "MEDIUM_LLAMA",
    "Nf4Matrix", "PackedEmbed", "QWEN25_14B", "QWEN25_32B", "QWEN25_3B", "SynthLayer",
    "SynthModel", "TINY_INTERNLM", "TINY_LLAMA", "apply_rope_torch", "bind_embed", "build",
    "capture_greedy", "consume_prompt", "forward_decode", "forward_prefill", "gather_embed",
    "generate", "greedy_decode", "linear_backend", "nf4_linear", "prefill_chunk_width",
    "rope_tables_numpy", "rope_tables_torch", "set_fuse_rms", "set_linear_backend",
    "teacher_force_token", "with_max_seq", "Comm", "shard_spec", "shard_weights",
]
