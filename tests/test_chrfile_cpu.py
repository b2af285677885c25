"""A synthetic decoder through a CHR0 file and back on the CPU: the loader returns the very
bytes the model was built from, whole and per tensor-parallel rank."""

from __future__ import annotations

import dataclasses

import numpy as np
import pytest
import torch

from gpu.chr0.header import load_header
from gpu.decodev2.arch import MEDIUM_LLAMA, TINY_INTERNLM, TINY_LLAMA
from gpu.decodev2.chrfile import EMBED, LM_HEAD, load_weights, save_synth, tensor_names
from gpu.decodev2.synth import build
from gpu.decodev2.tp import shard_weights

from test_tp_cpu import cpu_weights


def same_linear(a, b) -> None:
    assert (a.M, a.K, a.K_pad) == (b.M, b.K, b.K_pad)
    assert torch.equal(a.packed.cpu().reshape(-1), b.packed.cpu().reshape(-1))
    assert torch.equal(a.scale.cpu().view(torch.int16).reshape(-1), b.scale.cpu().view(torch.int16).reshape(-1))


def same_weights(got, want) -> None:
    assert got.spec == want.spec
    same_linear(got.lm_head, want.lm_head)
    assert len(got.layers) == len(want.layers)
    for g, w in zip(got.layers, want.layers):
        for name in ("q", "k", "v", "wqkv", "o", "gate", "up", "down"):
            a, b = getattr(g, name), getattr(w, name)
            assert (a is None) == (b is None), name
            if a is not None:
                same_linear(a, b)


@pytest.mark.parametrize("spec,seed", [(TINY_LLAMA, 0), (TINY_INTERNLM, 1), (MEDIUM_LLAMA, 0)])
def test_file_round_trip_returns_the_models_bytes(tmp_path, spec, seed):
    model = build(spec, seed)
    path = save_synth(model, str(tmp_path / "m.chr"))
    hdr = load_header(path)
    assert (hdr.hidden_size, hdr.num_layers, hdr.vocab_size) == (spec.hidden, spec.n_layers, spec.vocab)
    assert EMBED in hdr and LM_HEAD in hdr and tensor_names(spec, 0)["down"] in hdr
    got = load_weights(path, spec, "cpu")
    same_weights(got, cpu_weights(model))
    from gpu.host.codec import encode_nf4

    e_packed, e_scale = encode_nf4(np.ascontiguousarray(model.embed, dtype=np.float32))
    assert got.embed.shape == (spec.vocab, spec.hidden)
    assert np.array_equal(got.embed.packed.numpy(), e_packed)
    assert np.array_equal(got.embed.scale.view(torch.int16).numpy().view(np.uint16),
                          np.asarray(e_scale).view(np.uint16))
    assert torch.equal(got.final_norm, torch.from_numpy(model.final_norm).to(torch.bfloat16))
    assert torch.equal(got.layers[0].norm1, torch.from_numpy(model.layers[0].norm1).to(torch.bfloat16))


MEDIUM_INTERNLM = dataclasses.replace(MEDIUM_LLAMA, name="medium-internlm", family="internlm_gqa",
                                      n_layers=2)


@pytest.mark.parametrize("spec,seed,world", [(MEDIUM_LLAMA, 0, 2), (MEDIUM_LLAMA, 0, 4),
                                             (MEDIUM_INTERNLM, 1, 2)])
def test_a_rank_reads_exactly_its_shard(tmp_path, spec, seed, world):
    model = build(spec, seed)
    path = save_synth(model, str(tmp_path / "m.chr"))
    full = cpu_weights(model)
    for rank in range(world):
        same_weights(load_weights(path, spec, "cpu", rank=rank, world=world),
                     shard_weights(full, rank, world))


def test_loader_refuses_a_file_of_another_model(tmp_path):
    path = save_synth(build(TINY_LLAMA, 0), str(tmp_path / "m.chr"))
    with pytest.raises(ValueError, match="differs"):
        load_weights(path, MEDIUM_LLAMA, "cpu")
