"""The float32 decoder oracle against ids/logits recorded from the reference's oracle."""

from __future__ import annotations

import numpy as np
import pytest

import model_ref as mr
from gpu.decodev2.arch import MEDIUM_LLAMA, TINY_INTERNLM, TINY_LLAMA
from gpu.decodev2.synth import build

CASES = {
    "tiny_llama_s0_p1357": (TINY_LLAMA, 0),
    "tiny_llama_s0_p456": (TINY_LLAMA, 0),
    "tiny_internlm_s1_p1357": (TINY_INTERNLM, 1),
    "medium_llama_s0_p1357": (MEDIUM_LLAMA, 0),
}


@pytest.mark.parametrize("tag", sorted(CASES))
def test_greedy_and_teacher_match_reference(golden, tag):
    g = golden("decodev2_oracle.npz")
    spec, seed = CASES[tag]
    model = build(spec, seed)
    prompt = g[tag + "_prompt"].tolist()
    assert mr.greedy_ids(model, prompt, 8) == g[tag + "_greedy"].tolist()
    np.testing.assert_allclose(mr.teacher_logits(model, prompt), g[tag + "_teacher"],
                               rtol=0, atol=2e-5)


def test_rope_tables_and_rotation_match_reference(golden):
    from gpu.decodev2.rope import rope_tables_numpy

    g = golden("rope.npz")
    for fn in (mr.rope_tables, rope_tables_numpy):
        cos, sin = fn(16, 16, 10000.0)
        assert np.array_equal(cos, g["cos"]) and np.array_equal(sin, g["sin"])
        cos6, sin6 = fn(8, 128, 1.0e6)
        assert np.array_equal(cos6, g["cos6"]) and np.array_equal(sin6, g["sin6"])
    cos, sin = mr.rope_tables(16, 16, 10000.0)
    assert np.array_equal(mr.rotate(g["t"], cos[4:6], sin[4:6]), g["t_rot"])


def test_dirty_cache_tail_is_ignored():
    model = build(TINY_LLAMA, 0)
    clean, dirty = mr.Cache(TINY_LLAMA), mr.Cache(TINY_LLAMA)
    mr.step_logits(model, clean, 1)
    mr.step_logits(model, dirty, 1)
    dirty.k[:, -1] = 1.0e4
    dirty.v[:, -1] = 1.0e4
    assert np.array_equal(mr.step_logits(model, clean, 3), mr.step_logits(model, dirty, 3))
