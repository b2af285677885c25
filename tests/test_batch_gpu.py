"""Batched greedy decode: B sequences share every weight read; each keeps the
single-sequence semantics (own position, valid length, KV block)."""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu

from gpu.decodev2 import MEDIUM_LLAMA, TINY_INTERNLM, DecodeV2Loop, DeviceWeights, build  # noqa: E402
from gpu.decodev2.batch import BatchLoop  # noqa: E402


def weights_of(spec, seed, **kw):
    return DeviceWeights.from_synth(build(spec, seed), "cuda", torch.bfloat16, **kw)


@pytest.mark.parametrize("spec,seed,kw", [(MEDIUM_LLAMA, 0, {}), (MEDIUM_LLAMA, 0, {"packed_embed": True}),
                                          (TINY_INTERNLM, 1, {})])
def test_identical_prompts_give_identical_streams_equal_to_the_single_sequence_run(spec, seed, kw):
    weights = weights_of(spec, seed, **kw)
    prompt = [1, 3, 5, 7, 2]
    single = DecodeV2Loop.from_weights(weights).generate_device_window(prompt, 9).tokens
    loop = BatchLoop(weights, 4)
    streams = loop.generate([prompt] * 4, 9)
    assert all(s == streams[0] for s in streams)
    assert streams[0] == single
    # as a captured graph
    loop.state.prefill(weights, [prompt] * 4)
    loop.capture_graph()
    again = loop.generate([prompt] * 4, 9)
    assert again == streams


def test_different_prompts_and_lengths_decode_independently():
    weights = weights_of(MEDIUM_LLAMA, 0)
    prompts = [[1, 3, 5, 7], [4, 5, 6], [9, 8, 7, 6, 5, 4], [2]]
    one = DecodeV2Loop.from_weights(weights)
    want = [one.generate_device_window(p, 8).tokens for p in prompts]
    got = BatchLoop(weights, 4).generate(prompts, 8)
    assert got == want
    st = BatchLoop(weights, 4).state
    st.prefill(weights, prompts)
    assert st.position.tolist() == [len(p) for p in prompts]


def test_large_batch_goes_through_the_tensor_core_rows_path():
    """12 sequences: the linears run as GEMMs on activation rows (bf16 weight operand), so
    streams are compared among themselves and, for the first id, with the single run."""
    weights = weights_of(MEDIUM_LLAMA, 0)
    prompt = [1, 3, 5, 7]
    single = DecodeV2Loop.from_weights(weights).generate_device_window(prompt, 6).tokens
    streams = BatchLoop(weights, 12).generate([prompt] * 12, 6)
    assert all(s == streams[0] for s in streams) and streams[0][0] == single[0]


def test_batched_pick_equals_one_pick_per_sequence():
    """``chr_nf4_pick_commit_batch``: every sequence's pick, commit and EOS flag as the
    one-sequence entry gives them (lowest index on ties), scratch left zeroed."""
    from gpu.nf4 import nf4_pick_commit, nf4_pick_commit_batch

    b, n = 7, 40000
    gen = torch.Generator(device="cuda").manual_seed(9)
    logits = torch.randn((b, n + 8), generator=gen, device="cuda").to(torch.bfloat16)[:, :n]  # strided rows
    logits[2, 123] = logits[2].max() + 1
    logits[2, 77] = logits[2, 123]                      # a tie: the lower index wins
    logits[5, n - 1] = 100.0                             # the last column
    eos = 77
    nxt = torch.zeros(b, dtype=torch.int64, device="cuda")
    tok = torch.zeros(b, dtype=torch.int64, device="cuda")
    pos = torch.arange(b, dtype=torch.int64, device="cuda") * 10
    fin = torch.zeros(b, dtype=torch.uint8, device="cuda")
    scratch = torch.zeros((b, 16), dtype=torch.uint8, device="cuda")
    for _ in range(2):                                   # the second call finds the scratch as it must
        nf4_pick_commit_batch(logits, nxt, scratch, tok, pos, fin, eos)
    want = torch.zeros(b, dtype=torch.int64, device="cuda")
    one = torch.zeros((), dtype=torch.int64, device="cuda")
    s1 = torch.zeros(16, dtype=torch.uint8, device="cuda")
    for i in range(b):
        nf4_pick_commit(logits[i].contiguous(), one, s1)
        want[i] = one
    assert torch.equal(nxt, want) and torch.equal(tok, want)
    assert int(nxt[2]) == 77 and int(nxt[5]) == n - 1
    assert torch.equal(pos, torch.arange(b, dtype=torch.int64, device="cuda") * 10 + 2)
    assert fin.tolist() == [1 if int(t) == eos else 0 for t in want.tolist()]
    assert not scratch.any()
