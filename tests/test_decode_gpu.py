"""Resident executor on the GPU: greedy ids against the reference's float32 oracle
(recorded in tests/golden), graph replay against eager, chunked prefill against
token-by-token, packed embedding against dense, no allocation on the step path.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import model_ref as mr

pytestmark = pytest.mark.gpu

from gpu.decodev2 import (MEDIUM_LLAMA, TINY_INTERNLM, TINY_LLAMA, DecodeState, DecodeV2Loop,  # noqa: E402
                          DeviceWeights, build, capture_greedy, consume_prompt, generate,
                          greedy_decode, set_fuse_rms, teacher_force_token)

CASES = {
    "tiny_llama_s0_p1357": (TINY_LLAMA, 0),
    "tiny_llama_s0_p456": (TINY_LLAMA, 0),
    "tiny_internlm_s1_p1357": (TINY_INTERNLM, 1),
    "medium_llama_s0_p1357": (MEDIUM_LLAMA, 0),
}


def session(spec, seed, **kw):
    model = build(spec, seed)
    weights = DeviceWeights.from_synth(model, "cuda", torch.bfloat16, **kw)
    state = DecodeState.allocate(spec, weights.embed)
    return model, state, weights


def greedy_by_steps(state, weights, prompt, n_new):
    for tok in prompt:
        teacher_force_token(state, weights, tok)
    out = [int(state.next_token.item())]
    state.token.copy_(state.next_token)
    for _ in range(n_new - 1):
        if out[-1] == int(state.spec.eos_id):
            break
        greedy_decode(state, weights)
        out.append(int(state.token.item()))
    return out


@pytest.mark.parametrize("tag", sorted(CASES))
@pytest.mark.parametrize("fused", [True, False])
def test_eager_greedy_ids_match_reference_oracle(golden, tag, fused):
    g = golden("decodev2_oracle.npz")
    spec, seed = CASES[tag]
    _, state, weights = session(spec, seed)
    set_fuse_rms(fused)
    try:
        got = greedy_by_steps(state, weights, g[tag + "_prompt"].tolist(), 8)
    finally:
        set_fuse_rms(True)
    want = g[tag + "_greedy"].tolist()
    assert got == want[: len(got)] and len(got) == len(want)


@pytest.mark.parametrize("tag", sorted(CASES))
def test_teacher_forced_logits_track_the_oracle(golden, tag):
    g = golden("decodev2_oracle.npz")
    spec, seed = CASES[tag]
    _, state, weights = session(spec, seed)
    want = g[tag + "_teacher"]
    for i, tok in enumerate(g[tag + "_prompt"].tolist()):
        teacher_force_token(state, weights, tok)
        got = state.arena.logits[0].float().cpu().numpy()
        top2 = np.sort(want[i])[-2:]
        # logits are stored as bf16: only a margin above a few ulps pins the argmax
        if top2[1] - top2[0] > 8 * 2.0 ** -8 * np.abs(want[i]).max():
            assert int(state.next_token.item()) == int(want[i].argmax())
        assert np.abs(got - want[i]).max() <= 0.05 * max(1.0, np.abs(want[i]).max())


@pytest.mark.parametrize("spec,seed", [(TINY_LLAMA, 0), (TINY_INTERNLM, 1), (MEDIUM_LLAMA, 0)])
def test_graph_replay_equals_eager(spec, seed):
    prompt = [1, 3, 5, 7]
    _, s_eager, w = session(spec, seed)
    eager = greedy_by_steps(s_eager, w, prompt, 9)
    _, s_graph, w2 = session(spec, seed)
    graph = capture_greedy(s_graph, w2, warmup=2)
    s_graph.reset()
    for tok in prompt:
        teacher_force_token(s_graph, w2, tok)
    out = [int(s_graph.next_token.item())]
    s_graph.token.copy_(s_graph.next_token)
    for _ in range(8):
        graph.replay()
        out.append(int(s_graph.token.item()))
    # the eager helper stops at EOS, the replay loop does not
    assert out[: len(eager)] == eager and (len(eager) == 9 or eager[-1] == spec.eos_id)
    assert int(s_graph.position.item()) == len(prompt) + 8
    assert int(s_graph.valid_len.item()) == len(prompt) + 8


def test_step_path_does_not_allocate():
    _, state, weights = session(MEDIUM_LLAMA, 0)
    for tok in (1, 3, 5):
        teacher_force_token(state, weights, tok)
    state.token.copy_(state.next_token)
    greedy_decode(state, weights)
    torch.cuda.synchronize()
    before = torch.cuda.memory_stats()["allocation.all.allocated"]
    held = torch.cuda.memory_allocated()
    for _ in range(4):
        greedy_decode(state, weights)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == held
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == before


def test_dirty_kv_tail_is_ignored():
    _, clean, w = session(TINY_LLAMA, 0)
    _, dirty, w2 = session(TINY_LLAMA, 0)
    teacher_force_token(clean, w, 1)
    teacher_force_token(dirty, w2, 1)
    dirty.kv.k[:, -1].fill_(1.0e4)
    dirty.kv.v[:, -1].fill_(1.0e4)
    teacher_force_token(clean, w, 3)
    teacher_force_token(dirty, w2, 3)
    assert torch.equal(clean.arena.logits, dirty.arena.logits)


@pytest.mark.parametrize("spec,seed", [(TINY_LLAMA, 0), (TINY_INTERNLM, 1), (MEDIUM_LLAMA, 0)])
@pytest.mark.parametrize("chunk", [None, 3, 1])
def test_chunked_prefill_tracks_token_by_token(spec, seed, chunk):
    prompt = [1, 3, 5, 7, 2, 9, 11]
    model, s_tok, w = session(spec, seed)
    for tok in prompt:
        teacher_force_token(s_tok, w, tok)
    _, s_pre, w2 = session(spec, seed)
    consume_prompt(s_pre, w2, prompt, chunk=chunk)
    assert int(s_pre.position.item()) == len(prompt) == int(s_pre.valid_len.item())
    want = mr.teacher_logits(model, prompt)[-1]
    got = s_pre.arena.logits[0].float().cpu().numpy()
    assert np.abs(got - want).max() <= 0.05 * max(1.0, np.abs(want).max())
    assert int(s_pre.next_token.item()) == int(want.argmax())
    # KV rows written by the GEMM prefill and by GEMV decode agree to bf16 noise
    n = len(prompt)
    dk = (s_pre.kv.k[:, :n].float() - s_tok.kv.k[:, :n].float()).abs().max().item()
    assert dk <= 0.05 * max(1.0, s_tok.kv.k[:, :n].float().abs().max().item())


def test_generate_and_loop_agree_with_oracle(golden):
    g = golden("decodev2_oracle.npz")
    tag = "medium_llama_s0_p1357"
    model, state, weights = session(MEDIUM_LLAMA, 0)
    prompt = g[tag + "_prompt"].tolist()
    got = generate(state, weights, prompt, 8, ignore_eos=True)
    want = mr.greedy_ids(model, prompt, 8)
    assert got[: len(want)] == want
    loop = DecodeV2Loop(state, weights)
    assert loop.capture_graphs() == "decodev2", loop.graph_error
    res = loop.generate(torch.tensor(prompt), 8)
    assert res.tokens == got[: len(res.tokens)] and res.graph == "decodev2"
    assert res.decode_steps == len(res.tokens) - 1 and res.prefill_ms > 0 and res.decode_ms > 0
    win = loop.generate_device_window(prompt, 8)
    assert win.tokens == got


def test_packed_embed_equals_dense_of_same_codes():
    import nf4_ref as o

    model = build(MEDIUM_LLAMA, 0)
    packed_w = DeviceWeights.from_synth(model, "cuda", packed_embed=True)
    p, s = o.quantize(np.ascontiguousarray(model.embed, dtype=np.float32))
    model.embed = o.dequantize(p, s, *model.embed.shape)
    dense_w = DeviceWeights.from_synth(model, "cuda")
    sp = DecodeState.allocate(MEDIUM_LLAMA, packed_w.embed)
    sd = DecodeState.allocate(MEDIUM_LLAMA, dense_w.embed)
    a = greedy_by_steps(sp, packed_w, [1, 3, 5, 7], 8)
    b = greedy_by_steps(sd, dense_w, [1, 3, 5, 7], 8)
    assert a == b and torch.equal(sp.arena.logits, sd.arena.logits)
    assert int(sp.arena.status.item()) == 0


def test_state_reset_and_registers():
    _, state, weights = session(TINY_LLAMA, 0)
    teacher_force_token(state, weights, 1)
    assert int(state.position.item()) == 1 and int(state.valid_len.item()) == 1
    state.reset()
    assert int(state.position.item()) == 0 and int(state.valid_len.item()) == 0
    with pytest.raises(ValueError):
        consume_prompt(state, weights, list(range(17)))
    with pytest.raises(RuntimeError):
        DecodeState.allocate(TINY_LLAMA, torch.zeros(32, 64), device="cpu")


def test_token_loop_mma_path_tracks_decode_v2():
    from gpu.loop import TokenLoop

    model, state, weights = session(MEDIUM_LLAMA, 0)
    prompt = [1, 3, 5, 7]
    want = mr.greedy_ids(model, prompt, 8)
    loop = TokenLoop(state, weights)
    eager = loop.generate(torch.tensor(prompt), 8).tokens
    assert loop.capture_graphs() == "tokenloop", loop.graph_error
    graphed = loop.generate(torch.tensor(prompt), 8)
    assert graphed.tokens == eager and graphed.graph == "tokenloop"
    # the MMA path rounds W to bf16, so only the prefill token is pinned to the oracle;
    # later ids may part at near-ties
    assert eager[0] == want[0] and len(eager) == len(want)
    loop.reset()
    loop.prefill_from(prompt, 0)
    loop.state.token.copy_(loop.state.next_token)
    assert loop.step() == eager[1]
    # teacher-forced through the MMA step: its logits stay within the tolerance of the
    # float32 oracle at every position, and the argmax agrees wherever the oracle's
    # top-2 margin is more than a few bf16 ulps (the reference's own protocol for its
    # MMA loop, gpu/decodev2/test_step.py:45-50)
    from gpu.loop.generate import mma_decode

    loop._graph = None
    loop.reset()
    seq = prompt + want[:6]
    teacher = mr.teacher_logits(model, seq)
    for i, tok in enumerate(seq):
        loop.state.load_token(tok)
        mma_decode(loop.state, loop.weights)
        got = loop.state.arena.logits[0].float().cpu().numpy()
        assert np.abs(got - teacher[i]).max() <= 0.05 * max(1.0, np.abs(teacher[i]).max())
        top2 = np.sort(teacher[i])[-2:]
        if top2[1] - top2[0] > 8 * 2.0 ** -8 * np.abs(teacher[i]).max():
            assert int(loop.state.next_token.item()) == int(teacher[i].argmax())


def test_host_seats_linear_and_embedding(golden):
    import nf4_ref as o
    from gpu.chr0.loader import ChrMatrix
    from gpu.host.embedding import Nf4Embedding, dequant_nf4_rows
    from gpu.host.linear import CompressedLinear

    rng = np.random.default_rng(0)
    m, k = 192, 256
    w = (rng.standard_normal((m, k)) * 0.02).astype(np.float32)
    p, s = o.quantize(w)
    mat = ChrMatrix("toy", m, k, k, torch.from_numpy(p).cuda(), torch.from_numpy(s).cuda())
    seat = CompressedLinear(k, m, bias=True, device="cuda")
    assert not seat.is_loaded and seat.weight.numel() == 0
    with pytest.raises(RuntimeError):
        seat(torch.zeros(1, k, device="cuda", dtype=torch.bfloat16))
    bias = torch.from_numpy(rng.standard_normal(m).astype(np.float32)).to(torch.bfloat16)
    seat.attach(mat, bias)
    x = torch.from_numpy(rng.standard_normal((2, 5, k)).astype(np.float32)).to(torch.bfloat16).cuda()
    y = seat(x)
    assert y.shape == (2, 5, m) and y.dtype is torch.bfloat16
    want = x.float().cpu().numpy().reshape(10, k) @ o.dequantize_bf16(p, s, m, k).T + bias.float().numpy()
    assert np.abs(y.float().cpu().numpy().reshape(10, m) - want).max() <= 1e-2 * np.abs(want).max()
    with pytest.raises(ValueError):
        CompressedLinear(k + 64, m).attach(mat)
    g = golden("embed_rows.npz")
    emb = Nf4Embedding(40, 200, device="cuda")
    emb.attach(ChrMatrix("e", 40, 200, 256, torch.from_numpy(g["packed"]).cuda(),
                         torch.from_numpy(g["scale"].view(np.float16)).cuda()))
    ids = torch.from_numpy(g["ids"]).cuda()
    rows = emb(ids.view(1, -1))
    assert rows.shape == (1, 5, 200)
    assert np.array_equal(rows.view(torch.int16).cpu().numpy().view(np.uint16).reshape(5, 200),
                          g["rows_bf16_bits"])
    assert torch.equal(dequant_nf4_rows(emb.packed, emb.scale, ids, 200), rows.view(5, 200))


def test_prefill_graphs_replay_equals_eager():
    _, state, weights = session(MEDIUM_LLAMA, 0)
    loop = DecodeV2Loop(state, weights)
    prompt = [1, 3, 5, 7, 2, 9, 4]
    want = loop.generate_device_window(prompt, 6).tokens
    want_k = state.kv.k.clone()
    loop.enable_prefill_graphs()
    first = loop.generate_device_window(prompt, 6).tokens        # eager + capture
    again = loop.generate_device_window(prompt, 6).tokens        # replay
    other = loop.generate_device_window([9, 8, 7, 6, 5, 4, 3], 6).tokens   # same shape, new ids
    assert loop._prefill_graphs.replays == 2
    assert first == want and again == want
    loop.enable_prefill_graphs(False)
    assert other == loop.generate_device_window([9, 8, 7, 6, 5, 4, 3], 6).tokens
    loop.generate_device_window(prompt, 6)
    assert torch.equal(state.kv.k, want_k)


@pytest.mark.parametrize("spec,seed", [(MEDIUM_LLAMA, 0), (TINY_INTERNLM, 1)])
def test_weights_loaded_from_a_chr_file_decode_like_the_model_they_came_from(tmp_path, spec, seed):
    from gpu.decodev2 import load_weights, save_synth

    model = build(spec, seed)
    path = save_synth(model, str(tmp_path / "model.chr"))
    loaded = load_weights(path, spec, "cuda")
    direct = DeviceWeights.from_synth(model, "cuda", torch.bfloat16, packed_embed=True)
    for a, b in zip(loaded.layers, direct.layers):
        for name in ("q", "k", "v", "wqkv", "o", "gate", "up", "down"):
            x, y = getattr(a, name), getattr(b, name)
            assert (x is None) == (y is None)
            if x is not None:
                assert torch.equal(x.packed, y.packed) and torch.equal(x.scale, y.scale)
    prompt = [1, 3, 5, 7, 2]
    want = DecodeV2Loop.from_weights(direct).generate_device_window(prompt, 8).tokens
    loop = DecodeV2Loop.from_weights(loaded)
    assert loop.generate_device_window(prompt, 8).tokens == want
    assert loop.capture_graphs() == "decodev2", loop.graph_error
    assert loop.generate_device_window(prompt, 8).tokens == want


def test_prefill_with_fused_row_kernels_matches_the_torch_op_prefill():
    from gpu.decodev2.prefill import set_fused_rows

    _, state, weights = session(MEDIUM_LLAMA, 0)
    loop = DecodeV2Loop(state, weights)
    prompt = list(range(1, 21))
    try:
        set_fused_rows(False)
        want = loop.generate_device_window(prompt, 8).tokens
        want_v = state.kv.v.clone()
        want_k = state.kv.k.clone()
    finally:
        set_fused_rows(True)
    got = loop.generate_device_window(prompt, 8).tokens
    assert got == want
    assert torch.equal(state.kv.v[0], want_v[0]) and torch.equal(state.kv.k[0], want_k[0])
    # deeper layers see RMSNorm rounded by the decode formula instead of torch's: close, not equal
    assert (state.kv.k.float() - want_k.float()).abs().max() <= 0.05 * want_k.float().abs().max()
