"""Tensor-parallel host logic on CPU: shard arithmetic against the oracle, and the two
collectives of the step through a world-size-2 gloo group."""

from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import nf4_ref as o
from gpu.decodev2.arch import (MEDIUM_LLAMA, QWEN25_3B, QWEN25_14B, QWEN25_32B, INTERNLM25_20B,
                               group_range, shard_spec)
from gpu.decodev2.linear import DeviceLayer, DeviceLinear, DeviceWeights
from gpu.decodev2.synth import build
from gpu.decodev2.tp import Comm, kv_head_rows, shard_linear_cols, shard_linear_rows, shard_weights


def cpu_linear(mat) -> DeviceLinear:
    return DeviceLinear(torch.from_numpy(mat.packed.copy()), torch.from_numpy(mat.scale.copy()),
                        mat.M, mat.K, mat.K_pad, None)


def cpu_weights(model) -> DeviceWeights:
    c = lambda m: None if m is None else cpu_linear(m)
    layers = [DeviceLayer(torch.from_numpy(l.norm1), torch.from_numpy(l.norm2), c(l.q), c(l.k),
                          c(l.v), c(l.wqkv), c(l.o), c(l.gate), c(l.up), c(l.down))
              for l in model.layers]
    return DeviceWeights(model.spec, torch.from_numpy(model.embed), torch.from_numpy(model.final_norm),
                         c(model.lm_head), layers)


def deq(lin: DeviceLinear) -> np.ndarray:
    return o.dequantize(lin.packed.numpy(), lin.scale.numpy(), lin.M, lin.K)


def test_group_range_covers_axis_in_whole_groups():
    for total, world in ((11008, 8), (11008, 4), (27648, 8), (1024, 2), (128, 2)):
        edges = [group_range(total, world, r) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
        assert all(lo % 64 == 0 and hi % 64 == 0 and hi > lo for lo, hi in edges)
        sizes = [hi - lo for lo, hi in edges]
        assert max(sizes) - min(sizes) <= 64


@pytest.mark.parametrize("spec,world", [(QWEN25_3B, 2), (QWEN25_3B, 4), (QWEN25_3B, 8), (QWEN25_14B, 2),
                                        (INTERNLM25_20B, 8), (QWEN25_32B, 8), (QWEN25_32B, 4)])
def test_shard_spec_sizes(spec, world):
    shards = [shard_spec(spec, world, r) for r in range(world)]
    assert sum(s.intermediate for s in shards) == spec.intermediate
    assert all(s.hidden == spec.hidden and s.vocab == spec.vocab and s.tp == world for s in shards)
    assert all(s.n_q * world == spec.n_q for s in shards)
    if spec.n_kv >= world:
        assert all(s.n_kv * world == spec.n_kv and s.kv_replicas == 1 for s in shards)
    else:
        assert all(s.n_kv == 1 and s.kv_replicas == world // spec.n_kv for s in shards)
        rows = [kv_head_rows(spec, r, world) for r in range(world)]
        assert rows[0] == rows[world // spec.n_kv - 1] and rows[0] != rows[world // spec.n_kv]
    with pytest.raises(ValueError):
        shard_spec(shards[0], 2)


def test_shards_reassemble_the_full_matrices():
    model = build(MEDIUM_LLAMA, 0)
    full = cpu_weights(model)
    world = 2
    x = np.random.default_rng(0).standard_normal(MEDIUM_LLAMA.hidden).astype(np.float32)
    shards = [shard_weights(full, r, world) for r in range(world)]
    ly, parts = full.layers[0], [s.layers[0] for s in shards]
    # column splits: rows concatenate back, bytes untouched
    for name in ("q", "gate", "up"):
        cat = np.concatenate([deq(getattr(p, name)) for p in parts])
        assert np.array_equal(cat, deq(getattr(ly, name)))
    assert np.array_equal(np.concatenate([deq(p.k) for p in parts]), deq(ly.k))
    assert np.array_equal(np.concatenate([deq(s.lm_head) for s in shards]), deq(full.lm_head))
    # row splits: K ranges concatenate back, partial products sum to the full product
    for name, vec in (("o", x), ("down", np.random.default_rng(1).standard_normal(1024).astype(np.float32))):
        mats = [getattr(p, name) for p in parts]
        assert np.array_equal(np.concatenate([deq(m) for m in mats], axis=1), deq(getattr(ly, name)))
        lo = 0
        acc = np.zeros(mats[0].M, dtype=np.float64)
        for m in mats:
            acc += deq(m).astype(np.float64) @ vec[lo:lo + m.K]
            lo += m.K
        np.testing.assert_allclose(acc, deq(getattr(ly, name)).astype(np.float64) @ vec, rtol=1e-12)
    assert shard_weights(full, 0, 1) is full
    with pytest.raises(ValueError):
        shard_linear_rows(cpu_linear(model.layers[0].o), 0, 2, (0, 100))
    with pytest.raises(ValueError):
        shard_linear_cols(cpu_linear(model.layers[0].q), 0, 3)


@pytest.mark.parametrize("world", [4, 8])
def test_uneven_shares_and_replicated_kv_heads_reproduce_one_layer(world):
    """704 = 11 NF4 groups do not divide by 4 or 8 and 2 kv heads are fewer than the ranks:
    the per-rank MLP partials still sum to the full product and every rank's q heads sit
    next to the kv head they attend."""
    import dataclasses

    spec = dataclasses.replace(MEDIUM_LLAMA, name="uneven", n_layers=1, intermediate=704)
    model = build(spec, 3)
    full = cpu_weights(model)
    shards = [shard_weights(full, r, world) for r in range(world)]
    ly = full.layers[0]
    rng = np.random.default_rng(5)
    h = rng.standard_normal(spec.hidden)
    silu = lambda t: t / (1.0 + np.exp(-t))
    want = deq(ly.down).astype(np.float64) @ (silu(deq(ly.gate).astype(np.float64) @ h)
                                               * (deq(ly.up).astype(np.float64) @ h))
    acc = np.zeros(spec.hidden)
    covered = 0
    for r, sh in enumerate(shards):
        part = sh.layers[0]
        lo, hi = group_range(spec.intermediate, world, r)
        assert lo % 64 == 0 and hi % 64 == 0 and part.gate.M == hi - lo == part.down.K
        covered += hi - lo
        act = silu(deq(part.gate).astype(np.float64) @ h) * (deq(part.up).astype(np.float64) @ h)
        acc += deq(part.down).astype(np.float64) @ act
        # attention: this rank's q heads and the kv head stored beside them
        heads = spec.n_q // world
        first = r * heads
        assert np.array_equal(deq(part.q), deq(ly.q)[first * spec.head_dim:(first + heads) * spec.head_dim])
        kvh = first // spec.n_rep
        assert (first + heads - 1) // spec.n_rep == kvh
        assert np.array_equal(deq(part.k), deq(ly.k)[kvh * spec.head_dim:(kvh + 1) * spec.head_dim])
        assert np.array_equal(deq(part.v), deq(ly.v)[kvh * spec.head_dim:(kvh + 1) * spec.head_dim])
        assert sh.spec.n_kv == 1 and sh.spec.n_q == heads
    assert covered == spec.intermediate
    np.testing.assert_allclose(acc, want, rtol=1e-10, atol=1e-12)
    sizes = {sh.layers[0].down.K for sh in shards}
    assert len(sizes) == 2  # the shares really are uneven


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, out_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        model = build(MEDIUM_LLAMA, 0)
        full = cpu_weights(model)
        mine = shard_weights(full, rank, world)
        comm = Comm.from_env()
        assert (comm.rank, comm.world) == (rank, world)
        rng = np.random.default_rng(3)
        attn = rng.standard_normal(MEDIUM_LLAMA.hidden).astype(np.float32)     # full o-proj input
        o_shard = mine.layers[0].o
        lo = rank * o_shard.K
        part = torch.from_numpy(deq(o_shard) @ attn[lo:lo + o_shard.K])
        comm.all_reduce_sum(part)
        want = deq(full.layers[0].o) @ attn
        assert np.abs(part.numpy() - want).max() <= 1e-4
        # logits slices gathered in rank order
        h = rng.standard_normal(MEDIUM_LLAMA.hidden).astype(np.float32)
        local = torch.from_numpy(deq(mine.lm_head) @ h)
        gathered = torch.empty(MEDIUM_LLAMA.vocab, dtype=torch.float32)
        comm.all_gather_into(gathered, local)
        assert np.abs(gathered.numpy() - deq(full.lm_head) @ h).max() <= 1e-5
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")

        class _Loop:  # what shutdown() is handed: something that may hold a captured graph
            _graph, graph_mode = object(), "decodev2"

        holder = _Loop()
        comm.shutdown(holder)
        assert holder._graph is None and not dist.is_initialized()
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_two_rank_gloo_collectives(tmp_path):
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_single_rank_comm_is_a_no_op():
    comm = Comm()
    t = torch.arange(4.0)
    assert comm.all_reduce_sum(t) is t and torch.equal(t, torch.arange(4.0))
    out = torch.zeros(4)
    comm.all_gather_into(out, t)
    assert torch.equal(out, t)


def test_adjoin_rows_stacks_matrices_and_turns_the_handles_into_views():
    from gpu.decodev2.linear import adjoin_rows

    model = build(MEDIUM_LLAMA, 0)
    ly = model.layers[0]
    q, k, v = cpu_linear(ly.q), cpu_linear(ly.k), cpu_linear(ly.v)
    q.bias = torch.arange(q.M, dtype=torch.float32).to(torch.bfloat16)
    want = [deq(m) for m in (q, k, v)]
    stacked = adjoin_rows([q, k, v])
    assert stacked.M == q.M + k.M + v.M and stacked.K == q.K
    assert np.array_equal(deq(stacked), np.concatenate(want))
    # the handles now alias the blob, in order, without a second copy
    assert q.packed.data_ptr() == stacked.packed.data_ptr()
    assert k.packed.data_ptr() == stacked.packed.data_ptr() + q.M * (q.K_pad // 2)
    assert v.scale.data_ptr() == stacked.scale.data_ptr() + (q.M + k.M) * (q.K_pad // 64) * 2
    for m, w in zip((q, k, v), want):
        assert m.packed.is_contiguous() and np.array_equal(deq(m), w)
    assert stacked.bias is not None and stacked.bias.numel() == stacked.M
    assert torch.equal(stacked.bias[: q.M], q.bias) and not stacked.bias[q.M:].any()
    with pytest.raises(ValueError):
        adjoin_rows([cpu_linear(ly.q), cpu_linear(ly.down)])


def _gemv_shape(n_rows: int, k_pad: int, swiglu: bool = False):
    import ctypes

    from gpu.nf4 import _lib

    out = (ctypes.c_int32 * 6)()
    rc = _lib.load().chr_nf4_gemv_shape(n_rows, k_pad, int(swiglu), out)
    return rc, tuple(out)


@pytest.mark.parametrize("spec", [QWEN25_3B, QWEN25_14B, INTERNLM25_20B, QWEN25_32B])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_gemv_work_split_is_valid_and_agreed_between_ranks(spec, world):
    """The fused exchange needs every rank to tile a row-split matrix alike: with the widest
    share's K_pad as the hint they do, and the split stays inside the kernels' limits."""
    if world > 1:
        try:
            shard_spec(spec, world)
        except ValueError:
            pytest.skip("this architecture does not shard that way")
    q_dim = spec.n_q * spec.head_dim
    for full_k in (q_dim, spec.intermediate):
        shares = [group_range(full_k, world, r) for r in range(world)] if world > 1 else [(0, full_k)]
        widest = max(hi - lo for lo, hi in shares)
        rc, hinted = _gemv_shape(spec.hidden, widest)
        assert rc == 0
        r_, c_, s_, g_, tiles, grid = hinted
        assert r_ in (1, 2, 4, 8) and c_ in (1, 2) and 1 <= s_ * g_ <= 15
        assert tiles == -(-spec.hidden // (g_ * r_)) and 1 <= grid <= 256
        assert s_ * c_ * 1024 >= widest          # the slices cover the longest share ...
        for lo, hi in shares:                    # ... hence every share
            assert hi - lo <= s_ * c_ * 1024 and (hi - lo) % 64 == 0
    rc, sw = _gemv_shape(spec.intermediate // world, 64 * -(-spec.hidden // 64), swiglu=True)
    assert rc == 0 and sw[0] * 2 * sw[1] <= 8    # gate + up row segments a warp holds per tile
    assert _gemv_shape(128, 64 * 600)[0] == -3   # K beyond what a CTA can stage (30080)
    assert _gemv_shape(0, 64)[0] == -3
