"""CHR0 container: byte-exact golden header, writer -> loader round trip, every
rejection the format specifies, and tensor-parallel shard materialisation."""

from __future__ import annotations

import json
import struct

import numpy as np
import pytest
import torch

import nf4_ref as o
from gpu.chr0 import (AlignmentError, Chr0Error, CodecError, GroupSizeError, HeaderError, OverlapError,
                      SizeMismatchError, TensorNotFoundError, TruncatedError, iter_linears, load_header,
                      materialize_bf16, materialize_nf4, quantized_codec)
from gpu.chr0.writer import Bf16Entry, Nf4Entry, plan_file, write_chr

# docs/spec/chr0.md §2.4: the byte-level header reference of the 3-tensor toy model (N = 516)
GOLDEN_JSON = (
    '{"magic":"CHR0","version":1,"arch":"toy","hidden_size":64,"intermediate_size":128,'
    '"num_layers":1,"vocab_size":0,"tile":{"row":64,"col_group":8},"tensors":'
    '{"model.layers.0.mlp.down_proj":{"layer":0,"kind":"down","codec":"nf4","shape":[32,128],'
    '"group_size":64,"data":[2752,4800],"scale":[4800,4928]},'
    '"model.layers.0.self_attn.q_proj":{"layer":0,"kind":"q","codec":"nf4","shape":[64,64],'
    '"group_size":64,"data":[576,2624],"scale":[2624,2752]},'
    '"model.norm":{"kind":"norm","codec":"bf16","shape":[64],"data":[4928,5056]}}}'
)
ROOT = dict(arch="toy", hidden_size=64, intermediate_size=128, num_layers=1, vocab_size=0)


def toy_entries(seed=0, zeros=False):
    out = []
    for name, kind, m, k in (("model.layers.0.self_attn.q_proj", "q", 64, 64),
                             ("model.layers.0.mlp.down_proj", "down", 32, 128)):
        if zeros:
            p = np.full((m, k // 2), 0x77, dtype=np.uint8)
            s = np.ones((m, k // 64), dtype=np.float16)
        else:
            p, s = o.random_blobs(m, k, seed + m)
        out.append(Nf4Entry(name, kind, p, s, k))
    out.append(Bf16Entry("model.norm", "norm", np.full(64, 0x3F80, dtype=np.uint16)))
    return out


def test_writer_emits_the_golden_header():
    js, plan, size = plan_file(toy_entries(zeros=True), **ROOT)
    assert len(js) == 516 and js.decode() == GOLDEN_JSON and size == 5056
    assert plan["model.layers.0.self_attn.q_proj"]["data"] == (576, 2624)


def test_round_trip_and_views(tmp_path):
    entries = toy_entries(seed=3)
    path = write_chr(str(tmp_path / "toy.chr"), entries, **ROOT)
    hdr = load_header(path)
    assert hdr.header_nbytes == 516 and hdr.payload_start == 576 and hdr.file_size == 5056
    assert list(iter_linears(hdr)) == ["model.layers.0.mlp.down_proj", "model.layers.0.self_attn.q_proj"]
    assert quantized_codec(hdr) == "nf4" and "model.norm" in hdr
    for e in entries[:2]:
        mat = materialize_nf4(path, e.name, "cpu", header=hdr)
        assert (mat.M, mat.K, mat.K_pad) == (e.packed.shape[0], e.K, e.K)
        assert np.array_equal(mat.packed.numpy(), e.packed)
        assert np.array_equal(mat.scale.numpy().view(np.uint16), e.scale.view(np.uint16))
        assert mat.packed.data_ptr() % 16 == 0 and mat.nbytes == e.packed.nbytes + e.scale.nbytes
        # packed and scale are views of one allocation
        assert mat.scale.untyped_storage().data_ptr() == mat.packed.untyped_storage().data_ptr()
    norm = materialize_bf16(path, "model.norm", "cpu", header=hdr)
    assert norm.dtype is torch.bfloat16 and float(norm.float().sum()) == 64.0
    with pytest.raises(TensorNotFoundError):
        materialize_nf4(path, "nope", "cpu", header=hdr)
    with pytest.raises(CodecError):
        materialize_nf4(path, "model.norm", "cpu", header=hdr)


def test_tensor_parallel_shards_are_slices_of_the_file(tmp_path):
    m, k = 96, 256
    p, s = o.random_blobs(m, k, 11)
    path = write_chr(str(tmp_path / "w.chr"), [Nf4Entry("model.layers.0.mlp.up_proj", "up", p, s, k)],
                     arch="toy", hidden_size=k, intermediate_size=m, num_layers=1, vocab_size=0)
    for world in (2, 3):
        rows = [materialize_nf4(path, "model.layers.0.mlp.up_proj", "cpu", rank=r, world=world, split="col")
                for r in range(world)]
        assert np.array_equal(np.concatenate([x.packed.numpy() for x in rows]), p)
        assert all(x.K == k and x.M == m // world for x in rows)
    for world in (2, 4):
        cols = [materialize_nf4(path, "model.layers.0.mlp.up_proj", "cpu", rank=r, world=world, split="row")
                for r in range(world)]
        assert np.array_equal(np.concatenate([x.packed.numpy() for x in cols], axis=1), p)
        assert np.array_equal(np.concatenate([x.scale.numpy().view(np.uint16) for x in cols], axis=1),
                              s.view(np.uint16))
        full = o.dequantize(p, s, m, k)
        parts = [o.dequantize(x.packed.numpy(), x.scale.numpy(), x.M, x.K) for x in cols]
        assert np.array_equal(np.concatenate(parts, axis=1), full)
    part = materialize_nf4(path, "model.layers.0.mlp.up_proj", "cpu", rows=(10, 20))
    assert np.array_equal(part.packed.numpy(), p[10:20])


def _rewrite(path, mutate):
    raw = open(path, "rb").read()
    (n,) = struct.unpack("<Q", raw[:8])
    root = json.loads(raw[8:8 + n])
    mutate(root)
    js = json.dumps(root, separators=(",", ":")).encode()
    start = (8 + n + 63) & ~63                  # blobs stay where they are
    assert 8 + len(js) <= start, "mutated header must still end before the first blob"
    open(path, "wb").write(struct.pack("<Q", len(js)) + js + b"\0" * (start - 8 - len(js)) + raw[start:])


Q = "model.layers.0.self_attn.q_proj"
CASES = [
    (lambda r: r["tensors"][Q].__setitem__("data", [568, 2616]), AlignmentError),
    (lambda r: r["tensors"][Q].__setitem__("scale", [576, 704]), OverlapError),
    (lambda r: r["tensors"][Q].__setitem__("group_size", 32), GroupSizeError),
    (lambda r: r["tensors"][Q].__setitem__("data", [576, 2688]), SizeMismatchError),
    (lambda r: r["tensors"][Q].__setitem__("data", [576, 570]), SizeMismatchError),
    (lambda r: r.__setitem__("magic", "CHR1"), HeaderError),
    (lambda r: r.__setitem__("version", 2), HeaderError),
    (lambda r: r["tile"].__setitem__("row", 32), HeaderError),
    (lambda r: r["tensors"][Q].__setitem__("codec", "zip"), CodecError),
    (lambda r: r["tensors"][Q].__setitem__("kind", "x"), HeaderError),
    (lambda r: r["tensors"][Q].__setitem__("layer", 1), HeaderError),
    (lambda r: r["tensors"][Q].pop("layer"), HeaderError),
    (lambda r: r["tensors"][Q].__setitem__("shape", [64]), HeaderError),
    (lambda r: r["tensors"]["model.norm"].__setitem__("layer", 0), HeaderError),
    (lambda r: r["tensors"][Q].__setitem__("codec", "bf16") or r["tensors"][Q].pop("scale")
     or r["tensors"][Q].pop("group_size"), Chr0Error),
    (lambda r: r.pop("arch"), HeaderError),
    (lambda r: r.__setitem__("tensors", {}), HeaderError),
]


@pytest.mark.parametrize("idx", range(len(CASES)))
def test_malformed_headers_are_refused(tmp_path, idx):
    mutate, err = CASES[idx]
    path = write_chr(str(tmp_path / "bad.chr"), toy_entries(zeros=True), **ROOT)
    _rewrite(path, mutate)
    with pytest.raises(err):
        load_header(path)


def test_raw_header_damage(tmp_path):
    good = write_chr(str(tmp_path / "g.chr"), toy_entries(zeros=True), **ROOT)
    raw = open(good, "rb").read()

    def variant(name, data):
        p = tmp_path / name
        p.write_bytes(data)
        return str(p)

    with pytest.raises(TruncatedError):
        load_header(variant("a", raw[:4]))
    with pytest.raises(TruncatedError):
        load_header(variant("b", raw[:300]))
    with pytest.raises(HeaderError):
        load_header(variant("c", struct.pack("<Q", 1) + raw[8:]))
    with pytest.raises(HeaderError):
        load_header(variant("d", struct.pack("<Q", 10**9) + raw[8:]))
    with pytest.raises(HeaderError):
        load_header(variant("e", raw[:8] + b" " + raw[9:]))
    with pytest.raises(HeaderError):   # a float in the header
        load_header(variant("f", raw[:8] + raw[8:524].replace(b'"intermediate_size":128', b'"intermediate_size":1e2') + raw[524:]))
    dup = raw[8:524].replace(b'"vocab_size":0', b'"version":1    ')
    with pytest.raises(HeaderError):   # duplicate key
        load_header(variant("g", raw[:8] + dup + raw[524:]))


def test_truncated_payload_fails_before_any_allocation(tmp_path, monkeypatch):
    path = write_chr(str(tmp_path / "t.chr"), toy_entries(seed=1), **ROOT)
    hdr = load_header(path)
    with open(path, "r+b") as f:
        f.truncate(hdr.file_size - 64 - 2048)

    def boom(*a, **k):
        raise AssertionError("device allocation attempted for a truncated file")

    monkeypatch.setattr(torch, "empty", boom)
    with pytest.raises(TruncatedError):
        load_header(path)                       # a fresh validation refuses it outright
    with pytest.raises(TruncatedError):         # a stale header still fails at the host read
        materialize_nf4(path, "model.layers.0.mlp.down_proj", "cpu", header=hdr)
