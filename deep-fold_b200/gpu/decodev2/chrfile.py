"""A decoder's weights as one CHR0 file, and back: whole, or one tensor-parallel rank's share.

The reference reaches its executor from a ``.chr`` file through its HF model glue
(gpu/host/model.py, attach.py), which needs real checkpoints. This module is the
part of that route the hot path owns: the tensor names of a decoder in the
container, a writer for synthetic models, and a loader that builds
``DeviceWeights`` straight from the file's bytes - every NF4 matrix is one ``pread``
of exactly the rows (or the K range) the rank keeps and one copy to the device,
nothing is re-quantized, and a rank never reads another rank's bytes of a
column-split matrix (container: docs/spec/chr0.md; sharding rules: ``tp.py``).
"""

from __future__ import annotations

import numpy as np
import torch

from gpu.chr0.header import load_header
from gpu.chr0.loader import materialize_bf16, materialize_nf4
from gpu.chr0.writer import Bf16Entry, Nf4Entry, write_chr
from gpu.host.codec import encode_nf4

from .arch import ArchSpec, group_range, shard_spec
from .embed import PackedEmbed
from .linear import DeviceLayer, DeviceLinear, DeviceWeights
from .synth import Nf4Matrix, SynthModel
from .tp import kv_head_rows

__all__ = ["tensor_names", "save_synth", "load_weights"]


def tensor_names(spec: ArchSpec, layer: int) -> dict[str, str]:
    """Names of one layer's tensors (weights; a bias is the same name with ``.bias``)."""
    p = f"model.layers.{layer}"
    names = {
        "norm1": f"{p}.input_layernorm.weight", "norm2": f"{p}.post_attention_layernorm.weight",
        "gate": f"{p}.mlp.gate_proj.weight", "up": f"{p}.mlp.up_proj.weight",
        "down": f"{p}.mlp.down_proj.weight",
    }
    if spec.family == "internlm_gqa":
        names.update(wqkv=f"{p}.attention.wqkv.weight", o=f"{p}.attention.wo.weight")
    else:
        names.update(q=f"{p}.self_attn.q_proj.weight", k=f"{p}.self_attn.k_proj.weight",
                     v=f"{p}.self_attn.v_proj.weight", o=f"{p}.self_attn.o_proj.weight")
    return names


EMBED, FINAL_NORM, LM_HEAD = "model.embed_tokens.weight", "model.norm.weight", "lm_head.weight"


def _bf16_bits(a: np.ndarray) -> np.ndarray:
    t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16)
    return t.view(torch.int16).numpy().view(np.uint16)


def _bias_name(weight_name: str) -> str:
    return weight_name[: -len(".weight")] + ".bias"


def save_synth(model: SynthModel, path: str) -> str:
    """Write a synthetic model as a CHR0 file (NF4 linears and embedding rows, bf16 norms / biases)."""
    spec = model.spec
    # a file carries one codec for all quantizable tensors, the embedding among them: its
    # rows are NF4 too (decoded one row at a time by the executor, never as a dense table)
    e_packed, e_scale = encode_nf4(np.ascontiguousarray(model.embed, dtype=np.float32))
    entries: list = [Nf4Entry(EMBED, "embed", e_packed, e_scale.view(np.float16)
                              if e_scale.dtype != np.float16 else e_scale, spec.hidden)]

    def add(name: str, kind: str, mat: Nf4Matrix | None) -> None:
        if mat is None:
            return
        entries.append(Nf4Entry(name, kind, mat.packed, mat.scale.view(np.float16)
                                if mat.scale.dtype != np.float16 else mat.scale, mat.K))
        if mat.bias is not None:
            entries.append(Bf16Entry(_bias_name(name), "other", _bf16_bits(mat.bias)))

    for li, ly in enumerate(model.layers):
        n = tensor_names(spec, li)
        entries.append(Bf16Entry(n["norm1"], "norm", _bf16_bits(ly.norm1)))
        entries.append(Bf16Entry(n["norm2"], "norm", _bf16_bits(ly.norm2)))
        if ly.wqkv is not None:
            add(n["wqkv"], "qkv", ly.wqkv)
        else:
            add(n["q"], "q", ly.q)
            add(n["k"], "k", ly.k)
            add(n["v"], "v", ly.v)
        add(n["o"], "o", ly.o)
        add(n["gate"], "gate", ly.gate)
        add(n["up"], "up", ly.up)
        add(n["down"], "down", ly.down)
    entries.append(Bf16Entry(FINAL_NORM, "norm", _bf16_bits(model.final_norm)))
    add(LM_HEAD, "lm_head", model.lm_head)
    return write_chr(path, entries, arch=spec.name, hidden_size=spec.hidden,
                     intermediate_size=spec.intermediate, num_layers=spec.n_layers,
                     vocab_size=spec.vocab)


def load_weights(path: str, spec: ArchSpec, device="cuda", *, rank: int = 0,
                 world: int = 1, dtype: torch.dtype = torch.bfloat16) -> DeviceWeights:
    """``DeviceWeights`` of ``spec`` from a CHR0 file; with ``world > 1`` only this rank's
    shard is read: column splits by row range, row splits by K range at NF4 group
    boundaries, exactly the bytes ``shard_weights`` would keep of the full model."""
    hdr = load_header(path)
    if (hdr.hidden_size, hdr.num_layers, hdr.vocab_size) != (spec.hidden, spec.n_layers, spec.vocab):
        raise ValueError(f"{path}: header describes hidden={hdr.hidden_size} layers={hdr.num_layers} "
                         f"vocab={hdr.vocab_size}, spec {spec.name} differs")
    dev = torch.device(device)
    local = shard_spec(spec, world, rank) if world > 1 else spec

    def vec(name: str, rows: tuple[int, int] | None = None) -> torch.Tensor | None:
        if name not in hdr:
            return None
        t = materialize_bf16(path, name, dev, header=hdr).to(dtype)
        return t if rows is None else t[rows[0]:rows[1]].contiguous()

    def lin(name: str, *, split: str | None = None, rows: tuple[int, int] | None = None,
            bias_rows: tuple[int, int] | None = None, bias: bool = True) -> DeviceLinear:
        m = materialize_nf4(path, name, dev, header=hdr, rank=rank, world=world, split=split,
                            rows=rows)
        b = vec(_bias_name(name), bias_rows) if bias else None
        return DeviceLinear(m.packed, m.scale, m.M, m.K, m.K_pad, b)

    def col(name: str) -> DeviceLinear:
        """Rows ``rank * M / world ...`` of a matrix, bias sliced alike."""
        if world == 1:
            return lin(name)
        m_full = hdr.tensor(name).M
        step = m_full // world
        return lin(name, split="col", bias_rows=(rank * step, (rank + 1) * step))

    mlp = group_range(spec.intermediate, world, rank) if world > 1 else None
    layers = []
    for li in range(spec.n_layers):
        n = tensor_names(spec, li)
        q = k = v = wqkv = None
        if spec.family == "internlm_gqa":
            if world == 1:
                wqkv = lin(n["wqkv"])
            else:
                if spec.n_kv % world:
                    raise ValueError("fused wqkv needs n_kv divisible by the tensor-parallel degree")
                group = (spec.n_rep + 2) * spec.head_dim
                per = spec.n_kv // world
                r = (rank * per * group, (rank + 1) * per * group)
                wqkv = lin(n["wqkv"], rows=r, bias_rows=r)
        else:
            q = col(n["q"])
            if world == 1:
                k, v = lin(n["k"]), lin(n["v"])
            else:
                r = kv_head_rows(spec, rank, world)
                k, v = lin(n["k"], rows=r, bias_rows=r), lin(n["v"], rows=r, bias_rows=r)
        o = lin(n["o"], split="row" if world > 1 else None, bias=rank == 0)
        gate = lin(n["gate"], rows=mlp, bias_rows=mlp)
        up = lin(n["up"], rows=mlp, bias_rows=mlp)
        down = lin(n["down"], split="row" if world > 1 else None, bias=rank == 0)
        layer = DeviceLayer(vec(n["norm1"]), vec(n["norm2"]), q, k, v, wqkv, o, gate, up, down)
        layers.append(layer.adjoin() if world == 1 and dev.type == "cuda" else layer)
    if EMBED not in hdr:
        raise ValueError(f"{path}: no {EMBED}")
    table = materialize_nf4(path, EMBED, dev, header=hdr)  # replicated on every rank
    embed = PackedEmbed(table.packed, table.scale, spec.vocab, spec.hidden)
    return DeviceWeights(local, embed, vec(FINAL_NORM), col(LM_HEAD), layers)
