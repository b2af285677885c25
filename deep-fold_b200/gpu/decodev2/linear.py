"""Device-resident NF4 weights and the ``[N, K] -> [N, M]`` linear.

Mirrors the reference's handles (gpu/decodev2/linear.py:47-235): ``DeviceLinear``
is the Python twin of ``chr_nf4_dev_t`` plus an optional bias, ``DeviceLayer`` /
``DeviceWeights`` group them per decoder layer, ``nf4_linear`` routes N == 1 to
the GEMV and N > 1 to the tensor-core GEMM in chunks of ``LIVE_MAX_N``.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from gpu.host.codec import encode_nf4, encode_nf4_device
from gpu.nf4 import LIVE_MAX_N, nf4_gemm, nf4_gemm_rows, nf4_gemv
from gpu.nf4.plan import k_pad

from .arch import ArchSpec
from .embed import PackedEmbed
from .synth import Nf4Matrix, SynthLayer, SynthModel

__all__ = [
    "DeviceLinear",
    "DeviceLayer",
    "DeviceWeights",
    "adjoin_rows",
    "linear_backend",
    "nf4_linear",
    "set_linear_backend",
    "set_rows_gemm",
]

_BACKEND = "gemv"
_ROWS_GEMM = True


def set_rows_gemm(on: bool) -> None:
    """``True`` (default): N > 1 linears take the wide row-layout GEMM in one call;
    ``False``: the reference's shape, ``[K, N]`` chunks of ``LIVE_MAX_N`` through ``nf4_gemm``."""
    global _ROWS_GEMM
    _ROWS_GEMM = bool(on)



def linear_backend() -> str:
    """``gemv``: N == 1 linears run the CUDA-core GEMV; ``mma``: the GEMM at N == 1."""
    return _BACKEND


def set_linear_backend(name: str) -> None:
    global _BACKEND
    key = str(name).strip().lower()
    if key not in {"mma", "gemv"}:
        raise ValueError(f"linear backend {name!r} not in mma|gemv")
    _BACKEND = key


@dataclass
class DeviceLinear:
    packed: torch.Tensor
    scale: torch.Tensor
    M: int
    K: int
    K_pad: int
    bias: torch.Tensor | None = None

    @classmethod
    def from_nf4(cls, mat: Nf4Matrix, device, dtype: torch.dtype = torch.bfloat16) -> "DeviceLinear":
        dev = torch.device(device)
        if dev.type != "cuda":
            raise RuntimeError("NF4 linears are CUDA-only (no CPU path)")
        bias = None
        if mat.bias is not None:
            bias = torch.from_numpy(np.ascontiguousarray(mat.bias)).to(device=dev, dtype=dtype)
        return cls(
            packed=torch.from_numpy(np.ascontiguousarray(mat.packed)).to(dev),
            scale=torch.from_numpy(np.ascontiguousarray(mat.scale)).to(dev),
            M=mat.M, K=mat.K, K_pad=mat.K_pad, bias=bias,
        )

    @classmethod
    def from_compressed(cls, lin) -> "DeviceLinear":
        """Alias a loaded seat (``packed``/``scale``/``M``/``K``/``K_pad``/``bias``); no copy."""
        if lin.packed is None or int(lin.packed.numel()) == 0:
            raise RuntimeError("seat has no packed weights")
        bias = getattr(lin, "bias", None)
        if bias is not None and int(bias.numel()) == 0:
            bias = None
        return cls(lin.packed, lin.scale, int(lin.M), int(lin.K), int(lin.K_pad), bias)

    @classmethod
    def random(cls, m: int, k: int, gen: torch.Generator, device, *, std: float = 0.02,
               bias: bool = False, dtype: torch.dtype = torch.bfloat16) -> "DeviceLinear":
        """``std * randn`` float32 weights drawn and quantized on the device."""
        w = torch.randn((m, k), generator=gen, device=device, dtype=torch.float32) * std
        packed, scale = encode_nf4_device(w)
        b = None
        if bias:
            b = (torch.randn((m,), generator=gen, device=device, dtype=torch.float32) * std).to(dtype)
        return cls(packed, scale, m, k, k_pad(k), b)

    @property
    def nbytes(self) -> int:
        return int(self.packed.numel()) + 2 * int(self.scale.numel())


def nf4_linear(mat: DeviceLinear, x: torch.Tensor, add: torch.Tensor | None = None) -> torch.Tensor:
    """``x`` ``[N, K]`` -> ``[N, M]`` bf16 on ``x.device`` (+ bias) (+ ``add`` ``[N, M]``). On the
    wide-GEMM path bias and ``add`` are folded into the epilogue (one rounding); elsewhere they
    are added as tensor ops."""
    if x.shape[-1] != mat.K:
        raise ValueError(f"x K={x.shape[-1]} != {mat.K}")
    if x.device.type != "cuda":
        raise RuntimeError("nf4_linear is CUDA-only (no CPU path)")
    rows = x.reshape(-1, mat.K)
    n = int(rows.size(0))
    if rows.dtype is not torch.bfloat16:
        rows = rows.to(torch.bfloat16)
    if n == 1 and _BACKEND == "gemv":
        y = nf4_gemv(mat.packed, mat.scale, rows.reshape(mat.K), mat.M, mat.K, mat.K_pad).view(1, mat.M)
    elif n == 1:
        y = nf4_gemm(mat.packed, mat.scale, rows.reshape(mat.K), mat.M, mat.K, mat.K_pad).view(1, mat.M)
    elif _ROWS_GEMM and mat.K % 8 == 0:
        fused_add = None
        if add is not None and add.dtype is torch.bfloat16:
            fused_add = add.reshape(n, mat.M).contiguous()
        y = nf4_gemm_rows(mat.packed, mat.scale, rows.contiguous(), mat.M, mat.K, mat.K_pad,
                          bias=mat.bias, add=fused_add)
        return y if add is None or fused_add is not None else y + add.reshape(n, mat.M).to(y.dtype)
    else:
        cols = []
        for lo in range(0, n, LIVE_MAX_N):
            xk = rows[lo: lo + LIVE_MAX_N].t().contiguous()
            cols.append(nf4_gemm(mat.packed, mat.scale, xk, mat.M, mat.K, mat.K_pad))
        y = (cols[0] if len(cols) == 1 else torch.cat(cols, dim=1)).t().contiguous()
    if mat.bias is not None:
        y = y + mat.bias.to(dtype=y.dtype)
    if add is not None:
        y = y + add.reshape(n, mat.M).to(dtype=y.dtype)
    return y


def adjoin_rows(mats: list[DeviceLinear]) -> DeviceLinear:
    """Re-home matrices that share K into one contiguous blob and return the matrix whose
    rows are theirs in order. The given handles become row views of the blob (no second
    copy stays alive), so the N = 1 path keeps addressing them one by one while a wide
    GEMM can take them all in a single pass over the activations."""
    k, kp = mats[0].K, mats[0].K_pad
    if any(m.K != k or m.K_pad != kp for m in mats):
        raise ValueError("matrices to adjoin must share K")
    packed = torch.cat([m.packed for m in mats], dim=0)
    scale = torch.cat([m.scale for m in mats], dim=0)
    bias = None
    if any(m.bias is not None for m in mats):
        ref = next(m.bias for m in mats if m.bias is not None)
        bias = torch.cat([m.bias if m.bias is not None else torch.zeros(m.M, dtype=ref.dtype,
                                                                        device=ref.device)
                          for m in mats])
    lo = 0
    for m in mats:
        m.packed, m.scale = packed[lo:lo + m.M], scale[lo:lo + m.M]
        lo += m.M
    return DeviceLinear(packed, scale, lo, k, kp, bias)


@dataclass
class DeviceLayer:
    norm1: torch.Tensor
    norm2: torch.Tensor
    q: DeviceLinear | None
    k: DeviceLinear | None
    v: DeviceLinear | None
    wqkv: DeviceLinear | None
    o: DeviceLinear
    gate: DeviceLinear
    up: DeviceLinear
    down: DeviceLinear
    qkv_rows: DeviceLinear | None = None   # q, k, v stacked (set by adjoin)
    gate_up: DeviceLinear | None = None    # gate, up stacked (set by adjoin)

    def adjoin(self) -> "DeviceLayer":
        """Stack q/k/v and gate/up in memory so that the prefill runs each group as one GEMM."""
        if self.q is not None and self.qkv_rows is None:
            self.qkv_rows = adjoin_rows([self.q, self.k, self.v])
        if self.gate_up is None:
            self.gate_up = adjoin_rows([self.gate, self.up])
        return self


@dataclass
class DeviceWeights:
    spec: ArchSpec
    embed: "torch.Tensor | PackedEmbed"
    final_norm: torch.Tensor
    lm_head: DeviceLinear
    layers: list[DeviceLayer]

    @classmethod
    def from_synth(cls, model: SynthModel, device, dtype: torch.dtype = torch.bfloat16, *,
                   packed_embed: bool = False) -> "DeviceWeights":
        device = torch.device(device)
        up = lambda m: None if m is None else DeviceLinear.from_nf4(m, device, dtype)
        vec = lambda a: torch.from_numpy(a.copy()).to(device=device, dtype=dtype)

        def layer(ly: SynthLayer) -> DeviceLayer:
            return DeviceLayer(vec(ly.norm1), vec(ly.norm2), up(ly.q), up(ly.k), up(ly.v),
                               up(ly.wqkv), up(ly.o), up(ly.gate), up(ly.up), up(ly.down))

        if packed_embed:
            p, s = encode_nf4(np.ascontiguousarray(model.embed, dtype=np.float32))
            embed = PackedEmbed(torch.from_numpy(p).to(device), torch.from_numpy(s).to(device),
                                model.spec.vocab, model.spec.hidden)
        else:
            embed = vec(model.embed)
        return cls(model.spec, embed, vec(model.final_norm), up(model.lm_head),
                   [layer(ly).adjoin() for ly in model.layers])

    @classmethod
    def random_init(cls, spec: ArchSpec, seed: int, device="cuda",
                    dtype: torch.dtype = torch.bfloat16) -> "DeviceWeights":
        """Checkpoint-shaped random model built on the device: every linear is
        ``0.02 * randn`` quantized to NF4, q/k/v carry a bias when the spec says so,
        norm weights are ones, the embedding is an NF4 table (shared with lm_head
        when tied). Matrix order of the draws: per layer q,k,v | wqkv, o, gate, up,
        down; then embed, lm_head."""
        device = torch.device(device)
        gen = torch.Generator(device=device)
        gen.manual_seed(int(seed))
        h, kv, inter = spec.hidden, spec.kv_dim, spec.intermediate
        ones = lambda n: torch.ones(n, dtype=dtype, device=device)
        rnd = lambda m, k, bias=False: DeviceLinear.random(m, k, gen, device, bias=bias, dtype=dtype)
        layers = []
        for _ in range(spec.n_layers):
            q = k = v = wqkv = None
            if spec.family == "llama_swiglu":
                q, k, v = (rnd(h, h, spec.qkv_bias), rnd(kv, h, spec.qkv_bias),
                           rnd(kv, h, spec.qkv_bias))
            else:
                wqkv = rnd(spec.wqkv_out, h)
            layers.append(DeviceLayer(ones(h), ones(h), q, k, v, wqkv, rnd(h, spec.q_dim),
                                      rnd(inter, h), rnd(inter, h), rnd(h, inter)).adjoin())
        table = rnd(spec.vocab, h)
        embed = PackedEmbed(table.packed, table.scale, spec.vocab, h)
        lm_head = table if spec.tied_embed else rnd(spec.vocab, h)
        return cls(spec, embed, ones(h), lm_head, layers)

    @property
    def nbytes(self) -> int:
        seen: dict[int, int] = {}
        mats = [self.lm_head]
        for ly in self.layers:
            mats += [m for m in (ly.q, ly.k, ly.v, ly.wqkv, ly.o, ly.gate, ly.up, ly.down) if m]
        for m in mats:
            seen[m.packed.data_ptr()] = m.nbytes
        if isinstance(self.embed, PackedEmbed):
            seen[self.embed.packed.data_ptr()] = self.embed.nbytes
        else:
            seen[self.embed.data_ptr()] = self.embed.numel() * self.embed.element_size()
        return sum(seen.values())
