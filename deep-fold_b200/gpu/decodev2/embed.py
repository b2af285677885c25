"""NF4 embedding rows for the resident executor: no dense ``[vocab, hidden]`` table.

``PackedEmbed.gather`` decodes only the requested rows with one kernel
(``chr_nf4_embed_rows``); the reference does the same arithmetic with about ten
torch ops (gpu/decodev2/embed.py:15-50, gpu/host/embedding.py:74-107).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from gpu.nf4 import nf4_embed_rows
from gpu.nf4.plan import k_pad

from .arch import ArchSpec

__all__ = ["PackedEmbed", "bind_embed", "gather_embed"]


@dataclass
class PackedEmbed:
    packed: torch.Tensor
    scale: torch.Tensor
    vocab: int
    hidden: int

    @property
    def device(self) -> torch.device:
        return self.packed.device

    @property
    def shape(self) -> tuple[int, int]:
        return (self.vocab, self.hidden)

    @property
    def nbytes(self) -> int:
        return int(self.packed.numel()) + 2 * int(self.scale.numel())

    def gather(self, ids: torch.Tensor, *, dtype: torch.dtype = torch.bfloat16,
               out: torch.Tensor | None = None, status: torch.Tensor | None = None,
               position: torch.Tensor | None = None,
               valid_len: torch.Tensor | None = None) -> torch.Tensor:
        if dtype is not torch.bfloat16:
            raise TypeError("PackedEmbed decodes to bfloat16 only")
        ids = ids.reshape(-1).to(device=self.device, dtype=torch.int64)
        return nf4_embed_rows(
            self.packed, self.scale, ids, self.vocab, self.hidden, k_pad(self.hidden),
            out=out, status=status, position=position, valid_len=valid_len,
        )


def bind_embed(mod, spec: ArchSpec, dtype: torch.dtype) -> "torch.Tensor | PackedEmbed":
    """Alias a module's packed NF4 rows, or its dense weight when it has one."""
    packed = getattr(mod, "packed", None)
    scale = getattr(mod, "scale", None)
    if packed is not None and int(packed.numel()) > 0 and scale is not None:
        m = int(packed.shape[0])
        k = int(getattr(mod, "embedding_dim", getattr(mod, "K", spec.hidden)))
        if (m, k) != (spec.vocab, spec.hidden):
            raise ValueError(f"embed [{m},{k}] != spec [{spec.vocab},{spec.hidden}]")
        return PackedEmbed(packed=packed, scale=scale, vocab=spec.vocab, hidden=spec.hidden)
    weight = getattr(mod, "weight", None)
    if weight is None or int(weight.numel()) == 0:
        raise RuntimeError("embed has neither NF4 packed rows nor a dense weight")
    table = weight.to(dtype=dtype)
    if tuple(table.shape) != (spec.vocab, spec.hidden):
        raise ValueError(f"embed weight {tuple(table.shape)} != {(spec.vocab, spec.hidden)}")
    return table


def gather_embed(embed, ids: torch.Tensor, *, dtype: torch.dtype) -> torch.Tensor:
    """``[n, hidden]`` rows of a dense table or a ``PackedEmbed``."""
    if isinstance(embed, PackedEmbed):
        return embed.gather(ids, dtype=dtype)
    flat = ids.reshape(-1).to(device=embed.device, dtype=torch.long)
    return embed.index_select(0, flat).to(dtype=dtype)
