"""NF4 embedding seat: rows are decoded on the fly by ``chr_nf4_embed_rows``; the dense
``[vocab, hidden]`` table is never materialised (reference: gpu/host/embedding.py:74-205)."""

from __future__ import annotations

import torch
import torch.nn as nn

from gpu.nf4 import nf4_embed_rows
from gpu.nf4.plan import GROUP_SIZE

__all__ = ["dequant_nf4_rows", "Nf4Embedding"]


def dequant_nf4_rows(packed: torch.Tensor, scale: torch.Tensor, ids: torch.Tensor, K: int, *,  # noqa: N803
                     lut: torch.Tensor | None = None, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Rows ``ids`` of an NF4 matrix as ``[len(ids), K]``: ``bf16(f32(LUT) * f32(scale))``.

    ``lut`` is accepted for signature compatibility; the codebook is built into the kernel."""
    del lut
    if packed.dim() != 2 or packed.dtype is not torch.uint8:
        raise TypeError(f"packed must be uint8 [M, K_pad/2], got {packed.dtype} {tuple(packed.shape)}")
    if scale.dtype is not torch.float16:
        raise TypeError(f"scale must be float16, got {scale.dtype}")
    kp = packed.shape[1] * 2
    if scale.shape[1] != kp // GROUP_SIZE:
        raise ValueError(f"scale has {scale.shape[1]} groups, packed implies {kp // GROUP_SIZE}")
    flat = ids.reshape(-1).to(device=packed.device, dtype=torch.int64)
    rows = nf4_embed_rows(packed, scale, flat, int(packed.shape[0]), int(K), kp)
    return rows if dtype is torch.bfloat16 else rows.to(dtype)


class Nf4Embedding(nn.Module):
    """``nn.Embedding`` whose table stays packed (shared with a tied ``lm_head``)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, *, padding_idx: int | None = None,
                 dtype: torch.dtype = torch.bfloat16, device=None) -> None:
        super().__init__()
        self.num_embeddings, self.embedding_dim = int(num_embeddings), int(embedding_dim)
        self.padding_idx = padding_idx
        self.compute_dtype = dtype
        dev = torch.device(device) if device is not None else torch.device("cpu")
        self.register_buffer("packed", torch.empty(0, dtype=torch.uint8, device=dev), persistent=False)
        self.register_buffer("scale", torch.empty(0, dtype=torch.float16, device=dev), persistent=False)
        self.chr_name: str | None = None

    @property
    def weight(self) -> torch.Tensor:
        return torch.empty(0, dtype=self.compute_dtype, device=self.packed.device)

    @property
    def is_loaded(self) -> bool:
        return self.packed.numel() > 0

    def attach(self, matrix) -> None:
        if (int(matrix.M), int(matrix.K)) != (self.num_embeddings, self.embedding_dim):
            raise ValueError(f"{matrix.name}: matrix is [{matrix.M},{matrix.K}], embedding is "
                             f"[{self.num_embeddings},{self.embedding_dim}]")
        self.packed, self.scale, self.chr_name = matrix.packed, matrix.scale, matrix.name

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        if not self.is_loaded:
            raise RuntimeError("Nf4Embedding has no weights: attach a ChrMatrix first")
        rows = dequant_nf4_rows(self.packed, self.scale, input_ids, self.embedding_dim,
                                dtype=self.compute_dtype)
        return rows.view(*input_ids.shape, self.embedding_dim)
