"""``CompressedLinear``: an ``nn.Linear`` seat whose weight lives as CHR0 NF4 bytes.

Same role and surface as the reference seat (gpu/host/linear.py:31-227): the module
holds the file's bytes (``packed``, ``scale``) and no ``[out, in]`` parameter, and
activations shaped ``[..., K]`` go to the kernel and come back ``[..., M]``. Here no
transposes are needed: the wide tensor-core GEMM takes activation rows as they are.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from gpu.nf4 import LIVE_MAX_N, nf4_gemm, nf4_gemm_rows
from gpu.nf4.plan import k_pad

__all__ = ["CompressedLinear", "nf4_linear", "k_pad"]


def nf4_linear(x: torch.Tensor, packed: torch.Tensor, scale: torch.Tensor, M: int, K: int,  # noqa: N803
               K_pad: int, bias: torch.Tensor | None = None) -> torch.Tensor:  # noqa: N803
    """``y = x @ dequant_nf4(packed, scale).T`` for activations shaped ``[..., K]``."""
    if x.shape[-1] != K:
        raise ValueError(f"x has {x.shape[-1]} features, this linear takes K={K}")
    lead = tuple(x.shape[:-1])
    n = 1
    for d in lead:
        n *= int(d)
    if n < 1:
        raise ValueError(f"CompressedLinear: empty leading dims x{tuple(x.shape)}")
    if x.dtype is not torch.bfloat16:
        x = x.to(torch.bfloat16)
    rows = x.contiguous().view(n, K)
    if K % 8 == 0:
        out = nf4_gemm_rows(packed, scale, rows, M, K, K_pad)
    else:  # TMA needs a 16-byte activation row pitch; odd K goes through [K, N] chunks
        cols = [nf4_gemm(packed, scale, rows[lo:lo + LIVE_MAX_N].t().contiguous(), M, K, K_pad)
                for lo in range(0, n, LIVE_MAX_N)]
        out = torch.cat(cols, dim=1).t().contiguous()
    if bias is not None:
        out = out + bias
    return out.view(*lead, M)


class CompressedLinear(nn.Module):
    """Drop-in for ``nn.Linear``; buffers are empty until :meth:`attach` gets a ``ChrMatrix``."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, *,
                 device=None, dtype: torch.dtype = torch.bfloat16) -> None:
        super().__init__()
        self.in_features, self.out_features = int(in_features), int(out_features)
        self.compute_dtype = dtype
        dev = torch.device(device) if device is not None else torch.device("cpu")
        self.register_buffer("packed", torch.empty(0, dtype=torch.uint8, device=dev), persistent=False)
        self.register_buffer("scale", torch.empty(0, dtype=torch.float16, device=dev), persistent=False)
        self.register_buffer("bias", torch.zeros(out_features, dtype=dtype, device=dev) if bias
                             else torch.empty(0, dtype=dtype, device=dev), persistent=False)
        self.has_bias = bool(bias)
        self.chr_name: str | None = None

    M = property(lambda self: self.out_features)
    K = property(lambda self: self.in_features)
    K_pad = property(lambda self: k_pad(self.in_features))

    @property
    def weight(self) -> torch.Tensor:
        """0-numel stand-in: the dense matrix never exists."""
        return torch.empty(0, dtype=self.compute_dtype, device=self.packed.device)

    @property
    def is_loaded(self) -> bool:
        return self.packed.numel() > 0

    @property
    def nbytes(self) -> int:
        return self.packed.numel() + self.scale.numel() * 2

    def attach(self, matrix, bias: torch.Tensor | None = None) -> None:
        if (int(matrix.M), int(matrix.K)) != (self.out_features, self.in_features):
            raise ValueError(f"{matrix.name}: matrix is [{matrix.M},{matrix.K}], seat is "
                             f"[{self.out_features},{self.in_features}]")
        self.packed, self.scale, self.chr_name = matrix.packed, matrix.scale, matrix.name
        if bias is not None:
            if not self.has_bias or bias.numel() != self.out_features:
                raise ValueError("bias does not fit this seat")
            self.bias = bias.to(device=self.packed.device, dtype=self.compute_dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.is_loaded:
            raise RuntimeError("CompressedLinear has no weights: attach a ChrMatrix first")
        return nf4_linear(x, self.packed, self.scale, self.M, self.K, self.K_pad,
                          self.bias if self.has_bias else None)

    def extra_repr(self) -> str:
        return f"{self.in_features}, {self.out_features}, codec=nf4-g64, loaded={self.is_loaded}"
