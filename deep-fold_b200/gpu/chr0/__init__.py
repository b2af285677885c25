"""Read-only CHR0 loader (``.chr`` on disk -> NF4 tensors on a CUDA device) plus a
minimal writer for synthetic models. Public names follow the reference package
(gpu/chr0/__init__.py:43-63)."""

from __future__ import annotations

from .errors import (AlignmentError, Chr0Error, CodecError, GroupSizeError, HeaderError,
                     OverlapError, SizeMismatchError, TensorNotFoundError, TruncatedError)
from .header import (NF4_GROUP_SIZE, Blob, Header, TensorInfo, align64, iter_linears, load_header,
                     quantized_codec)

__all__ = [
    "load_header", "iter_linears", "quantized_codec", "materialize_nf4", "materialize_bf16",
    "ChrMatrix", "Header", "TensorInfo", "Blob", "align64", "NF4_GROUP_SIZE", "Chr0Error",
    "TruncatedError", "HeaderError", "AlignmentError", "SizeMismatchError", "OverlapError",
    "CodecError", "GroupSizeError", "TensorNotFoundError",
]


def __getattr__(name: str):
    # torch is only needed to materialize; parsing a header must not pay for it
    if name in ("materialize_nf4", "materialize_bf16", "ChrMatrix"):
        from . import loader

        return getattr(loader, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
