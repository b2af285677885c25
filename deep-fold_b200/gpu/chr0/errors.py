"""Rejections of a ``.chr`` file, one class per failure mode so callers and tests can
be specific (same taxonomy as the reference loader, gpu/chr0/errors.py:22-55)."""

from __future__ import annotations


class Chr0Error(Exception):
    """Any rejection of a ``.chr`` file."""


class TruncatedError(Chr0Error):
    """The file ends before the header or a blob range does."""


class HeaderError(Chr0Error):
    """``header_nbytes`` or the JSON header breaks the format."""


class AlignmentError(Chr0Error):
    """A blob does not start on a 64-byte boundary."""


class SizeMismatchError(Chr0Error):
    """A blob's length disagrees with its codec's size formula."""


class OverlapError(Chr0Error):
    """Two blob ranges intersect."""


class CodecError(Chr0Error):
    """Unknown codec, wrong keys for a codec, or mixed codecs in one file."""


class GroupSizeError(Chr0Error):
    """``group_size`` is not the codec's canonical value."""


class TensorNotFoundError(Chr0Error):
    """The requested name is not in ``tensors``."""


__all__ = [n for n, v in list(globals().items()) if isinstance(v, type) and issubclass(v, Exception)]
