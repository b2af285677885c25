"""CHR0 header: parse and validate everything before any payload byte is read.

Format (docs/spec/chr0.md §1-§2): ``u64 little-endian N``, then ``N`` bytes of
compact JSON, then blobs at 64-byte aligned offsets. Every rule the reference's
reader enforces (gpu/chr0/header.py:399-502 and its helpers) is enforced here, so
a malformed file is refused before a device allocation or copy can start.
"""

from __future__ import annotations

import json
import struct
from dataclasses import dataclass
from typing import Any, Iterator, Mapping

from .errors import (AlignmentError, CodecError, GroupSizeError, HeaderError, OverlapError,
                     SizeMismatchError, TensorNotFoundError, TruncatedError)

__all__ = ["Blob", "TensorInfo", "Header", "load_header", "parse_header", "iter_linears",
           "quantized_codec", "align64", "NF4_GROUP_SIZE"]

NF4_GROUP_SIZE = 64
VQ_GROUP_SIZE = 8
MAX_HEADER_NBYTES = 100_000_000
MAX_TENSORS = 1_000_000
MAX_AXIS = (1 << 24) - 1
MAX_NAME_BYTES = 1024

ROOT_KEYS = ("magic", "version", "arch", "hidden_size", "intermediate_size", "num_layers",
             "vocab_size", "tile", "tensors")
KINDS = {"q", "k", "v", "o", "qkv", "gate", "up", "down", "embed", "lm_head", "norm", "other"}
QUANTIZABLE = KINDS - {"norm", "other"}
BLOB_KEYS = ("data", "scale", "zero", "codebook", "index")
# codec -> (required, optional) keys beyond kind / codec / shape / layer
CODEC_KEYS = {
    "bf16": ({"data"}, set()),
    "nf4": ({"group_size", "data", "scale"}, set()),
    "int4": ({"group_size", "data", "scale"}, {"zero"}),
    "vq": ({"group_size", "n_codebooks", "codebook_bits", "codebook", "index"}, set()),
}


def align64(x: int) -> int:
    return (x + 63) & ~63


def _ceil_to(n: int, g: int) -> int:
    return -(-n // g) * g


@dataclass(frozen=True)
class Blob:
    start: int
    end: int

    @property
    def nbytes(self) -> int:
        return self.end - self.start


@dataclass(frozen=True)
class TensorInfo:
    name: str
    kind: str
    codec: str
    shape: tuple[int, ...]
    layer: int | None
    group_size: int | None
    n_codebooks: int | None
    codebook_bits: int | None
    blobs: Mapping[str, Blob]

    @property
    def M(self) -> int:  # noqa: N802
        return self.shape[0]

    @property
    def K(self) -> int:  # noqa: N802
        if len(self.shape) != 2:
            raise SizeMismatchError(f"{self.name}: rank {len(self.shape)} has no K")
        return self.shape[1]

    @property
    def K_pad(self) -> int:  # noqa: N802
        return _ceil_to(self.K, self.group_size or NF4_GROUP_SIZE)

    @property
    def n_groups(self) -> int:
        return self.K_pad // (self.group_size or NF4_GROUP_SIZE)


@dataclass(frozen=True)
class Header:
    path: str
    header_nbytes: int
    payload_start: int
    file_size: int
    magic: str
    version: int
    arch: str
    hidden_size: int
    intermediate_size: int
    num_layers: int
    vocab_size: int
    tile_row: int
    tile_col_group: int
    tensors: Mapping[str, TensorInfo]

    def tensor(self, name: str) -> TensorInfo:
        if name not in self.tensors:
            raise TensorNotFoundError(f"not_found: {name!r} not in {self.path}")
        return self.tensors[name]

    def __contains__(self, name: object) -> bool:
        return name in self.tensors


# ------------------------------------------------------------------ JSON strictness
def _no_float(lit: str):
    raise HeaderError(f"json_invalid: non-integer number {lit!r} in header")


def _no_const(lit: str):
    raise HeaderError(f"json_invalid: JSON constant {lit!r} in header")


def _unique(pairs):
    out: dict[str, Any] = {}
    for k, v in pairs:
        if k in out:
            raise HeaderError(f"json_invalid: duplicate key {k!r}")
        out[k] = v
    return out


def _int(v: Any, what: str) -> int:
    if isinstance(v, bool) or not isinstance(v, int):
        raise HeaderError(f"{what}: expected integer, got {type(v).__name__}")
    return v


def _str(v: Any, what: str) -> str:
    if not isinstance(v, str):
        raise HeaderError(f"{what}: expected string, got {type(v).__name__}")
    return v


# ------------------------------------------------------------------ per-tensor rules
def expected_blob_sizes(codec: str, shape: tuple[int, ...]) -> dict[str, int]:
    """Bytes each blob of a tensor must have (docs/spec/stitch-gpu.md size formulas)."""
    if codec == "bf16":
        n = 1
        for a in shape:
            n *= a
        return {"data": 2 * n}
    m, k = shape
    if codec in ("nf4", "int4"):
        kp = _ceil_to(k, NF4_GROUP_SIZE)
        sc = m * (kp // NF4_GROUP_SIZE) * 2
        return {"data": m * kp // 2, "scale": sc, "zero": sc}
    if codec == "vq":
        return {"codebook": 2 * 256 * 8 * 2, "index": m * (_ceil_to(k, VQ_GROUP_SIZE) // VQ_GROUP_SIZE) * 2}
    raise CodecError(f"unknown codec {codec!r}")


def _layer_in_name(name: str) -> int | None:
    parts = name.split(".")
    for a, b in zip(parts, parts[1:]):
        if a == "layers":
            return int(b) if b.isascii() and b.isdigit() else None
    return None


def _blob(name: str, key: str, value: Any, want: int, file_size: int) -> Blob:
    what = f"{name}.{key}"
    if not isinstance(value, list) or len(value) != 2:
        raise HeaderError(f"{what}: expected [start, end)")
    start, end = _int(value[0], what + ".start"), _int(value[1], what + ".end")
    if start < 0 or end > (1 << 63) - 1:
        raise HeaderError(f"{what}: offsets out of range")
    if end <= start:
        raise SizeMismatchError(f"{what}: end {end} <= start {start}")
    if start % 64:
        raise AlignmentError(f"{what}: start {start} is not 64-aligned")
    if end - start != want:
        raise SizeMismatchError(f"{what}: {end - start} bytes on disk, formula says {want}")
    if end > file_size:
        raise TruncatedError(f"truncated: {what} ends at {end}, file is {file_size} bytes")
    return Blob(start, end)


def _tensor(name: str, obj: Any, num_layers: int, file_size: int) -> TensorInfo:
    if not isinstance(obj, dict):
        raise HeaderError(f"{name}: tensor entry is not an object")
    raw = name.encode("utf-8")
    if not 1 <= len(raw) <= MAX_NAME_BYTES or any(c < 0x20 for c in raw):
        raise HeaderError(f"tensor name {name!r}: bad length or control byte")
    codec = _str(obj.get("codec"), f"{name}.codec")
    if codec not in CODEC_KEYS:
        raise CodecError(f"{name}: unknown codec {codec!r}")
    required, optional = CODEC_KEYS[codec]
    base = {"kind", "codec", "shape"}
    extra = set(obj) - (base | {"layer"} | required | optional)
    if extra:
        raise HeaderError(f"{name}: unexpected key(s) {sorted(extra)} for codec {codec}")
    missing = (base | required) - set(obj)
    if missing:
        raise HeaderError(f"{name}: missing key(s) {sorted(missing)} for codec {codec}")
    kind = _str(obj["kind"], f"{name}.kind")
    if kind not in KINDS:
        raise HeaderError(f"{name}: bad kind {kind!r}")
    if not isinstance(obj["shape"], list) or not 1 <= len(obj["shape"]) <= 2:
        raise HeaderError(f"{name}.shape: rank must be 1 or 2")
    shape = tuple(_int(a, f"{name}.shape") for a in obj["shape"])
    if any(not 1 <= a <= MAX_AXIS for a in shape):
        raise HeaderError(f"{name}.shape: axis out of range 1..{MAX_AXIS}")
    numel = shape[0] * (shape[1] if len(shape) == 2 else 1)
    if numel * 4 > 1 << 32:
        raise HeaderError(f"{name}.shape: {numel} elements exceeds the 4 GiB tensor limit")
    if codec != "bf16" and len(shape) != 2:
        raise HeaderError(f"{name}: codec {codec} requires rank 2, got {shape}")

    named_layer = _layer_in_name(name)
    layer = None
    if named_layer is None:
        if "layer" in obj:
            raise HeaderError(f"{name}: has 'layer' but no 'layers.<n>' segment")
    else:
        if "layer" not in obj:
            raise HeaderError(f"{name}: missing 'layer' for 'layers.{named_layer}'")
        layer = _int(obj["layer"], f"{name}.layer")
        if layer != named_layer:
            raise HeaderError(f"{name}: layer {layer} disagrees with name segment {named_layer}")
        if num_layers > 0 and not 0 <= layer < num_layers:
            raise HeaderError(f"{name}: layer {layer} outside 0..{num_layers - 1}")

    group = n_books = book_bits = None
    if "group_size" in obj:
        group = _int(obj["group_size"], f"{name}.group_size")
        want = VQ_GROUP_SIZE if codec == "vq" else NF4_GROUP_SIZE
        if group != want:
            raise GroupSizeError(f"{name}: group_size {group} for codec {codec}, must be {want}")
    if "n_codebooks" in obj:
        n_books = _int(obj["n_codebooks"], f"{name}.n_codebooks")
        if n_books != 2:
            raise HeaderError(f"{name}: n_codebooks must be 2, got {n_books}")
    if "codebook_bits" in obj:
        book_bits = _int(obj["codebook_bits"], f"{name}.codebook_bits")
        if book_bits != 8:
            raise HeaderError(f"{name}: codebook_bits must be 8, got {book_bits}")
    sizes = expected_blob_sizes(codec, shape)
    blobs = {k: _blob(name, k, obj[k], sizes[k], file_size) for k in BLOB_KEYS if k in obj}
    return TensorInfo(name, kind, codec, shape, layer, group, n_books, book_bits, blobs)


def _quantized_codecs(tensors: Mapping[str, TensorInfo]) -> set[str]:
    return {t.codec for t in tensors.values() if t.kind in QUANTIZABLE and not t.name.endswith(".bias")}


def parse_header(raw: bytes, *, path: str, header_nbytes: int, file_size: int) -> Header:
    """Validate the JSON bytes of a header against a file of ``file_size`` bytes."""
    if not raw or raw[0] != 0x7B:
        raise HeaderError("json_invalid: header does not start with '{' (BOM? padding?)")
    try:
        root = json.loads(raw.decode("utf-8"), parse_float=_no_float, parse_constant=_no_const,
                          object_pairs_hook=_unique)
    except UnicodeDecodeError as exc:
        raise HeaderError(f"json_invalid: header is not valid UTF-8 ({exc})") from None
    except json.JSONDecodeError as exc:
        raise HeaderError(f"json_invalid: {exc}") from None
    if not isinstance(root, dict):
        raise HeaderError("json_invalid: header root is not an object")
    if set(root) != set(ROOT_KEYS):
        raise HeaderError(f"header root keys: missing={sorted(set(ROOT_KEYS) - set(root))} "
                          f"unexpected={sorted(set(root) - set(ROOT_KEYS))}")
    if _str(root["magic"], "magic") != "CHR0":
        raise HeaderError(f"magic: expected 'CHR0', got {root['magic']!r}")
    if _int(root["version"], "version") != 1:
        raise HeaderError(f"unsupported version: {root['version']}")
    arch = _str(root["arch"], "arch")
    if not arch:
        raise HeaderError("arch: must be non-empty")
    hidden, inter, layers, vocab = (_int(root[k], k) for k in
                                    ("hidden_size", "intermediate_size", "num_layers", "vocab_size"))
    if hidden < 1 or min(inter, layers, vocab) < 0:
        raise HeaderError("header root: negative or zero size field")
    tile = root["tile"]
    if not isinstance(tile, dict) or set(tile) != {"row", "col_group"}:
        raise HeaderError("tile: expected exactly {'row', 'col_group'}")
    row, col = _int(tile["row"], "tile.row"), _int(tile["col_group"], "tile.col_group")
    if (row, col) != (64, 8):
        raise HeaderError(f"tile: expected row=64 col_group=8, got {row}/{col}")
    entries = root["tensors"]
    if not isinstance(entries, dict) or not entries:
        raise HeaderError("no tensors: 'tensors' must be a non-empty object")
    if len(entries) > MAX_TENSORS:
        raise HeaderError(f"too many tensors: {len(entries)}")
    tensors = {n: _tensor(n, o, layers, file_size) for n, o in entries.items()}

    spans = sorted((b.start, b.end, f"{t.name}.{k}") for t in tensors.values() for k, b in t.blobs.items())
    for (s0, e0, n0), (s1, e1, n1) in zip(spans, spans[1:]):
        if s1 < e0:
            raise OverlapError(f"overlap: {n0} [{s0},{e0}) and {n1} [{s1},{e1})")
    codecs = _quantized_codecs(tensors)
    if len(codecs) > 1:
        raise CodecError(f"mixed codecs in one file: {sorted(codecs)}")
    if codecs and codecs <= {"bf16"}:
        raise CodecError("quantizable tensors carry codec bf16; expected nf4/vq/int4")
    return Header(path, header_nbytes, align64(8 + header_nbytes), file_size, "CHR0", 1, arch, hidden,
                  inter, layers, vocab, row, col, tensors)


def load_header(path: str) -> Header:
    """Open ``path`` read-only, read ``8 + N`` bytes, close it, validate everything."""
    path = str(path)
    with open(path, "rb") as f:
        f.seek(0, 2)
        size = f.tell()
        if size < 8:
            raise TruncatedError(f"truncated: {path} is {size} bytes, need at least 8")
        f.seek(0)
        (n,) = struct.unpack("<Q", f.read(8))
        if n < 2:
            raise HeaderError(f"header_nbytes: {n} cannot hold a JSON object")
        if n > MAX_HEADER_NBYTES:
            raise HeaderError(f"header_too_large: header_nbytes={n}")
        if 8 + n > size:
            raise TruncatedError(f"truncated: header_nbytes={n} runs past EOF at {size}")
        raw = f.read(n)
    if len(raw) != n:
        raise TruncatedError(f"truncated: short read of header at {path}")
    return parse_header(raw, path=path, header_nbytes=n, file_size=size)


def quantized_codec(header: Header) -> str:
    """The one packed codec of the file (``nf4`` / ``vq`` / ``int4``)."""
    codecs = _quantized_codecs(header.tensors)
    if len(codecs) != 1:
        raise CodecError(f"expected one quantized codec, got {sorted(codecs) or 'none'}")
    return next(iter(codecs))


def iter_linears(header: Header) -> Iterator[str]:
    """Names whose codec is ``nf4``, in header key order (embed and lm_head included)."""
    return (n for n, t in header.tensors.items() if t.codec == "nf4")
