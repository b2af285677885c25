"""Minimal CHR0 writer: enough to put a synthetic NF4 model into a real ``.chr`` so
the loader is exercised end to end (the reference's writer is an offline Go tool,
internal/chr0/write.go:19-137; its header stabilisation rule, :191-237 and
docs/spec/chr0.md §3.3, is followed: blob offsets depend on the header length, so
the header is re-emitted until its length stops changing).
"""

from __future__ import annotations

import json
import struct
from dataclasses import dataclass

import numpy as np

from .header import align64

__all__ = ["Nf4Entry", "Bf16Entry", "plan_file", "write_chr"]

_ROOT_ORDER = ("magic", "version", "arch", "hidden_size", "intermediate_size", "num_layers",
               "vocab_size", "tile", "tensors")
_TENSOR_ORDER = ("layer", "kind", "codec", "shape", "group_size", "data", "scale")


@dataclass
class Nf4Entry:
    name: str
    kind: str
    packed: np.ndarray   # uint8 [M, K_pad/2]
    scale: np.ndarray    # float16 [M, K_pad/64]
    K: int               # logical in_features


@dataclass
class Bf16Entry:
    name: str
    kind: str
    bits: np.ndarray     # uint16 bf16 bit patterns, any shape of rank 1 or 2


def _layer(name: str):
    parts = name.split(".")
    for a, b in zip(parts, parts[1:]):
        if a == "layers" and b.isdigit():
            return int(b)
    return None


def _payloads(e) -> dict[str, bytes]:
    if isinstance(e, Nf4Entry):
        return {"data": np.ascontiguousarray(e.packed).tobytes(),
                "scale": np.ascontiguousarray(e.scale).astype("<f2").tobytes()}
    return {"data": np.ascontiguousarray(e.bits).astype("<u2").tobytes()}


def plan_file(entries, *, arch: str, hidden_size: int, intermediate_size: int, num_layers: int,
              vocab_size: int) -> tuple[bytes, dict[str, dict[str, tuple[int, int]]], int]:
    """(header JSON bytes, blob offsets, file size). Blobs follow ``entries`` order,
    tensors are listed sorted by UTF-8 name, JSON is compact."""
    entries = list(entries)
    payloads = {e.name: _payloads(e) for e in entries}
    n = 0
    for _ in range(16):
        pos = align64(8 + n)
        plan: dict[str, dict[str, tuple[int, int]]] = {}
        for e in entries:
            plan[e.name] = {}
            for key, raw in payloads[e.name].items():
                plan[e.name][key] = (pos, pos + len(raw))
                pos = align64(pos + len(raw))
        objs = {}
        for e in entries:
            obj = {"kind": e.kind}
            if _layer(e.name) is not None:
                obj["layer"] = _layer(e.name)
            if isinstance(e, Nf4Entry):
                obj.update(codec="nf4", shape=[int(e.packed.shape[0]), int(e.K)], group_size=64,
                           data=list(plan[e.name]["data"]), scale=list(plan[e.name]["scale"]))
            else:
                obj.update(codec="bf16", shape=[int(a) for a in e.bits.shape],
                           data=list(plan[e.name]["data"]))
            objs[e.name] = {k: obj[k] for k in _TENSOR_ORDER if k in obj}
        root = {"magic": "CHR0", "version": 1, "arch": arch, "hidden_size": hidden_size,
                "intermediate_size": intermediate_size, "num_layers": num_layers,
                "vocab_size": vocab_size, "tile": {"row": 64, "col_group": 8},
                "tensors": {k: objs[k] for k in sorted(objs, key=lambda s: s.encode("utf-8"))}}
        js = json.dumps({k: root[k] for k in _ROOT_ORDER}, separators=(",", ":"),
                        ensure_ascii=False).encode("utf-8")
        if len(js) == n:
            return js, plan, pos
        n = len(js)
    raise RuntimeError("header_not_stable")


def write_chr(path: str, entries, **root) -> str:
    entries = list(entries)
    js, plan, size = plan_file(entries, **root)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(js)))
        f.write(js)
        for e in entries:
            for key, raw in _payloads(e).items():
                f.seek(plan[e.name][key][0])
                f.write(raw)
        f.truncate(size)
    return str(path)
