"""Map an NF4 tensor of a CHR0 file onto device memory: the bytes on disk are the
bytes in HBM, nothing is decoded here.

Copy strategy of the reference (gpu/chr0/loader.py:74-130, docs/spec/gpu-abi.md §4):
read host-side first (a short file fails before any device allocation), one
allocation per matrix, ``packed`` / ``scale`` are views of it. Additive:
``split="col"|"row"`` with ``rank`` / ``world`` materializes only this rank's
tensor-parallel shard - whole rows for a column split, K ranges cut at NF4 group
boundaries for a row split - reading just those byte ranges from the file.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .errors import CodecError, GroupSizeError, TruncatedError
from .header import NF4_GROUP_SIZE, Header, load_header

__all__ = ["ChrMatrix", "materialize_nf4", "materialize_bf16"]


@dataclass(frozen=True)
class ChrMatrix:
    """Python twin of ``chr_nf4_dev_t`` (field names and order frozen)."""

    name: str
    M: int
    K: int
    K_pad: int
    packed: torch.Tensor  # uint8   [M, K_pad // 2]
    scale: torch.Tensor   # float16 [M, K_pad // 64]

    @property
    def n_groups(self) -> int:
        return self.K_pad // NF4_GROUP_SIZE

    @property
    def device(self) -> torch.device:
        return self.packed.device

    @property
    def nbytes(self) -> int:
        return self.packed.numel() + self.scale.numel() * 2


def _pread(path: str, start: int, nbytes: int, what: str) -> bytearray:
    buf = bytearray(nbytes)
    with open(path, "rb") as f:
        f.seek(start)
        got = f.readinto(memoryview(buf))
    if got != nbytes:
        raise TruncatedError(f"truncated: {what} wanted {nbytes} bytes at {start}, got {got}")
    return buf


def _group_range(total: int, world: int, rank: int) -> tuple[int, int]:
    groups = total // NF4_GROUP_SIZE
    base, rem = divmod(groups, world)
    lo = rank * base + min(rank, rem)
    return lo * NF4_GROUP_SIZE, (lo + base + (1 if rank < rem else 0)) * NF4_GROUP_SIZE


def materialize_nf4(path: str, name: str, device: "str | torch.device" = "cuda", *,
                    header: Header | None = None, rank: int = 0, world: int = 1,
                    split: str | None = None, rows: tuple[int, int] | None = None) -> ChrMatrix:
    """Load the NF4 blobs of ``name`` (or this rank's shard of them) onto ``device``."""
    path = str(path)
    hdr = header if header is not None else load_header(path)
    info = hdr.tensor(name)
    if info.codec != "nf4":
        raise CodecError(f"{name}: codec {info.codec!r}; only nf4 is materialized")
    if info.group_size != NF4_GROUP_SIZE:
        raise GroupSizeError(f"{name}: group_size {info.group_size}, must be {NF4_GROUP_SIZE}")
    if split not in (None, "col", "row"):
        raise ValueError(f"split {split!r} not in col|row")
    m, k, kp, ng = info.M, info.K, info.K_pad, info.n_groups
    data, scale = info.blobs["data"], info.blobs["scale"]
    row_lo, row_hi, k_lo, k_hi = 0, m, 0, kp
    if rows is not None:
        row_lo, row_hi = int(rows[0]), int(rows[1])
        if not 0 <= row_lo < row_hi <= m:
            raise ValueError(f"rows {rows} outside 0..{m}")
    elif split == "col" and world > 1:
        if m % world:
            raise ValueError(f"{name}: M={m} does not divide by {world}")
        row_lo, row_hi = rank * (m // world), (rank + 1) * (m // world)
    elif split == "row" and world > 1:
        if k != kp:
            raise ValueError(f"{name}: a row split needs K to be a multiple of 64")
        k_lo, k_hi = _group_range(k, world, rank)

    # host reads first: nothing touches the device until every byte is in hand
    n_rows = row_hi - row_lo
    if k_lo == 0 and k_hi == kp:
        p_host = _pread(path, data.start + row_lo * (kp // 2), n_rows * (kp // 2), f"{name}.data")
        s_host = _pread(path, scale.start + row_lo * ng * 2, n_rows * ng * 2, f"{name}.scale")
        p_cpu = torch.frombuffer(p_host, dtype=torch.uint8)
        s_cpu = torch.frombuffer(s_host, dtype=torch.uint8)
    else:
        p_all = torch.frombuffer(_pread(path, data.start, data.nbytes, f"{name}.data"), dtype=torch.uint8)
        s_all = torch.frombuffer(_pread(path, scale.start, scale.nbytes, f"{name}.scale"), dtype=torch.uint8)
        p_cpu = p_all.view(m, kp // 2)[:, k_lo // 2:k_hi // 2].contiguous().view(-1)
        s_cpu = s_all.view(m, ng * 2)[:, k_lo // 32:k_hi // 32].contiguous().view(-1)
    dev = torch.device(device)
    if dev.type == "cuda" and not torch.cuda.is_available():
        raise RuntimeError("device='cuda' requested but torch.cuda.is_available() is False")
    # one allocation; the scale view starts on a 256-byte boundary inside it
    p_bytes = p_cpu.numel()
    s_off = (p_bytes + 255) & ~255
    arena = torch.empty(s_off + s_cpu.numel(), dtype=torch.uint8, device=dev)
    arena[:p_bytes].copy_(p_cpu)
    arena[s_off:].copy_(s_cpu)
    k_local = (k_hi - k_lo) if (k_lo, k_hi) != (0, kp) else k
    kp_local = k_hi - k_lo
    return ChrMatrix(
        name=name, M=n_rows, K=k_local, K_pad=kp_local,
        packed=arena[:p_bytes].view(n_rows, kp_local // 2),
        scale=arena[s_off:].view(torch.float16).view(n_rows, kp_local // NF4_GROUP_SIZE),
    )


def materialize_bf16(path: str, name: str, device: "str | torch.device" = "cuda", *,
                     header: Header | None = None) -> torch.Tensor:
    """A bf16 tensor (norm weight, bias) of the file as a device tensor of its shape."""
    path = str(path)
    hdr = header if header is not None else load_header(path)
    info = hdr.tensor(name)
    if info.codec != "bf16":
        raise CodecError(f"{name}: codec {info.codec!r}, expected bf16")
    blob = info.blobs["data"]
    host = torch.frombuffer(_pread(path, blob.start, blob.nbytes, f"{name}.data"), dtype=torch.bfloat16)
    return host.view(*info.shape).to(torch.device(device))
