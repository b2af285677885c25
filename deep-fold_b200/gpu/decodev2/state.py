"""Device-resident decode registers, static KV cache and activation arena.

Keeps the reference's three classes and their fields (gpu/decodev2/state.py:19-107,
kv.py:14-120, arena.py:17-59): position / valid_len / token live in device
scalars so one captured step replays for every token; the KV cache is
``[layers, max_seq, n_kv, head_dim]`` bf16 with a device ``valid_len`` hiding the
dirty tail; nothing on the step path allocates.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .arch import ArchSpec
from .embed import PackedEmbed
from .rope import rope_tables_torch

__all__ = ["Arena", "DecodeState", "GraphSafeKV"]

ATTN_SPLIT = 32


class GraphSafeKV:
    __slots__ = ("k", "v", "valid_len", "n_layers", "max_seq", "n_kv", "head_dim")

    def __init__(self, spec: ArchSpec, *, device, dtype: torch.dtype = torch.bfloat16,
                 valid_len: torch.Tensor | None = None) -> None:
        self.n_layers, self.max_seq = spec.n_layers, spec.max_seq
        self.n_kv, self.head_dim = spec.n_kv, spec.head_dim
        shape = (spec.n_layers, spec.max_seq, spec.n_kv, spec.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        if valid_len is None:
            valid_len = torch.zeros((), dtype=torch.int32, device=device)
        elif valid_len.device != self.k.device:
            raise ValueError("valid_len must live on the KV device")
        self.valid_len = valid_len.view(())

    @property
    def device(self) -> torch.device:
        return self.k.device

    @property
    def dtype(self) -> torch.dtype:
        return self.k.dtype

    @property
    def nbytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()

    def view(self, layer: int, seq: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Prefill window ``[1, n_kv, seq, hd]`` (eager only; a Python-int slice)."""
        seq = int(seq)
        if not 0 <= seq <= self.max_seq:
            raise ValueError(f"KV view seq={seq} not in 0..{self.max_seq}")
        k = self.k[layer, :seq].permute(1, 0, 2).unsqueeze(0)
        v = self.v[layer, :seq].permute(1, 0, 2).unsqueeze(0)
        return k, v

    def write(self, layer: int, position: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
        idx = position.reshape(1).to(dtype=torch.long)
        self.k[layer].index_copy_(0, idx, k.reshape(1, self.n_kv, self.head_dim))
        self.v[layer].index_copy_(0, idx, v.reshape(1, self.n_kv, self.head_dim))

    def write_range(self, layer: int, start: int, k: torch.Tensor, v: torch.Tensor) -> None:
        n = int(k.shape[0])
        end = int(start) + n
        if start < 0 or end > self.max_seq:
            raise ValueError(f"KV overflow: writing slots {start}..{end} into max_seq={self.max_seq}")
        self.k[layer, start:end].copy_(k.reshape(n, self.n_kv, self.head_dim))
        self.v[layer, start:end].copy_(v.reshape(n, self.n_kv, self.head_dim))

    def mark_written(self, position: torch.Tensor) -> None:
        """``valid_len = position + 1`` in place (capturable, no temporaries)."""
        self.valid_len.copy_(position.reshape(()))
        self.valid_len.add_(1)


@dataclass
class Arena:
    spec: ArchSpec
    x: torch.Tensor
    h: torch.Tensor
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    qkv: torch.Tensor
    attn: torch.Tensor
    down_in: torch.Tensor
    logits: torch.Tensor
    attn_ws: torch.Tensor
    pick_scratch: torch.Tensor
    status: torch.Tensor
    partial: torch.Tensor        # FP32 [hidden]: row-split partial sums under tensor parallelism
    logits_local: torch.Tensor   # bf16 [vocab / tp]: this rank's lm_head rows

    @classmethod
    def allocate(cls, spec: ArchSpec, *, device, dtype: torch.dtype = torch.bfloat16) -> "Arena":
        z = lambda *shape: torch.zeros(shape, dtype=dtype, device=device)
        return cls(
            spec=spec,
            x=z(1, spec.hidden),
            h=z(1, spec.hidden),
            q=z(1, spec.n_q, spec.head_dim),
            k=z(1, spec.n_kv, spec.head_dim),
            v=z(1, spec.n_kv, spec.head_dim),
            qkv=z(1, spec.wqkv_out),
            attn=z(1, spec.q_dim),
            down_in=z(1, spec.intermediate),
            logits=z(1, spec.vocab),
            attn_ws=torch.zeros(
                spec.n_q * ATTN_SPLIT * (spec.head_dim + 2), dtype=torch.float32, device=device
            ),
            pick_scratch=torch.zeros(16, dtype=torch.uint8, device=device),
            status=torch.zeros((), dtype=torch.int32, device=device),
            partial=torch.zeros(spec.hidden, dtype=torch.float32, device=device),
            logits_local=z(1, spec.vocab // spec.tp),
        )


@dataclass
class DecodeState:
    spec: ArchSpec
    token: torch.Tensor
    position: torch.Tensor
    valid_len: torch.Tensor
    next_token: torch.Tensor
    finished: torch.Tensor
    kv: GraphSafeKV
    arena: Arena
    cos: torch.Tensor
    sin: torch.Tensor
    embed: "torch.Tensor | PackedEmbed"
    eos_id: torch.Tensor
    comm: object = None          # tp.Comm; None = single GPU
    peers: object = None         # tp.PeerExchange: row-split sums over peer memory instead of NCCL
    pick_peers: object = None    # tp.PeerExchange of the greedy pick (a set of its own)

    def enable_peer_exchange(self, on: bool = True) -> str | None:
        """Sum the row-split partials inside the GEMV launch, over NVLink peer memory
        (collective: call it on every rank at the same point). Returns how the buffers
        were mapped, or ``None`` when switched off / single GPU."""
        if not on or self.comm is None or self.comm.world < 2:
            self.peers = None
            self.pick_peers = None
            return None
        if self.peers is None:
            from .tp import PeerExchange

            self.peers = PeerExchange(self.comm, self.spec.hidden, self.device)
            # the pick's (value, id) pairs travel through a small set of their own
            self.pick_peers = PeerExchange(self.comm, 2, self.device)
        return self.peers.how

    @classmethod
    def allocate(cls, spec: ArchSpec, embed, *, device=None, dtype: torch.dtype = torch.bfloat16,
                 cos: torch.Tensor | None = None, sin: torch.Tensor | None = None,
                 comm=None) -> "DecodeState":
        if isinstance(embed, PackedEmbed):
            if embed.shape != (spec.vocab, spec.hidden):
                raise ValueError(f"embed shape {embed.shape} != {(spec.vocab, spec.hidden)}")
            device = embed.device if device is None else device
            held = embed
        else:
            if embed.ndim != 2 or tuple(embed.shape) != (spec.vocab, spec.hidden):
                raise ValueError(f"embed shape {tuple(embed.shape)} != {(spec.vocab, spec.hidden)}")
            device = embed.device if device is None else device
            held = embed.to(device=torch.device(device), dtype=dtype)
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError("the resident executor is CUDA-only (no CPU path)")
        if spec.tp > 1 and (comm is None or comm.world != spec.tp):
            raise ValueError(f"a tp={spec.tp} shard needs a communicator of that size")
        valid_len = torch.zeros((), dtype=torch.int32, device=device)
        if cos is None or sin is None:
            cos, sin = rope_tables_torch(
                spec.max_seq, spec.head_dim, spec.rope_theta, device=device, dtype=dtype
            )
        else:
            cos = cos.to(device=device, dtype=dtype)
            sin = sin.to(device=device, dtype=dtype)
        scalar = lambda dt: torch.zeros((), dtype=dt, device=device)
        return cls(
            spec=spec,
            token=scalar(torch.int64),
            position=scalar(torch.int64),
            valid_len=valid_len,
            next_token=scalar(torch.int64),
            finished=scalar(torch.uint8),
            kv=GraphSafeKV(spec, device=device, dtype=dtype, valid_len=valid_len),
            arena=Arena.allocate(spec, device=device, dtype=dtype),
            cos=cos.contiguous(),
            sin=sin.contiguous(),
            embed=held,
            eos_id=torch.tensor(spec.eos_id, dtype=torch.int64, device=device),
            comm=comm,
        )

    @property
    def device(self) -> torch.device:
        return self.token.device

    def reset(self) -> None:
        """New request; stale KV rows are legal, ``valid_len`` hides them."""
        for t in (self.token, self.position, self.valid_len, self.next_token, self.finished):
            t.zero_()

    def load_token(self, token_id: int) -> None:
        self.token.fill_(int(token_id))

    def commit_step(self) -> None:
        """Feed the greedy id back without a host round trip (tensor-op form)."""
        self.token.copy_(self.next_token)
        self.position.add_(1)
        self.finished.bitwise_or_((self.next_token == self.eos_id).to(dtype=self.finished.dtype))
