"""Tensor-parallel sharding of the NF4 decoder over the GPUs of one box.

Not in the reference (single GPU). Column-split (rows of W, contiguous slices of
the packed bytes, nothing repacked): q / k / v by head, InternLM's fused wqkv by kv
group, gate, up, lm_head. Row-split (K ranges that are multiples of 64, so no NF4
group straddles ranks; bytes are copied into a contiguous per-rank blob, never
re-quantized): o, down. One sum all-reduce of the FP32 partial per row-split
layer and one all-gather of the logits slices per token, both issued on the
capture stream so they become nodes of the step graph.

``Comm`` wraps ``torch.distributed``; the same code runs with the NCCL backend on
GPUs and with gloo on CPU (sharding arithmetic and the collectives' semantics are
tested there).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .arch import ArchSpec, group_range, shard_spec
from .linear import DeviceLayer, DeviceLinear, DeviceWeights

__all__ = ["Comm", "PeerExchange", "shard_linear_cols", "shard_linear_rows", "shard_weights",
           "kv_head_rows"]


@dataclass
class Comm:
    """Rank / world plus the two collectives the step needs."""

    rank: int = 0
    world: int = 1
    group: object | None = None

    @classmethod
    def from_env(cls) -> "Comm":
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            return cls(dist.get_rank(), dist.get_world_size(), None)
        return cls()

    def shutdown(self, *holders, grace_s: float = 20.0) -> None:
        """Leave the process group at the end of a run.

        ``destroy_process_group`` does not return while a CUDA graph that captured NCCL
        kernels is alive (seen with torch 2.11 / NCCL 2.28 on two B200s: both ranks sat
        in it until killed), so the graphs of the given loops are dropped first, the
        device is drained and the ranks meet at a barrier; the destroy then runs on a
        helper thread, and a rank whose destroy still has not returned after
        ``grace_s`` exits the process directly - nothing of its own is in flight by then.
        """
        import gc
        import os
        import sys
        import threading

        import torch.distributed as dist

        if not (dist.is_available() and dist.is_initialized()):
            return
        for h in holders:
            if hasattr(h, "_graph"):
                h._graph = None
                h.graph_mode = "off"
            if hasattr(h, "_prefill_graphs"):
                h._prefill_graphs = None
        gc.collect()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        dist.barrier(group=self.group)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        done = threading.Event()

        def _destroy() -> None:
            try:
                dist.destroy_process_group()
            finally:
                done.set()

        threading.Thread(target=_destroy, daemon=True).start()
        if not done.wait(grace_s):
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)

    def all_reduce_sum(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t

    def all_gather_into(self, out: torch.Tensor, part: torch.Tensor) -> torch.Tensor:
        """``out`` (world * part.numel()) <- every rank's ``part`` in rank order."""
        if self.world > 1:
            import torch.distributed as dist

            dist.all_gather_into_tensor(out, part, group=self.group)
        else:
            out.copy_(part.reshape(out.shape))
        return out


class PeerExchange:
    """Buffers of the fused row-split GEMV + all-reduce (``chr_nf4_gemv_allreduce``).

    Every rank allocates a receive buffer (two halves x one slot per source rank x
    ``max_rows`` 8-byte words of (value, epoch)) and a block of flag words in memory that all ranks of the box
    can address, exchanges the mappings once, and keeps the ``chr_nf4_peers_t`` the
    kernel takes. Mapping goes through torch's symmetric memory (NVLink peer access,
    multicast left off); when that is unavailable, through CUDA IPC handles of ordinary
    allocations. Collective: every rank of ``comm`` must construct it at the same point.
    """

    def __init__(self, comm: Comm, max_rows: int, device) -> None:
        import os

        import torch.distributed as dist

        from gpu.nf4._lib import AR_MAX_CTAS, AR_MAX_RANKS, ChrNf4Peers

        if comm.world < 2 or comm.world > AR_MAX_RANKS:
            raise ValueError(f"peer exchange needs 2..{AR_MAX_RANKS} ranks, got {comm.world}")
        self.comm, self.max_rows = comm, int(max_rows)
        self._per_shape: dict = {}
        dev = torch.device(device)
        n_recv = 2 * comm.world * self.max_rows * 2          # two halves x ranks x rows of 8-byte words
        n_flags = comm.world * AR_MAX_CTAS                   # uint32, kept as int32
        n_words = n_recv + n_flags
        self.how = "symmetric_memory"
        try:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm

            buf = symm.empty(n_words, dtype=torch.float32, device=dev)
            buf.zero_()
            hdl = symm.rendezvous(buf, dist.group.WORLD if comm.group is None else comm.group)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
            self._keep = (buf, hdl)
        except Exception as exc:  # noqa: BLE001 - fall back to IPC handles
            self.how = f"cuda_ipc ({type(exc).__name__})"
            buf = torch.zeros(n_words, dtype=torch.float32, device=dev)
            handle = buf.untyped_storage()._share_cuda_()
            gathered: list = [None] * comm.world
            dist.all_gather_object(gathered, handle, group=comm.group)
            opened, ptrs = [], []
            for r, h in enumerate(gathered):
                if r == comm.rank:
                    ptrs.append(buf.data_ptr())
                    continue
                st = torch.UntypedStorage._new_shared_cuda(*h)
                opened.append(st)
                ptrs.append(st.data_ptr())
            self._keep = (buf, opened)
        torch.cuda.synchronize(dev)
        dist.barrier(group=comm.group)
        self.local = buf
        self.epoch = torch.zeros(2, dtype=torch.int32, device=dev)
        self.status = torch.zeros((), dtype=torch.int32, device=dev)
        peers = ChrNf4Peers()
        peers.rank, peers.world = comm.rank, comm.world
        peers.capacity = self.max_rows
        for r, base in enumerate(ptrs):
            peers.recv[r] = base
            peers.flags[r] = base + 4 * n_recv
        peers.epoch, peers.status = self.epoch.data_ptr(), self.status.data_ptr()
        self.peers = peers

    def for_matrix(self, mat: DeviceLinear):
        """The ``chr_nf4_peers_t`` to pass for this row-split matrix: carries the largest
        ``K_pad`` any rank holds for it, so that all ranks tile its rows alike. The first
        call per shape is a collective (max over ranks) and must happen outside capture."""
        if int(mat.M) > self.max_rows:
            raise ValueError(f"matrix has {mat.M} rows, the receive buffers were sized for "
                             f"{self.max_rows}")
        key = (int(mat.M), int(mat.K_pad))
        got = self._per_shape.get(key)
        if got is None:
            import ctypes

            import torch.distributed as dist

            widest = torch.tensor([int(mat.K_pad)], dtype=torch.int64, device=self.local.device)
            dist.all_reduce(widest, op=dist.ReduceOp.MAX, group=self.comm.group)
            got = type(self.peers)()
            ctypes.memmove(ctypes.byref(got), ctypes.byref(self.peers), ctypes.sizeof(got))
            got.shape_k_pad = int(widest.item())
            self._per_shape[key] = got
        return got

    def timed_out(self) -> bool:
        """True when some wait for a peer ran out of polls since the last call (host read)."""
        hit = bool(self.status.item())
        if hit:
            self.status.zero_()
        return hit


def _rows(mat: DeviceLinear, lo: int, hi: int) -> DeviceLinear:
    """Rows lo..hi of a matrix: a view of the packed bytes, no copy."""
    bias = None if mat.bias is None else mat.bias[lo:hi].contiguous()
    return DeviceLinear(mat.packed[lo:hi], mat.scale[lo:hi], hi - lo, mat.K, mat.K_pad, bias)


def shard_linear_cols(mat: DeviceLinear, rank: int, world: int) -> DeviceLinear:
    """Output rows ``[rank*M/world, (rank+1)*M/world)``."""
    if mat.M % world:
        raise ValueError(f"M={mat.M} does not divide by {world}")
    step = mat.M // world
    return _rows(mat, rank * step, (rank + 1) * step)


def shard_linear_rows(mat: DeviceLinear, rank: int, world: int,
                      k_range: tuple[int, int] | None = None) -> DeviceLinear:
    """Input range ``k_range`` (default: the rank's even share) re-laid as its own
    matrix. The range must start and end on NF4 group boundaries. The bias (if any)
    stays on rank 0 only, so that the all-reduced sum carries it once."""
    lo, hi = k_range if k_range is not None else group_range(mat.K, world, rank)
    if lo % 64 or hi % 64 or not 0 <= lo < hi <= mat.K:
        raise ValueError(f"K range {lo}..{hi} of {mat.K} is not made of whole NF4 groups")
    packed = mat.packed[:, lo // 2:hi // 2].contiguous()
    scale = mat.scale[:, lo // 64:hi // 64].contiguous()
    return DeviceLinear(packed, scale, mat.M, hi - lo, hi - lo, mat.bias if rank == 0 else None)


def kv_head_rows(full: ArchSpec, rank: int, world: int) -> tuple[int, int]:
    """Row range of this rank's kv heads inside a full k or v projection."""
    hd = full.head_dim
    if full.n_kv % world == 0:
        per = full.n_kv // world
        return rank * per * hd, (rank + 1) * per * hd
    head = rank // (world // full.n_kv)
    return head * hd, (head + 1) * hd


def _shard_wqkv(mat: DeviceLinear, full: ArchSpec, rank: int, world: int) -> DeviceLinear:
    """InternLM packing [n_kv, n_rep + 2, hd]: kv groups are contiguous row blocks."""
    if full.n_kv % world:
        raise ValueError("fused wqkv needs n_kv divisible by the tensor-parallel degree")
    group = (full.n_rep + 2) * full.head_dim
    per = full.n_kv // world
    return _rows(mat, rank * per * group, (rank + 1) * per * group)


def shard_weights(weights: DeviceWeights, rank: int, world: int) -> DeviceWeights:
    """This rank's shard of a full model (views where possible)."""
    full = weights.spec
    if world == 1:
        return weights
    local = shard_spec(full, world, rank)
    mlp = group_range(full.intermediate, world, rank)
    layers = []
    for ly in weights.layers:
        q = k = v = wqkv = None
        if ly.wqkv is not None:
            wqkv = _shard_wqkv(ly.wqkv, full, rank, world)
        else:
            q = shard_linear_cols(ly.q, rank, world)
            lo, hi = kv_head_rows(full, rank, world)
            k, v = _rows(ly.k, lo, hi), _rows(ly.v, lo, hi)
        layer = DeviceLayer(
            ly.norm1, ly.norm2, q, k, v, wqkv,
            shard_linear_rows(ly.o, rank, world),
            _rows(ly.gate, *mlp),
            _rows(ly.up, *mlp),
            shard_linear_rows(ly.down, rank, world, mlp),
        )
        # on the device the shard's q/k/v and gate/up rows are copied next to each other
        # (the prefill then runs each group as one GEMM, and the shard no longer keeps
        # the full matrices alive through its views)
        layers.append(layer.adjoin() if ly.o.packed.is_cuda else layer)
    return DeviceWeights(local, weights.embed, weights.final_norm,
                         shard_linear_cols(weights.lm_head, rank, world), layers)
