"""Decoder architectures the executors can drive.

``ArchSpec`` keeps the field names and derived properties of the reference's
spec (gpu/decodev2/plan.py:17-78) so states, weights and tests read the same.
Besides the reference's three toy specs this module carries the four
checkpoint-shaped configurations the benchmarks use (random-init weights).
"""

from __future__ import annotations

from dataclasses import dataclass, replace

__all__ = [
    "ArchSpec",
    "TINY_LLAMA",
    "TINY_INTERNLM",
    "MEDIUM_LLAMA",
    "QWEN25_3B",
    "QWEN25_14B",
    "INTERNLM25_20B",
    "QWEN25_32B",
    "CONFIGS",
    "with_max_seq",
    "shard_spec",
    "group_range",
]

_FAMILIES = ("llama_swiglu", "internlm_gqa")


@dataclass(frozen=True)
class ArchSpec:
    """``llama_swiglu``: split q/k/v (+bias allowed); ``internlm_gqa``: fused wqkv
    whose rows are grouped per kv head as [n_rep q heads, k, v]."""

    name: str
    family: str
    n_layers: int
    hidden: int
    n_q: int
    n_kv: int
    head_dim: int
    intermediate: int
    vocab: int
    max_seq: int
    rms_eps: float = 1e-6
    rope_theta: float = 10000.0
    eos_id: int = 2
    tied_embed: bool = False
    qkv_bias: bool = False
    #: tensor-parallel degree this spec is one shard of; ``n_q``, ``n_kv`` and
    #: ``intermediate`` are the LOCAL sizes when ``tp > 1`` (``hidden`` and ``vocab`` stay
    #: global: the residual stream and the gathered logits are replicated).
    tp: int = 1
    #: ranks that hold a copy of the same kv head (``tp > n_kv`` of the full model)
    kv_replicas: int = 1

    def __post_init__(self) -> None:
        if self.family not in _FAMILIES:
            raise ValueError(f"unsupported family {self.family!r}")
        if self.n_layers < 1 or self.max_seq < 2:
            raise ValueError("need at least one layer and max_seq>=2")
        if self.hidden != self.n_q * self.head_dim * self.tp:
            raise ValueError(
                f"hidden {self.hidden} != n_q*head_dim*tp {self.n_q * self.head_dim * self.tp}")
        if self.n_q % self.n_kv:
            raise ValueError(f"n_q={self.n_q} is not a multiple of n_kv={self.n_kv}")
        if self.head_dim % 2:
            raise ValueError("RoPE needs even head_dim")
        if self.hidden % 64 or self.intermediate % 64:  # row-split shards keep whole NF4 groups
            raise ValueError("hidden and intermediate must be multiples of NF4 group 64")
        if not 0 <= self.eos_id < self.vocab:
            raise ValueError(f"eos_id {self.eos_id} out of vocab {self.vocab}")

    @property
    def n_rep(self) -> int:
        return self.n_q // self.n_kv

    @property
    def q_dim(self) -> int:
        return self.n_q * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv * self.head_dim

    @property
    def wqkv_out(self) -> int:
        return (self.n_q + 2 * self.n_kv) * self.head_dim

    @property
    def attn_scale(self) -> float:
        return self.head_dim**-0.5

    def linear_shapes(self) -> dict[str, tuple[int, int]]:
        """(M, K) of every linear of one layer plus lm_head."""
        h, i = self.hidden, self.intermediate
        out: dict[str, tuple[int, int]] = {}
        if self.family == "internlm_gqa":
            out["wqkv"] = (self.wqkv_out, h)
        else:
            out.update(q=(self.q_dim, h), k=(self.kv_dim, h), v=(self.kv_dim, h))
        out.update(o=(h, self.q_dim), gate=(i, h), up=(i, h), down=(h, i), lm_head=(self.vocab, h))
        return out

    def packed_bytes_per_token(self) -> int:
        """NF4 bytes (codes + scales) one decode step reads: all layers + lm_head."""
        per = lambda m, k: m * k // 2 + m * (k // 64) * 2
        shapes = self.linear_shapes()
        layer = sum(per(*mk) for name, mk in shapes.items() if name != "lm_head")
        return self.n_layers * layer + per(*shapes["lm_head"])


def group_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """Elements ``[lo, hi)`` of a ``total``-wide axis owned by ``rank`` when the axis
    is cut at NF4 group boundaries (multiples of 64); the first ranks take the
    remainder groups, so shards may differ by one group."""
    groups = total // 64
    base, rem = divmod(groups, world)
    lo = rank * base + min(rank, rem)
    return lo * 64, (lo + base + (1 if rank < rem else 0)) * 64


def shard_spec(spec: ArchSpec, world: int, rank: int = 0) -> ArchSpec:
    """The per-rank spec of ``spec`` under tensor parallelism of degree ``world``.

    Query heads, the MLP width and the lm_head rows are divided; kv heads are divided
    when there are enough of them and otherwise replicated (each rank keeps the one
    kv head its query heads attend to). The MLP width is cut at NF4 group
    boundaries, so it may differ by 64 between ranks."""
    world = int(world)
    if spec.tp != 1:
        raise ValueError("spec is already a shard")
    if world == 1:
        return spec
    if spec.n_q % world or spec.vocab % world or spec.intermediate // 64 < world:
        raise ValueError(f"{spec.name}: n_q / vocab / intermediate do not divide by tp={world}")
    if spec.n_kv % world == 0:
        n_kv, reps = spec.n_kv // world, 1
    elif world % spec.n_kv == 0:
        n_kv, reps = 1, world // spec.n_kv
    else:
        raise ValueError(f"{spec.name}: n_kv={spec.n_kv} and tp={world} do not nest")
    if (spec.n_q // world) % n_kv:
        raise ValueError("local query heads must be a multiple of local kv heads")
    # o_proj is cut along K at NF4 group boundaries and q along whole heads: the two
    # cuts only coincide when a rank's query width is made of whole groups; the MLP
    # width must be whole groups for its tail not to be dropped.
    if ((spec.n_q // world) * spec.head_dim) % 64 or spec.intermediate % 64:
        raise ValueError(f"{spec.name}: per-rank query width and the MLP width must be multiples "
                         f"of 64 under tp={world}")
    lo, hi = group_range(spec.intermediate, world, rank)
    return replace(spec, n_q=spec.n_q // world, n_kv=n_kv, intermediate=hi - lo,
                   tp=world, kv_replicas=reps)


def with_max_seq(spec: ArchSpec, max_seq: int) -> ArchSpec:
    return replace(spec, max_seq=int(max_seq))


TINY_LLAMA = ArchSpec("tiny-llama", "llama_swiglu", 2, 64, 4, 2, 16, 128, 32, 16)
TINY_INTERNLM = ArchSpec("tiny-internlm", "internlm_gqa", 2, 64, 4, 2, 16, 128, 32, 16)
MEDIUM_LLAMA = ArchSpec("medium-llama", "llama_swiglu", 4, 512, 8, 2, 64, 1024, 128, 32)

QWEN25_3B = ArchSpec(
    "qwen2.5-3b-arch", "llama_swiglu", 36, 2048, 16, 2, 128, 11008, 151936, 2048,
    rope_theta=1.0e6, eos_id=151645, tied_embed=True, qkv_bias=True,
)
QWEN25_14B = ArchSpec(
    "qwen2.5-14b-arch", "llama_swiglu", 48, 5120, 40, 8, 128, 13824, 152064, 2048,
    rope_theta=1.0e6, eos_id=151645, qkv_bias=True,
)
INTERNLM25_20B = ArchSpec(
    "internlm2.5-20b-arch", "internlm_gqa", 48, 6144, 48, 8, 128, 16384, 92544, 2048,
    rms_eps=1e-5, rope_theta=1.0e6, eos_id=2,
)
QWEN25_32B = ArchSpec(
    "qwen2.5-32b-arch", "llama_swiglu", 64, 5120, 40, 8, 128, 27648, 152064, 2048,
    rope_theta=1.0e6, eos_id=151645, qkv_bias=True,
)

CONFIGS = {s.name: s for s in (QWEN25_3B, QWEN25_14B, INTERNLM25_20B, QWEN25_32B)}
