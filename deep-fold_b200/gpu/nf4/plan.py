"""Pure-Python mirror of the library's GEMM launch planner (no GPU, no ctypes).

Keeps the reference's planner surface (gpu/nf4/plan.py:161-236): ``plan(M, K,
N, ...) -> Plan`` with the same fields, ``k_pad``, ``LIVE_MAX_N`` and
``PLAN_MAX_N``. The tile table is this library's (sm_100a), so the numbers are
not the reference's; the arithmetic (split-K aimed at two CTAs per SM, capped at
the K tiles, ``ws_floats = split*M*N``) is. ``tests`` check it against
``chr_nf4_gemm_plan`` whenever the library is loadable.
"""

from __future__ import annotations

from dataclasses import dataclass

__all__ = [
    "TCGEN05",
    "SIMT",
    "GROUP_SIZE",
    "LIVE_MAX_N",
    "PLAN_MAX_N",
    "ONE_WAVE",
    "Plan",
    "k_pad",
    "plan",
    "tc_supported",
]

TCGEN05 = 0
SIMT = 1

GROUP_SIZE = 64
#: widest N one ``nf4_gemm`` call launches; hosts chunk above it.
LIVE_MAX_N = 32
#: widest N the planner describes and ``max_n`` may unlock.
PLAN_MAX_N = 64
#: SMs of a B200; the unit of the split-K target when no device is visible.
ONE_WAVE = 148

_PATH_NAME = {TCGEN05: "tcgen05", SIMT: "simt"}

# SIMT tile: bm, bk, block, static shared bytes.
_SIMT_TILE = (64, 64, 256, 4 * (64 * 65 + 64 * 64 + 16))


def k_pad(k: int) -> int:
    """``64 * ceil(K / 64)``."""
    return GROUP_SIZE * ((int(k) + GROUP_SIZE - 1) // GROUP_SIZE)


def _ceil_div(a: int, b: int) -> int:
    return -(-int(a) // int(b))


def tc_bn(n: int) -> int:
    """Column tile of the tensor-core kernel: N rounded up to 16, 32 or 64."""
    n = int(n)
    return 16 if n <= 16 else (32 if n <= 32 else 64)


def tc_tile(n: int) -> tuple[int, int, int, int]:
    """(bm, bk, block, dynamic shared bytes) of the tensor-core kernel for N."""
    bn = tc_bn(n)
    stages = 4
    per_stage = 128 * 32 + 128 * 64 * 2 + bn * 64 * 2  # packed codes + bf16 A + bf16 B
    return 128, 64, 192, stages * per_stage + 1024 + 256


def tc_supported(m: int, kp: int, n: int) -> bool:
    """Shapes the tensor-core kernel takes: the packed row pitch must be a multiple
    of 16 bytes (always true for K_pad a multiple of 64) and N <= 64."""
    return 1 <= int(n) <= PLAN_MAX_N and (int(kp) // 2) % 16 == 0


@dataclass(frozen=True)
class Plan:
    path: int
    grid_x: int
    grid_y: int
    block: int
    bm: int
    bk: int
    n_ktiles: int
    tiles_per_split: int
    ctas: int
    smem_bytes: int
    ws_floats: int

    @property
    def path_name(self) -> str:
        return _PATH_NAME[self.path]

    @property
    def waves(self) -> float:
        return self.ctas / ONE_WAVE

    def as_dict(self) -> dict:
        return {f: getattr(self, f) for f in self.__dataclass_fields__}


def plan(
    M: int,  # noqa: N803
    K: int,  # noqa: N803
    N: int = 1,  # noqa: N803
    *,
    K_pad: int | None = None,  # noqa: N803
    have_ws: bool = True,
    force_path: int | None = None,
    force_split: int = 0,
    one_wave: int = ONE_WAVE,
) -> Plan:
    """Launch plan for ``y[M,N] = dequant_nf4(W[M,K]) @ x[K,N]``."""
    M, K, N = int(M), int(K), int(N)
    if M < 1 or K < 1:
        raise ValueError(f"M and K must be >= 1, got M={M} K={K}")
    if not 1 <= N <= PLAN_MAX_N:
        raise ValueError(f"N={N} not in 1..{PLAN_MAX_N} (live launch is 1..{LIVE_MAX_N})")
    kp = k_pad(K) if K_pad is None else int(K_pad)
    if kp != k_pad(K):
        raise ValueError(f"K_pad={kp} != 64*ceil(K/64) = {k_pad(K)}")

    if force_path is not None:
        path = int(force_path)
    else:
        path = TCGEN05 if tc_supported(M, kp, N) else SIMT
    bm, bk, block, smem = tc_tile(N) if path == TCGEN05 else _SIMT_TILE
    grid_x = _ceil_div(M, bm)
    n_ktiles = _ceil_div(kp, bk)
    want = 1
    if have_ws:
        want = force_split if force_split > 0 else _ceil_div(max(1, 2 * int(one_wave)), grid_x)
    want = max(1, min(want, n_ktiles))
    tiles_per_split = _ceil_div(n_ktiles, want)
    split = _ceil_div(n_ktiles, tiles_per_split)
    return Plan(
        path=path,
        grid_x=grid_x,
        grid_y=split,
        block=block,
        bm=bm,
        bk=bk,
        n_ktiles=n_ktiles,
        tiles_per_split=tiles_per_split,
        ctas=grid_x * split,
        smem_bytes=smem,
        ws_floats=split * M * N if split > 1 else 0,
    )
