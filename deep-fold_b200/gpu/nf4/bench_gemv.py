"""Microbenchmark of the decode GEMV family on the architectures' real shapes.

    python deep-fold_b200/gpu/nf4/bench_gemv.py [--op gemv|swiglu|qkv|gemv_n] [--shape NAME ...]
                                                [--rows 4] [--iters 40] [--plain]

Weights are random NF4 blobs; enough distinct copies are rotated through that the
working set is several times the 126 MB L2 (the reference's microbench rotates
copies the same way, gpu/nf4/bench_gemv.py:34-50). Launches are captured in a
CUDA graph and the replay is timed with CUDA events, so the figure is device
time per launch without Python overhead. ``--plain`` launches eagerly instead
(used when a profiler wants to see individual launches). One JSON line per shape:
algorithmic bytes (packed + scales + x + y), microseconds, GB/s.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parents[2]
if str(_PKG) not in sys.path:
    sys.path.insert(0, str(_PKG))

from gpu.nf4 import nf4_gemv, nf4_gemv_n, nf4_qkv, nf4_swiglu  # noqa: E402
from gpu.nf4.plan import k_pad  # noqa: E402

SHAPES = {
    "3b_q": (2048, 2048), "3b_kv": (256, 2048), "3b_gate": (11008, 2048), "3b_down": (2048, 11008),
    "3b_head": (151936, 2048), "14b_q": (5120, 5120), "14b_kv": (1024, 5120),
    "14b_gate": (13824, 5120), "14b_down": (5120, 13824), "20b_wqkv": (8192, 6144),
    "20b_o": (6144, 6144), "20b_gate": (16384, 6144), "20b_down": (6144, 16384),
    "20b_head": (92544, 6144), "32b_gate": (27648, 5120), "32b_down": (5120, 27648),
    "32b_head": (152064, 5120), "cfg1": (4096, 4096),
}
QKV = {"3b": (2048, 256, 2048), "14b": (5120, 1024, 5120), "32b": (5120, 1024, 5120)}
ROTATE_BYTES = 400e6


def blob(m: int, k: int, gen: torch.Generator):
    kp = k_pad(k)
    packed = torch.randint(0, 256, (m, kp // 2), generator=gen, device="cuda", dtype=torch.uint8)
    scale = (torch.rand((m, kp // 64), generator=gen, device="cuda") * 0.04 + 0.012).to(torch.float16)
    return packed, scale


def nf4_bytes(m: int, k: int) -> int:
    kp = k_pad(k)
    return m * kp // 2 + m * (kp // 64) * 2


def time_launches(fn, n_rot: int, iters: int, plain: bool) -> float:
    """Microseconds per launch of ``fn(i)``, i cycling over the rotated copies."""
    for i in range(min(3, n_rot) + 2):
        fn(i % n_rot)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if plain:
        e0.record()
        for i in range(iters):
            fn(i % n_rot)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / iters
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for i in range(iters):
                fn(i % n_rot)
    torch.cuda.current_stream().wait_stream(side)
    best = float("inf")
    for _ in range(5):
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3 / iters)
    return best


def run(op: str, name: str, iters: int, plain: bool, gen: torch.Generator, rows: int = 4) -> dict:
    if op == "qkv":
        mq, mkv, k = QKV[name]
        per = nf4_bytes(mq, k) + 2 * nf4_bytes(mkv, k) + k * 2 + (mq + 2 * mkv) * 2
        n_rot = max(2, min(64, int(ROTATE_BYTES // per) + 1))
        mats = [(blob(mq, k, gen), blob(mkv, k, gen), blob(mkv, k, gen)) for _ in range(n_rot)]
        x = torch.randn(k, device="cuda").to(torch.bfloat16)
        outs = [torch.empty(m, dtype=torch.bfloat16, device="cuda") for m in (mq, mkv, mkv)]

        def fn(i):
            (qp, qs), (kp_, ks), (vp, vs) = mats[i]
            nf4_qkv(qp, qs, kp_, ks, vp, vs, x, mq, mkv, mkv, k, k_pad(k), *outs)

        shape = [mq + 2 * mkv, k]
    else:
        m, k = SHAPES[name]
        n_mats = 2 if op == "swiglu" else 1
        per = n_mats * nf4_bytes(m, k) + k * 2 + m * 2
        n_rot = max(2, min(64, int(ROTATE_BYTES // per) + 1))
        mats = [[blob(m, k, gen) for _ in range(n_mats)] for _ in range(n_rot)]
        x = torch.randn(k, device="cuda").to(torch.bfloat16)
        y = torch.empty(m, dtype=torch.bfloat16, device="cuda")
        if op == "gemv_n":  # the multi-row GEMV: `rows` activation rows through one entry call
            xr = torch.randn((rows, k), device="cuda").to(torch.bfloat16)
            yr = torch.empty((rows, m), dtype=torch.bfloat16, device="cuda")
            per += (rows - 1) * (k * 2 + m * 2)

            def fn(i):
                (p, s), = mats[i]
                nf4_gemv_n(p, s, xr, m, k, k_pad(k), out=yr)
        elif op == "swiglu":
            def fn(i):
                (gp, gs), (up, us) = mats[i]
                nf4_swiglu(gp, gs, up, us, x, m, k, k_pad(k), y)
        else:
            def fn(i):
                (p, s), = mats[i]
                nf4_gemv(p, s, x, m, k, k_pad(k), y)
        shape = [m, k]
    us = time_launches(fn, n_rot, iters, plain)
    out = {"op": op, "shape": name, "MxK": shape, "bytes": per, "us": round(us, 2),
           "gbs": round(per / us / 1e3, 1), "rotated_copies": n_rot}
    if op == "gemv_n":
        out["rows"] = rows
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="gemv", choices=("gemv", "swiglu", "qkv", "gemv_n"))
    ap.add_argument("--rows", type=int, default=4, help="activation rows of --op gemv_n (1..8)")
    ap.add_argument("--shape", nargs="*", default=None)
    ap.add_argument("--iters", type=int, default=40)
    ap.add_argument("--plain", action="store_true")
    args = ap.parse_args()
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0)
    names = args.shape or (list(QKV) if args.op == "qkv" else
                           [n for n in SHAPES if args.op in ("gemv", "gemv_n") or "gate" in n])
    for name in names:
        print(json.dumps(run(args.op, name, args.iters, args.plain, gen, args.rows)), flush=True)
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
