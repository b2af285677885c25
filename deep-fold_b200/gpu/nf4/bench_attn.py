"""Microbenchmark of the GQA decode attention (``chr_nf4_attn``) on the architectures' head layouts.

    python deep-fold_b200/gpu/nf4/bench_attn.py [--layout 32b|20b|14b|3b ...] [--valid 256 1800]
                                                [--splits 8 16 32] [--layers 64] [--plain]

Every launch works on its own layer's cache (``--layers`` distinct K/V blocks of
``max_seq`` rows, together larger than L2), with RoPE and the cache write of the
current token fused in, as in the decode step. Launches are captured in a CUDA graph
and the replay is timed with CUDA events; ``--plain`` launches eagerly instead (for a
profiler that wants individual launches). One JSON line per (layout, valid, splits):
algorithmic bytes (K and V rows below ``valid``), microseconds per launch, GB/s.
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

from gpu.nf4 import nf4_attn  # noqa: E402

# n_q, n_kv, head_dim
LAYOUTS = {"32b": (40, 8, 128), "14b": (40, 8, 128), "20b": (48, 8, 128), "3b": (16, 2, 128),
           "32b_tp8": (5, 1, 128)}


def run(name: str, valid: int, splits: int, layers: int, max_seq: int, plain: bool) -> dict:
    n_q, n_kv, hd = LAYOUTS[name]
    dev, bf = "cuda", torch.bfloat16
    gen = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s: torch.randn(s, generator=gen, device=dev).to(bf)
    k, v = rnd(layers, max_seq, n_kv, hd), rnd(layers, max_seq, n_kv, hd)
    q, ka, va = rnd(n_q, hd), rnd(n_kv, hd), rnd(n_kv, hd)
    cos, sin = rnd(max_seq, hd), rnd(max_seq, hd)
    out = torch.zeros(n_q, hd, device=dev, dtype=bf)
    vl = torch.tensor(valid, dtype=torch.int32, device=dev)
    pos = torch.tensor(valid - 1, dtype=torch.int64, device=dev)
    ws = torch.zeros(n_q * 64 * (hd + 2), device=dev)
    scale = hd ** -0.5

    def sweep():
        for li in range(layers):
            nf4_attn(q, k[li], v[li], out, vl, scale, ws, splits, ka, va, cos, sin, pos)

    sweep()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if plain:
        e0.record()
        sweep()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / layers
    else:
        graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.cuda.graph(graph, stream=side):
            sweep()
        torch.cuda.current_stream().wait_stream(side)
        us = float("inf")
        for _ in range(5):
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            us = min(us, e0.elapsed_time(e1) * 1e3 / layers)
    nbytes = 2 * valid * n_kv * hd * 2
    return {"layout": name, "heads": [n_q, n_kv, hd], "valid": valid, "splits_asked": splits,
            "bytes": nbytes, "us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layout", nargs="*", default=["32b"])
    ap.add_argument("--valid", nargs="*", type=int, default=[256, 1800])
    ap.add_argument("--splits", nargs="*", type=int, default=[32])
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--max-seq", type=int, default=2048)
    ap.add_argument("--plain", action="store_true")
    args = ap.parse_args()
    for name in args.layout:
        for valid in args.valid:
            for splits in args.splits:
                print(json.dumps(run(name, valid, splits, args.layers, args.max_seq, args.plain)), flush=True)


if __name__ == "__main__":
    main()
