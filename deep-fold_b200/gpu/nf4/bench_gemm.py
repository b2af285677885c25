"""Microbenchmark of the wide NF4 GEMM (``chr_nf4_gemm_rows``) on the architectures' shapes.

    python deep-fold_b200/gpu/nf4/bench_gemm.py [--shape NAME ...] [--n 512 2048 4096] [--iters 10]

``y_rows[N, M] = x_rows[N, K] . dequant(W)^T`` with random NF4 blobs and bf16
activations. Launches go out back to back and are timed with CUDA events (the
split-K reduction, where the plan has one, is inside the timed region). One JSON
line per (shape, N): microseconds, TFLOP/s (2*M*K*N), and the fraction of the
burst and sustained bf16 peaks measured on this pool when ``MEASURED_PEAKS.json``
is present next to the repository root.
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

from gpu.nf4 import nf4_gemm_rows, nf4_gemm_status  # noqa: E402
from gpu.nf4.plan import k_pad  # noqa: E402

SHAPES = {
    "3b_qkv": (2560, 2048), "3b_o": (2048, 2048), "3b_gate_up": (22016, 2048), "3b_down": (2048, 11008),
    "14b_gate_up": (27648, 5120), "14b_down": (5120, 13824), "20b_gate_up": (32768, 6144),
    "32b_gate": (27648, 5120), "32b_down": (5120, 27648), "cfg1": (4096, 4096),
}


def peaks() -> dict:
    path = _PKG.parent / "MEASURED_PEAKS.json"
    try:
        d = json.loads(path.read_text())
        return {"burst": float(d["bf16_tflops"]), "sustained": float(d["bf16_tflops_sustained"])}
    except (OSError, KeyError, ValueError):
        return {}


def run(name: str, n: int, iters: int, gen: torch.Generator) -> dict:
    m, k = SHAPES[name]
    kp = k_pad(k)
    packed = torch.randint(0, 256, (m, kp // 2), generator=gen, device="cuda", dtype=torch.uint8)
    scale = (torch.rand((m, kp // 64), generator=gen, device="cuda") * 0.04 + 0.012).to(torch.float16)
    x = torch.randn((n, k), generator=gen, device="cuda").to(torch.bfloat16)
    for _ in range(3):
        nf4_gemm_rows(packed, scale, x, m, k, kp)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        nf4_gemm_rows(packed, scale, x, m, k, kp)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / iters
    tf = 2.0 * m * k * n / us / 1e6
    out = {"shape": name, "MxK": [m, k], "N": n, "us": round(us, 1), "tflops": round(tf, 1),
           "status": nf4_gemm_status()}
    for kind, peak in peaks().items():
        out[f"frac_of_{kind}_peak"] = round(tf / peak, 3)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", nargs="*", default=None)
    ap.add_argument("--n", nargs="*", type=int, default=[512, 2048, 4096])
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0)
    for name in args.shape or list(SHAPES):
        for n in args.n:
            print(json.dumps(run(name, n, args.iters, gen)), flush=True)


if __name__ == "__main__":
    main()
