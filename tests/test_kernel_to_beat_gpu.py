"""The reference's own CUDA kernels timed beside this library's on the same B200, same
inputs (the "kernel to beat" of the decode GEMV family: gpu/nf4/nf4_gemv.cu:291-324,
392-495, built into ``oracle/_ref/libchr_nf4_ref.so`` by ``oracle/build.py``).

Each launch reads rotated weight copies larger than L2 (as gpu/nf4/bench_gemv.py:34-50
does), is captured in a CUDA graph and timed with CUDA events. The results of both
libraries must agree within the GEMV tolerance, this library must not be slower, and the
numbers are written to ``kernel_to_beat.json`` in the run's output folder.
"""

from __future__ import annotations

import json
from pathlib import Path

import pytest
import torch

import ref_backend as ref

pytestmark = pytest.mark.gpu

from gpu.nf4 import nf4_gemv, nf4_swiglu  # noqa: E402

OUT = Path(__file__).resolve().parents[1] / "gpurun_out"
SHAPES = [("gemv", "32b_down", 5120, 27648), ("gemv", "3b_lm_head", 151936, 2048),
          ("swiglu", "32b_gate_up", 27648, 5120), ("swiglu", "3b_gate_up", 11008, 2048)]


def blob(m, k, gen):
    packed = torch.randint(0, 256, (m, k // 2), generator=gen, device="cuda", dtype=torch.uint8)
    scale = (torch.rand((m, k // 64), generator=gen, device="cuda") * 0.04 + 0.012).to(torch.float16)
    return packed, scale


def graph_us(fn, copies, iters=12):
    for i in range(3):
        fn(i % copies)
    torch.cuda.synchronize()
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side), torch.cuda.graph(graph, stream=side):
        for i in range(iters):
            fn(i % copies)
    torch.cuda.current_stream().wait_stream(side)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = float("inf")
    for _ in range(3):
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3 / iters)
    return best


def test_this_library_against_the_reference_kernels_on_the_same_gpu():
    if not ref.available():
        pytest.skip("oracle/_ref/libchr_nf4_ref.so is not built: no reference kernels to time "
                    "(python oracle/build.py --reference <checkout>)")
    gen = torch.Generator(device="cuda").manual_seed(0)
    rows = []
    for op, name, m, k in SHAPES:
        n_mats = 2 if op == "swiglu" else 1
        per = n_mats * (m * k // 2 + m * (k // 64) * 2) + 2 * k + 2 * m
        copies = max(2, min(8, int(300e6 // per) + 1))
        mats = [[blob(m, k, gen) for _ in range(n_mats)] for _ in range(copies)]
        x = torch.randn(k, generator=gen, device="cuda").to(torch.bfloat16)
        y_ours = torch.zeros(m, dtype=torch.bfloat16, device="cuda")
        y_ref = torch.zeros(m, dtype=torch.bfloat16, device="cuda")

        def run(lib, y):
            if op == "swiglu":
                return lambda i: lib.nf4_swiglu(*mats[i][0], *mats[i][1], x, m, k, k, y)
            return lambda i: lib.nf4_gemv(*mats[i][0], x, m, k, k, y)

        import gpu.nf4 as ours

        run(ours, y_ours)(0)
        try:
            run(ref, y_ref)(0)
        except RuntimeError as exc:  # a shape the reference's kernel does not take
            rows.append({"op": op, "shape": name, "MxK": [m, k], "reference_error": str(exc)})
            continue
        torch.cuda.synchronize()
        err = float((y_ours.float() - y_ref.float()).abs().max() / y_ref.float().abs().max().clamp_min(1e-6))
        assert err <= 1e-2, f"{name}: results differ from the reference kernel by {err:.3e}"
        us_ours = graph_us(run(ours, y_ours), copies)
        us_ref = graph_us(run(ref, y_ref), copies)
        rows.append({"op": op, "shape": name, "MxK": [m, k], "bytes": per, "us": round(us_ours, 2),
                     "gbs": round(per / us_ours / 1e3, 1), "reference_us": round(us_ref, 2),
                     "reference_gbs": round(per / us_ref / 1e3, 1), "speedup": round(us_ref / us_ours, 2),
                     "max_rel_diff": err})
        assert us_ours <= us_ref, f"{name}: {us_ours:.1f} us against the reference kernel's {us_ref:.1f} us"
        del mats
        torch.cuda.empty_cache()
    print("kernel to beat:", json.dumps(rows))
    OUT.mkdir(exist_ok=True)
    (OUT / "kernel_to_beat.json").write_text(json.dumps(rows, indent=1))
