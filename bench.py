"""Benchmark of the NF4 decode/prefill path: batch-1 greedy decode tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--model qwen2.5-3b-arch] [--prompt 512]

One JSON line on stdout. A "step" is one greedy decode token (one replay of the
captured step graph) of the named random-init architecture after a 512-token
prompt. ``value`` is the device-window rate (tokens resident, no host traffic),
``e2e`` the rate with a pinned-host token id copied in and the picked id read
back every step. ``roofline`` times the dominant kernel (fused SwiGLU GEMV over
the layers' gate/up matrices, far larger than L2 in total) with CUDA events in
this same process; ``cpu_baseline`` times the CPU oracle (numpy dequant + float32
matmul, the reference's CPU NF4 path restated) on a bounded sample.
``--impl reference`` runs only that CPU path and prints its line.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (str(ROOT / "deep-fold_b200"), str(ROOT / "oracle")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

METRIC = "decode_tok_s_bs1"
UNIT = "tok/s"
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the timed kernel, from
# the ncu capture summarised under profiles/ (SwiGLU GEMV, gate/up [M, K]); other
# shapes scale by their algorithmic bytes (traffic / algorithmic = 1.001 there).
NCU_TRAFFIC_RATIO = 24002560 / 23979520


def measured_peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except (KeyError, ValueError):
            pass
    return FALLBACK_HBM_GBS, "fallback"


# --------------------------------------------------------------------------- #
# CPU reference arm: numpy dequant + float32 matmul on a bounded sample
# --------------------------------------------------------------------------- #
def cpu_layer_sample(spec, repeats: int = 1, seed: int = 0) -> dict:
    """Time one decoder layer's linears (N=1) and extrapolate to a token.

    The sample is one layer (q,k,v | wqkv, o, gate, up, down) of the named
    architecture on random NF4 blobs; lm_head is charged by its byte share.
    """
    import numpy as np

    import nf4_ref as o

    shapes = spec.linear_shapes()
    rng = np.random.default_rng(seed)
    mats = {}
    for name, (m, k) in shapes.items():
        if name == "lm_head":
            continue
        p, s = o.random_blobs(m, k, seed + len(mats), pad_garbage=False)
        mats[name] = (p, s, m, k, rng.standard_normal((k, 1)).astype(np.float32))
    best = float("inf")
    for _ in range(max(1, repeats)):
        t0 = time.perf_counter()
        for p, s, m, k, x in mats.values():
            o.matmul(o.dequantize(p, s, m, k), x)
        best = min(best, time.perf_counter() - t0)
    layer_weights = sum(m * k for name, (m, k) in shapes.items() if name != "lm_head")
    head_weights = shapes["lm_head"][0] * shapes["lm_head"][1]
    token_s = best * (spec.n_layers + head_weights / layer_weights)
    try:
        import threadpoolctl

        blas = max((d.get("num_threads", 1) for d in threadpoolctl.threadpool_info()), default=1)
    except Exception:  # noqa: BLE001
        blas = os.cpu_count() or 1
    return {
        "value": 1.0 / token_s,
        "unit": UNIT,
        "cores": int(blas),
        "kind": "port",
        "sample": f"one {spec.name} decoder layer (dequant + f32 matmul, N=1) timed {best * 1e3:.0f} ms, "
                  f"x{spec.n_layers} layers + lm_head by weight share; host has {os.cpu_count()} cpus",
        "layer_ms": best * 1e3,
    }


def run_reference(args, spec) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    for _ in range(max(0, args.warmup)):
        cpu_layer_sample(spec)
    times = [cpu_layer_sample(spec) for _ in range(max(1, args.steps))]
    best = max(times, key=lambda d: d["value"])
    line = {
        "impl": "reference",
        "metric": METRIC, "value": best["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / best["value"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": dict(workload_config(spec, args), row_split_exchange="none", prefill="not timed"),
        "cpu_baseline": {k: best[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": best["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def workload_config(spec, args) -> dict:
    return {
        "workload": f"{spec.name} random-init NF4 g64, batch 1, {args.prompt}-token prompt then greedy decode",
        "prompt_tokens": args.prompt, "max_seq": spec.max_seq, "layers": spec.n_layers,
        "weights_gb_per_token": round(spec.packed_bytes_per_token() / 1e9, 3),
        "l2": "inputs larger than L2 (weights streamed once per token)",
        "parallelism": f"tp{args.gpus}",
    }


# --------------------------------------------------------------------------- #
# clocks sampler
# --------------------------------------------------------------------------- #
class Clocks:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index = index
        self.rows: list[list[str]] = []
        self.proc = None
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return

        def pump():
            for line in self.proc.stdout:
                self.rows.append([c.strip() for c in line.split(",")])

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = sorted({n for r in self.rows if len(r) >= 6
                          for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# --------------------------------------------------------------------------- #
# our arm
# --------------------------------------------------------------------------- #
def run_ours(args, spec) -> None:
    import torch

    from gpu.decodev2 import DecodeV2Loop, DeviceWeights
    from gpu.nf4 import nf4_swiglu

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    full_spec = spec
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        import datetime

        dist.init_process_group("nccl", device_id=torch.device("cuda", local),
                                timeout=datetime.timedelta(seconds=180))
    from gpu.decodev2 import Comm, shard_weights

    # every rank draws the same full model (seeded device RNG) and keeps its shard
    comm = Comm.from_env() if world > 1 else None
    weights = DeviceWeights.random_init(spec, seed=0, device=f"cuda:{local}")
    if world > 1:
        weights = shard_weights(weights, rank, world)
        torch.cuda.empty_cache()
    spec = weights.spec
    loop = DecodeV2Loop.from_weights(weights, comm=comm)
    exchange = "none"
    if comm is not None:
        exchange = "nccl" if args.nccl else f"peer memory ({loop.state.enable_peer_exchange()})"
    gen = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, spec.vocab, (args.prompt,), generator=gen).tolist()
    loop.warmup(prompt=8, tokens=4)
    fused_why = loop.enable_fused_step() if args.fused else "default"
    mode = loop.capture_graphs()
    if mode != "decodev2":
        raise SystemExit(f"graph capture failed: {loop.graph_error}")
    step = loop._step()
    state = loop.state

    # prefill (timed apart), leaves next_token ready; one untimed pass first so that
    # lazily loaded kernels and torch's attention setup are not in the timed window. That
    # pass also captures the chunk, and the timed pass replays it (a prompt shape that comes
    # back); --eager-prefill times the Python-issued chunk instead.
    prefill_mode = "eager"
    # measured with the chunk graph at 1 and 2 GPUs; wider groups keep the eager chunk
    # (their NCCL all-reduces inside a captured chunk have not been run on this pool)
    if not args.eager_prefill and (world <= 2 or args.prefill_graphs):
        loop.enable_prefill_graphs()
        prefill_mode = "captured chunk graph, replayed"
    loop.reset()
    loop.prefill_from(prompt, 0)
    loop.reset()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    torch.cuda.synchronize()
    ev[0].record()
    loop.prefill_from(prompt, 0)
    ev[1].record()
    torch.cuda.synchronize()
    prefill_ms = ev[0].elapsed_time(ev[1])
    state.token.copy_(state.next_token)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # device window: K steps back to back
    for _ in range(args.warmup):
        step(state, weights)
    clocks = Clocks(local)
    clocks.start()
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        step(state, weights)
    t1.record()
    barrier()
    dev_ms = t0.elapsed_time(t1)

    # end to end: pinned host token in, picked id out, every step
    host_tok = torch.zeros((), dtype=torch.int64).pin_memory()
    host_tok.copy_(state.token)
    stream = torch.cuda.current_stream()
    for _ in range(args.warmup):
        state.token.copy_(host_tok, non_blocking=True)
        step(state, weights)
        host_tok.copy_(state.token, non_blocking=True)
        stream.synchronize()
    barrier()
    w0 = time.perf_counter()
    t0.record()
    for _ in range(args.steps):
        state.token.copy_(host_tok, non_blocking=True)
        step(state, weights)
        host_tok.copy_(state.token, non_blocking=True)
        stream.synchronize()
    t1.record()
    barrier()
    e2e_ms = max(t0.elapsed_time(t1), (time.perf_counter() - w0) * 1e3)
    clk = clocks.stop()

    # dominant kernel, timed alone over every layer's gate/up (>> L2 in total)
    ar = state.arena
    layers = weights.layers
    g0 = layers[0].gate
    per_launch = 2 * g0.nbytes + g0.K * 2 + g0.M * 2
    reps = max(3, min(20, args.steps))

    def sweep():
        for ly in layers:
            g, u = ly.gate, ly.up
            nf4_swiglu(g.packed, g.scale, u.packed, u.scale, ar.x, g.M, g.K, g.K_pad,
                       ar.down_in.view(-1), ly.norm2, spec.rms_eps)

    for _ in range(3):
        sweep()
    torch.cuda.synchronize()
    # captured, so the figure is device time per launch without Python between launches
    sweep_graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(sweep_graph, stream=side):
            sweep()
    torch.cuda.current_stream().wait_stream(side)
    sweep_graph.replay()
    torch.cuda.synchronize()
    t0.record()
    for _ in range(reps):
        sweep_graph.replay()
    t1.record()
    torch.cuda.synchronize()
    k_us = t0.elapsed_time(t1) * 1e3 / (reps * len(layers))
    peak, peak_kind = measured_peaks()
    achieved = per_launch / (k_us * 1e-6) / 1e9

    times = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device=f"cuda:{local}")
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = (float(t) for t in times.tolist())
    if dist is not None:
        dist.barrier()
    if rank != 0:
        if comm is not None:
            del step, sweep_graph
            comm.shutdown(loop)
        return
    if loop.fused:
        launches_per_step = 1  # the whole step is one persistent kernel
        status = loop._fused.status()
        if status != 0:
            raise SystemExit(f"persistent step reported status {status}")
    else:
        launches_per_step = 1 + spec.n_layers * 5 + 2
    step_bytes = full_spec.packed_bytes_per_token()
    line = {
        "metric": METRIC, "value": args.steps / (dev_ms / 1e3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(full_spec, args),
        "prefill_tok_s": args.prompt / (prefill_ms / 1e3), "prefill_ms": prefill_ms,
        "step_hbm_gbs": step_bytes / (dev_ms / args.steps / 1e3) / 1e9,
        "step_frac_of_hbm_peak": step_bytes / (dev_ms / args.steps / 1e3) / 1e9 / peak,
        "e2e": {"value": args.steps / (e2e_ms / 1e3), "unit": UNIT, "h2d_bytes_per_step": 8,
                "d2h_bytes_per_step": 8},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clk,
    }
    gemv_roof = {"kernel": "nf4_gemv_kernel<swiglu> (gate+up, fused RMSNorm)", "bound": "hbm",
                 "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                 "frac": achieved / peak, "bytes_per_launch": per_launch, "us_per_launch": k_us,
                 "traffic": int(round(per_launch * NCU_TRAFFIC_RATIO)),
                 "traffic_source": "ncu capture of the 3B gate/up launch (24,002,560 B), scaled by "
                                   "algorithmic bytes for other shapes"}
    if loop.fused:
        # one launch = one token: every packed weight byte and scale is read once
        step_us = dev_ms / args.steps * 1e3
        line["roofline"] = {"kernel": "decode_step_kernel (whole greedy step, persistent)",
                            "bound": "hbm", "achieved": step_bytes / (step_us * 1e-6) / 1e9,
                            "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                            "frac": step_bytes / (step_us * 1e-6) / 1e9 / peak,
                            "bytes_per_launch": step_bytes, "us_per_launch": step_us,
                            "traffic": None}
        line["gemv_alone"] = gemv_roof
    else:
        line["roofline"] = gemv_roof
        line["step_mode"] = f"launch chain ({fused_why})"
    line["config"]["row_split_exchange"] = exchange
    line["config"]["prefill"] = prefill_mode
    if not args.no_cpu:
        cb = cpu_layer_sample(full_spec)
        line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line), flush=True)
    if comm is not None:
        del step, sweep_graph
        comm.shutdown(loop)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--model", default="qwen2.5-3b-arch")
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--eager-prefill", action="store_true",
                    help="time the prefill as issued from Python instead of as a replayed chunk graph")
    ap.add_argument("--prefill-graphs", action="store_true",
                    help="replay the prefill chunk as a graph at more than 2 GPUs as well")
    ap.add_argument("--nccl", action="store_true",
                    help="N > 1: sum the row-split partials with NCCL all-reduce launches instead of "
                         "inside the GEMV launch over peer memory")
    ap.add_argument("--fused", action="store_true",
                    help="run the step as one persistent kernel instead of the graph of one launch "
                         "per operation (same bits; slower on the 3B shapes as measured)")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    from gpu.decodev2.arch import CONFIGS

    spec = CONFIGS[args.model]
    if args.impl == "reference":
        run_reference(args, spec)
    else:
        run_ours(args, spec)


if __name__ == "__main__":
    main()
