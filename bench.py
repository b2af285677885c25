"""Benchmark of the NF4 decode/prefill path: batch-1 greedy decode tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--model qwen2.5-32b-arch] [--prompt T] [--chunk 512] [--batch B[,B...]]
                    [--prefill-sweep T[,T...]] [--breakdown] [--nccl] [--no-cpu]

One JSON line on stdout. A "step" is one greedy decode token (one replay of the
captured step graph) of the named random-init architecture after a prompt that
fills the context (default: the Qwen2.5-32B architecture; the prompt length is the
context minus the room the warm-up and the timed windows need, at most 1792 tokens, so
the 128 timed steps run against a ~2k-token KV cache). ``value`` is the
device-window rate (tokens resident, no host traffic), ``e2e`` the rate with a
pinned-host token id copied in and the picked id read back every step.
``roofline`` times the dominant kernel (fused SwiGLU GEMV over the layers'
gate/up matrices, far larger than L2 in total) with CUDA events in this same
process; ``gemm_roofline`` does the same for the prefill GEMM (stacked gate/up at
one prompt chunk); ``cpu_baseline`` times the CPU oracle (numpy dequant + float32
matmul, the reference's CPU NF4 path restated) on the 4096 x 4096 layer at N = 1
and N = 32, dequant and matmul apart, median of 5. ``--impl reference`` runs only
the CPU path: each step is a bounded sample (a slab of one gate matrix) that is
really timed, and the tokens/s it prints is that time scaled by the model's
weight count. ``--batch`` decodes B sequences together (one line per size),
``--prefill-sweep`` times the chunked prefill per prompt length, ``--breakdown`` adds
the per-layer time of every operation kind; under ``torch.distributed.run`` the model is
tensor-parallel over the ranks, ``exchange_us`` is the cost of the exchange fused into
the row-split linears, and the ranks' first ids must agree.
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
FALLBACK_TFLOPS = 1590.0
# dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic bytes of one launch
# of the timed SwiGLU GEMV, from the ncu capture of the 32B gate/up launch summarised in
# profiles/nf4_gemv_swiglu_32b_gate_up.md (150.46 MB read + 3.7-4.4 MB written for
# 150.47 MB): other models' launches are scaled by their algorithmic bytes.
NCU_TRAFFIC_RATIO = 1.027


def measured_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            d = json.loads(path.read_text())
            return {"hbm": float(d["hbm_gbs"]), "tf_burst": float(d["bf16_tflops"]),
                    "tf_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    "kind": "measured"}
        except (KeyError, ValueError):
            pass
    return {"hbm": FALLBACK_HBM_GBS, "tf_burst": FALLBACK_TFLOPS, "tf_sustained": 1400.0,
            "kind": "fallback"}


def blas_threads() -> int:
    try:
        import threadpoolctl

        return max((d.get("num_threads", 1) for d in threadpoolctl.threadpool_info()), default=1)
    except Exception:  # noqa: BLE001
        return os.cpu_count() or 1


# --------------------------------------------------------------------------- #
# CPU legs: numpy dequant + float32 matmul (the reference's CPU NF4 path restated)
# --------------------------------------------------------------------------- #
def cpu_config1(repeats: int = 5) -> dict:
    """The 4096 x 4096 layer at N = 1 and N = 32: dequantize and matmul timed apart,
    median of ``repeats`` (protocol of the reference's CPU oracle, gpu/tests/nf4_oracle.py:119-142)."""
    import numpy as np

    import nf4_ref as o

    m = k = 4096
    p, s = o.random_blobs(m, k, 0, pad_garbage=False)
    rng = np.random.default_rng(1)
    out = {"shape": [m, k], "cpu_count": os.cpu_count(), "blas_threads": blas_threads()}
    med = lambda xs: sorted(xs)[len(xs) // 2]
    t_deq = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        w = o.dequantize(p, s, m, k)
        t_deq.append(time.perf_counter() - t0)
    out["dequant_ms"] = med(t_deq) * 1e3
    for n in (1, 32):
        x = rng.standard_normal((k, n)).astype(np.float32)
        t_mm = []
        for _ in range(repeats):
            t0 = time.perf_counter()
            o.matmul(w, x)
            t_mm.append(time.perf_counter() - t0)
        out[f"matmul_n{n}_ms"] = med(t_mm) * 1e3
    return out


def cpu_sample(spec, rows: int = 8192, seed: int = 0):
    """One bounded sample of the decode workload on the CPU: the first ``rows`` rows of a
    gate matrix ([rows, hidden]) dequantized and multiplied with one activation vector.
    Returns a closure that runs it and the number of weights it covers."""
    import numpy as np

    import nf4_ref as o

    m, k = min(rows, spec.intermediate), spec.hidden
    p, s = o.random_blobs(m, k, seed, pad_garbage=False)
    x = np.random.default_rng(seed).standard_normal((k, 1)).astype(np.float32)

    def run() -> float:
        t0 = time.perf_counter()
        o.matmul(o.dequantize(p, s, m, k), x)
        return time.perf_counter() - t0

    return run, m * k


def model_weights(spec) -> int:
    shapes = spec.linear_shapes()
    layer = sum(m * k for name, (m, k) in shapes.items() if name != "lm_head")
    return spec.n_layers * layer + shapes["lm_head"][0] * shapes["lm_head"][1]


def cpu_baseline(spec, samples: int = 5) -> dict:
    run, n_weights = cpu_sample(spec)
    run()
    times = sorted(run() for _ in range(samples))
    med = times[len(times) // 2]
    token_s = med * model_weights(spec) / n_weights
    return {
        "value": 1.0 / token_s, "unit": UNIT, "cores": int(blas_threads()), "kind": "port",
        "sample": f"{n_weights / 1e6:.0f} M weights of a {spec.name} gate matrix (numpy dequant + f32 "
                  f"matmul, N=1), median of {samples}: {med * 1e3:.0f} ms, scaled by the model's "
                  f"{model_weights(spec) / 1e9:.2f} G weights; host has {os.cpu_count()} cpus",
        "sample_ms": med * 1e3,
        "config1": cpu_config1(),
    }


def run_reference(args, spec) -> None:
    """The CPU arm: every step is one really timed sample; value scales it to a token."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    run, n_weights = cpu_sample(spec)
    for _ in range(max(1, args.warmup)):
        run()
    t0 = time.perf_counter()
    for _ in range(max(1, args.steps)):
        run()
    per_sample = (time.perf_counter() - t0) / max(1, args.steps)
    token_s = per_sample * model_weights(spec) / n_weights
    value = 1.0 / token_s
    line = {
        "impl": "reference",
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_sample * 1e3,
        "step_is": "one bounded sample, not one token (see cpu_baseline.sample)",
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(spec, args),
        "cpu_baseline": {
            "value": value, "unit": UNIT, "cores": int(blas_threads()), "kind": "port",
            "sample": f"each step: {n_weights / 1e6:.0f} M weights of a {spec.name} gate matrix, numpy "
                      f"dequant + f32 matmul at N=1 ({per_sample * 1e3:.0f} ms measured); tokens/s = "
                      f"1 / (that x {model_weights(spec) / n_weights:.0f}, the model's weight count "
                      f"over the sample's); host has {os.cpu_count()} cpus",
        },
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def workload_config(spec, args) -> dict:
    return {
        "workload": f"{spec.name} random-init NF4 g64, batch {args.batch}, {args.prompt}-token prompt "
                    f"then greedy decode",
        "prompt_tokens": args.prompt, "max_seq": spec.max_seq, "layers": spec.n_layers,
        "batch": args.batch,
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


def graph_timed(fn, reps: int, torch) -> float:
    """Milliseconds of one call of ``fn`` when captured in a CUDA graph and replayed
    ``reps`` times back to back (device time, no Python between the launches)."""
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(reps):
        graph.replay()
    t1.record()
    torch.cuda.synchronize()
    del graph
    return t0.elapsed_time(t1) / reps


# --------------------------------------------------------------------------- #
# our arm
# --------------------------------------------------------------------------- #
def run_ours(args, spec) -> None:
    import torch

    from gpu.decodev2 import DecodeV2Loop, DeviceWeights
    from gpu.nf4 import _lib, nf4_gemm_rows, nf4_swiglu

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    full_spec = spec
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import datetime

        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local),
                                timeout=datetime.timedelta(seconds=300))
    from gpu.decodev2 import Comm, shard_weights

    # every rank draws the same full model (seeded device RNG) and keeps its shard
    comm = Comm.from_env() if world > 1 else None
    weights = DeviceWeights.random_init(spec, seed=0, device=f"cuda:{local}")
    if world > 1:
        weights = shard_weights(weights, rank, world)
        torch.cuda.empty_cache()
    spec = weights.spec
    if args.batches != [1]:
        if world > 1:
            raise SystemExit("--batch > 1 runs on one GPU")
        for b in args.batches:
            args.batch = b
            run_batched(args, spec, weights, local)
            torch.cuda.empty_cache()
        return
    if args.prefill_sweep:
        return run_prefill_sweep(args, spec, full_spec, weights, comm, rank, world)
    loop = DecodeV2Loop.from_weights(weights, comm=comm)
    exchange = "none"
    if comm is not None:
        exchange = "nccl" if args.nccl else f"peer memory ({loop.state.enable_peer_exchange()})"
    gen = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, spec.vocab, (args.prompt,), generator=gen).tolist()
    loop.warmup(prompt=8, tokens=4)
    mode = loop.capture_graphs()
    if mode != "decodev2":
        raise SystemExit(f"graph capture failed: {loop.graph_error}")
    step = loop._step()
    state = loop.state

    # prefill (timed apart), leaves next_token ready; one untimed pass first so that
    # lazily loaded kernels are not in the timed window. Issued from Python at every N
    # unless --prefill-graphs asks for the captured chunk.
    prefill_mode = f"eager, chunks of {args.chunk}"
    if args.prefill_graphs:
        loop.enable_prefill_graphs()
        prefill_mode = f"captured chunk graphs, replayed, chunks of {args.chunk}"
    loop.reset()
    loop.prefill_from(prompt, 0, chunk=args.chunk)
    loop.reset()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    torch.cuda.synchronize()
    ev[0].record()
    loop.prefill_from(prompt, 0, chunk=args.chunk)
    ev[1].record()
    torch.cuda.synchronize()
    prefill_ms = ev[0].elapsed_time(ev[1])
    state.token.copy_(state.next_token)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def check_status(where: str) -> None:
        st = _lib.load().chr_nf4_gemv_status()
        if st != 0:
            raise SystemExit(f"{where}: GEMV status {st}")
        for px in (state.peers, state.pick_peers):
            if px is not None and px.timed_out():
                raise SystemExit(f"{where}: a wait for a peer GPU ran out; the results are not trustworthy")

    # the first ids of the run, read once: the same at every N when tensor parallelism
    # is correct (and the same on every rank)
    head_n = min(16, args.steps)
    head = torch.zeros(head_n, dtype=torch.int64, device=f"cuda:{local}")
    snap = {"token": state.token.clone(), "position": state.position.clone(),
            "valid_len": state.valid_len.clone()}
    for i in range(head_n):
        step(state, weights)
        head[i].copy_(state.token.view(-1)[0])
    torch.cuda.synchronize()
    greedy_head = [int(t) for t in head.tolist()]
    if dist is not None:
        gathered = [torch.zeros_like(head) for _ in range(world)]
        dist.all_gather(gathered, head)
        for r, other in enumerate(gathered):
            if [int(t) for t in other.tolist()] != greedy_head:
                raise SystemExit(f"rank {r} decoded different ids than rank {rank}")
    check_status("after the first ids")
    state.token.copy_(snap["token"])
    state.position.copy_(snap["position"])
    state.valid_len.copy_(snap["valid_len"])

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
    check_status("after the device window")

    # end to end: pinned host token in, picked id out, every step
    host_tok = torch.zeros(state.token.shape, dtype=torch.int64).pin_memory()
    host_tok.copy_(state.token)
    stream = torch.cuda.current_stream()
    state.position.copy_(snap["position"])
    state.valid_len.copy_(snap["valid_len"])
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
    check_status("after the end-to-end window")

    # dominant kernel, timed alone over every layer's gate/up (>> L2 in total)
    peaks = measured_peaks()
    ar = state.arena
    layers = weights.layers
    g0 = layers[0].gate
    per_launch = 2 * g0.nbytes + g0.K * 2 + g0.M * 2
    reps = max(3, min(10, args.steps))

    def sweep():
        for ly in layers:
            g, u = ly.gate, ly.up
            nf4_swiglu(g.packed, g.scale, u.packed, u.scale, ar.x, g.M, g.K, g.K_pad,
                       ar.down_in.view(-1), ly.norm2, spec.rms_eps)

    k_us = graph_timed(sweep, reps, torch) * 1e3 / len(layers)
    achieved = per_launch / (k_us * 1e-6) / 1e9

    # prefill GEMM: the stacked gate/up matrix of every layer against one prompt chunk
    gu = [ly.gate_up for ly in layers if ly.gate_up is not None]
    gemm_roof = None
    if gu:
        n_tok = args.chunk
        xin = torch.randn(n_tok, gu[0].K, device=f"cuda:{local}").to(torch.bfloat16)
        yout = torch.empty(n_tok, gu[0].M, dtype=torch.bfloat16, device=f"cuda:{local}")

        def gemm_sweep():
            for m in gu:
                nf4_gemm_rows(m.packed, m.scale, xin, m.M, m.K, m.K_pad, out=yout)

        g_ms = graph_timed(gemm_sweep, max(2, reps // 2), torch) / len(gu)
        flops = 2.0 * gu[0].M * gu[0].K * n_tok
        tf = flops / (g_ms * 1e-3) / 1e12
        gemm_roof = {"kernel": "gemm_rows_kernel (tcgen05, stacked gate/up)", "bound": "tensor",
                     "achieved": tf, "peak": peaks["tf_sustained"], "peak_kind": peaks["kind"] +
                     ", sustained (back-to-back launches inside a long sweep)",
                     "peak_burst": peaks["tf_burst"], "unit": "TFLOP/s",
                     "frac": tf / peaks["tf_sustained"], "frac_of_burst": tf / peaks["tf_burst"],
                     "frac_of_nominal_2250": tf / 2250.0,
                     "shape": [gu[0].M, gu[0].K, n_tok], "us_per_launch": g_ms * 1e3, "traffic": None}
        del xin, yout

    # where the step's time goes: every operation kind swept over all layers as its own
    # captured graph (collective under tensor parallelism: all ranks run the same sweeps)
    breakdown = None
    if args.breakdown:
        from gpu.decodev2 import step as stepmod
        from gpu.nf4 import ATTN_SPLIT, nf4_attn

        def per_layer(fn):
            def run():
                for li, ly in enumerate(layers):
                    fn(li, ly)
            return graph_timed(run, 3, torch) * 1e3 / len(layers)

        state.position.copy_(snap["position"])
        state.valid_len.copy_(snap["valid_len"])
        head = weights.lm_head
        breakdown = {
            "qkv": per_layer(lambda li, ly: stepmod._qkv(state, ly)),
            "attention": per_layer(lambda li, ly: nf4_attn(
                ar.q, state.kv.k[li], state.kv.v[li], ar.attn, state.valid_len, spec.attn_scale,
                ar.attn_ws, ATTN_SPLIT, ar.k, ar.v, state.cos, state.sin, state.position)),
            "o_proj(+exchange)": per_layer(lambda li, ly: stepmod._accumulate(state, ly.o, ar.attn, ar.x)),
            "gate_up_swiglu": k_us,
            "down_proj(+exchange)": per_layer(
                lambda li, ly: stepmod._accumulate(state, ly.down, ar.down_in, ar.x)),
        }
        breakdown["per_layer_sum"] = sum(breakdown.values())
        breakdown["layers_ms"] = breakdown["per_layer_sum"] * len(layers) / 1e3
        breakdown["unit"] = "us per launch (layers_ms: all layers, ms)"
        check_status("after the breakdown sweeps")

    # cost of the exchange fused into the row-split linears: the fused launch minus the
    # partial-only launch of the same shard, swept over all layers (collective: every
    # rank runs both sweeps)
    exchange_us = None
    if spec.tp > 1 and state.peers is not None:
        from gpu.decodev2 import step as stepmod
        from gpu.nf4 import nf4_gemv_f32

        def sweep_of(fn):
            def run():
                for ly in layers:
                    fn(ly)
            return graph_timed(run, 3, torch) * 1e3 / len(layers)

        exchange_us = {}
        for name, pick, src in (("o_proj", lambda ly: ly.o, ar.attn), ("down_proj", lambda ly: ly.down, ar.down_in)):
            fused = sweep_of(lambda ly: stepmod._accumulate(state, pick(ly), src, ar.x))
            alone = sweep_of(lambda ly: nf4_gemv_f32(pick(ly).packed, pick(ly).scale, src.reshape(pick(ly).K),
                                                    pick(ly).M, pick(ly).K, pick(ly).K_pad, ar.partial,
                                                    pick(ly).bias))
            exchange_us[name] = {"fused": fused, "partial_only": alone, "exchange": fused - alone}
        check_status("after the exchange sweeps")

    times = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device=f"cuda:{local}")
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = (float(t) for t in times.tolist())
    if dist is not None:
        dist.barrier()
    if rank != 0:
        if comm is not None:
            del step
            comm.shutdown(loop)
        return
    launches_per_step = 1 + spec.n_layers * 5 + 2
    step_bytes = full_spec.packed_bytes_per_token()
    tokens = args.steps * args.batch
    line = {
        "metric": METRIC if args.batch == 1 else f"decode_tok_s_bs{args.batch}",
        "value": tokens / (dev_ms / 1e3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(full_spec, args),
        "prefill_tok_s": args.prompt / (prefill_ms / 1e3), "prefill_ms": prefill_ms,
        "step_hbm_gbs": step_bytes / (dev_ms / args.steps / 1e3) / 1e9,
        "step_frac_of_hbm_peak": step_bytes / (dev_ms / args.steps / 1e3) / 1e9 / peaks["hbm"],
        "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": UNIT,
                "h2d_bytes_per_step": 8 * args.batch, "d2h_bytes_per_step": 8 * args.batch},
        "gpu_launches": launches_per_step * args.steps,
        "greedy_ids_head": greedy_head,
        "clocks": clk,
    }
    line["roofline"] = {"kernel": "nf4_gemv_kernel<swiglu> (gate+up, fused RMSNorm)", "bound": "hbm",
                        "achieved": achieved, "peak": peaks["hbm"], "peak_kind": peaks["kind"],
                        "unit": "GB/s", "frac": achieved / peaks["hbm"],
                        "frac_of_nominal_8tbs": achieved / 8000.0,
                        "bytes_per_launch": per_launch, "us_per_launch": k_us,
                        "traffic": int(round(per_launch * NCU_TRAFFIC_RATIO)),
                        "traffic_source": "ncu capture of one 32B gate/up launch "
                                          "(profiles/nf4_gemv_swiglu_32b_gate_up.md), scaled by algorithmic bytes"}
    if gemm_roof is not None:
        line["gemm_roofline"] = gemm_roof
    if breakdown is not None:
        line["step_breakdown"] = breakdown
    line["step_mode"] = "launch chain in one CUDA graph"
    line["row_split_exchange"] = exchange
    if exchange_us is not None:
        line["exchange_us"] = exchange_us
    line["prefill_mode"] = prefill_mode
    if not args.no_cpu and world == 1:  # the CPU leg belongs to the one-GPU line
        line["cpu_baseline"] = cpu_baseline(full_spec)
    print(json.dumps(line), flush=True)
    if comm is not None:
        del step
        comm.shutdown(loop)


def run_prefill_sweep(args, spec, full_spec, weights, comm, rank: int, world: int) -> None:
    """``--prefill-sweep``: chunked prefill of prompts of the given lengths on one set of
    weights; device time per length (max over ranks), one JSON line."""
    import torch
    import torch.distributed as dist

    from gpu.decodev2 import DecodeV2Loop
    from gpu.nf4 import _lib

    loop = DecodeV2Loop.from_weights(weights, comm=comm)
    gen = torch.Generator().manual_seed(2)
    ids = torch.randint(0, spec.vocab, (max(args.sweep),), generator=gen).tolist()
    loop.reset()
    loop.prefill_from(ids[: min(args.sweep)], 0, chunk=args.chunk)      # lazy kernel loads
    rows = []
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    for n in args.sweep:
        best = None
        for _ in range(2 if n >= 1024 else 3):
            loop.reset()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            ev[0].record()
            loop.prefill_from(ids[:n], 0, chunk=args.chunk)
            ev[1].record()
            torch.cuda.synchronize()
            ms = torch.tensor([ev[0].elapsed_time(ev[1])], dtype=torch.float64, device="cuda")
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            best = float(ms) if best is None else min(best, float(ms))
        rows.append({"tokens": n, "ms": best, "tok_s": n / (best / 1e3),
                     "tflops": 2.0 * full_spec.packed_bytes_per_token() / 0.53125 * n / (best / 1e3) / 1e12})
    if _lib.load().chr_nf4_gemv_status() != 0:
        raise SystemExit("GEMV status word set")
    if rank == 0:
        print(json.dumps({"metric": "prefill_tok_s", "unit": "tok/s", "n_gpus": world,
                          "config": {"workload": f"{full_spec.name} chunked prefill sweep", "chunk": args.chunk,
                                     "parallelism": f"tp{world}", "timing": "best of 2-3, device events, "
                                     "max over ranks"},
                          "prefill_sweep": rows}), flush=True)
    if comm is not None:
        comm.shutdown(loop)


def run_batched(args, spec, weights, local: int) -> None:
    """``--batch B``: B sequences with a prompt each, decoded together (one graph per step)."""
    import torch

    from gpu.decodev2.batch import BatchLoop
    from gpu.nf4 import _lib

    b = args.batch
    loop = BatchLoop(weights, b)
    st = loop.state
    prompts = [torch.randint(0, spec.vocab, (args.prompt,),
                             generator=torch.Generator().manual_seed(2 + i)).tolist() for i in range(b)]
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    if not getattr(args, "prefill_warm", False):
        st.prefill(weights, prompts[:1] * b, chunk=args.chunk)    # untimed pass (lazy kernel loads)
        args.prefill_warm = True
    torch.cuda.synchronize()
    ev[0].record()
    st.prefill(weights, prompts, chunk=args.chunk)
    ev[1].record()
    torch.cuda.synchronize()
    prefill_ms = ev[0].elapsed_time(ev[1])
    loop.capture_graph()
    head_n = min(16, args.steps)
    head = torch.zeros((head_n, b), dtype=torch.int64, device=st.device)
    snap = [t.clone() for t in (st.token, st.position, st.valid_len)]
    for i in range(head_n):
        loop.step()
        head[i].copy_(st.token)
    torch.cuda.synchronize()
    for t, s0 in zip((st.token, st.position, st.valid_len), snap):
        t.copy_(s0)
    for _ in range(args.warmup):
        loop.step()
    clocks = Clocks(local)
    clocks.start()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        loop.step()
    t1.record()
    torch.cuda.synchronize()
    dev_ms = t0.elapsed_time(t1)
    host_tok = torch.zeros(b, dtype=torch.int64).pin_memory()
    host_tok.copy_(st.token)
    for t, s0 in zip((st.position, st.valid_len), snap[1:]):
        t.copy_(s0)
    stream = torch.cuda.current_stream()
    w0 = time.perf_counter()
    t0.record()
    for _ in range(args.steps):
        st.token.copy_(host_tok, non_blocking=True)
        loop.step()
        host_tok.copy_(st.token, non_blocking=True)
        stream.synchronize()
    t1.record()
    torch.cuda.synchronize()
    e2e_ms = max(t0.elapsed_time(t1), (time.perf_counter() - w0) * 1e3)
    clk = clocks.stop()
    if _lib.load().chr_nf4_gemv_status() != 0:
        raise SystemExit("GEMV status word set")
    peaks = measured_peaks()
    step_bytes = spec.packed_bytes_per_token()
    tokens = args.steps * b
    path = "chr_nf4_gemv_n (CUDA cores, FP32 weights)" if b <= 4 else "chr_nf4_gemm_rows (tcgen05)"
    line = {
        "metric": f"decode_tok_s_bs{b}", "value": tokens / (dev_ms / 1e3), "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(spec, args),
        "prefill_tok_s": b * args.prompt / (prefill_ms / 1e3), "prefill_ms": prefill_ms,
        "linears": path,
        "step_hbm_gbs": step_bytes / (dev_ms / args.steps / 1e3) / 1e9,
        "step_frac_of_hbm_peak": step_bytes / (dev_ms / args.steps / 1e3) / 1e9 / peaks["hbm"],
        "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": UNIT, "h2d_bytes_per_step": 8 * b,
                "d2h_bytes_per_step": 8 * b},
        # this library's kernels per step, counted from below: embedding rows, per layer two
        # row norms, four linears, attention, SiLU*up (split-K reductions not counted),
        # final norm, lm_head, one pick
        "gpu_launches": args.steps * (1 + spec.n_layers * 8 + 3),
        "greedy_ids_head": [int(t) for t in head[:, 0].tolist()],
        "clocks": clk,
    }
    print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--model", default="qwen2.5-32b-arch")
    ap.add_argument("--prompt", type=int, default=None,
                    help="prompt tokens (default: fills the context up to the timed steps)")
    ap.add_argument("--chunk", type=int, default=512, help="prefill chunk width")
    ap.add_argument("--batch", default="1",
                    help="sequences decoded together; a comma list runs one line per size on one "
                         "set of weights")
    ap.add_argument("--prefill-sweep", default="",
                    help="comma list of prompt lengths: time the chunked prefill of each and print "
                         "one JSON line with the table (no decode window)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--breakdown", action="store_true",
                    help="also time every operation kind of the step on its own (per-layer sweeps)")
    ap.add_argument("--prefill-graphs", action="store_true",
                    help="replay the prefill chunks as captured graphs instead of issuing them from Python")
    ap.add_argument("--nccl", action="store_true",
                    help="N > 1: sum the row-split partials with NCCL all-reduce launches instead of "
                         "inside the GEMV launch over peer memory")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    args.batches = [int(b) for b in str(args.batch).split(",")]
    args.batch = args.batches[0]
    from gpu.decodev2.arch import CONFIGS, with_max_seq

    spec = CONFIGS[args.model]
    if args.prefill_sweep:
        args.sweep = [int(n) for n in args.prefill_sweep.split(",")]
        spec = with_max_seq(spec, max(spec.max_seq, max(args.sweep) + 64))
    if args.prompt is None:
        # leave room for the first ids, the warm-up and two timed windows
        room = 16 + 2 * (args.warmup + args.steps) + 8
        args.prompt = max(32, min(1792, spec.max_seq - room))
    if args.impl == "reference":
        run_reference(args, spec)
    else:
        run_ours(args, spec)


if __name__ == "__main__":
    main()
