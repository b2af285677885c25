"""The C-ABI library loads without a GPU and exports what ``include/chr_gpu.h`` declares."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_functions() -> list[str]:
    text = (ROOT / "include" / "chr_gpu.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(chr_nf4_\w+)\s*\(", text)))


def test_header_declares_the_reference_entry_points():
    names = declared_functions()
    for kept in ("chr_nf4_gemm", "chr_nf4_gemm_plan", "chr_nf4_gemm_ws", "chr_nf4_gemm_ws_max",
                 "chr_nf4_set_tuning", "chr_nf4_gemv", "chr_nf4_gemv_qkv", "chr_nf4_gemv_swiglu",
                 "chr_nf4_rope_kv", "chr_nf4_attn", "chr_nf4_rms"):
        assert kept in names


def test_library_exports_every_declared_symbol():
    from gpu.nf4 import _lib

    lib = _lib.load()
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} declared in chr_gpu.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(declared_functions())
    assert _lib.load().chr_nf4_version().decode().startswith("chr_nf4 sm_100a")


def test_struct_layout_is_the_frozen_one():
    from gpu.nf4._lib import ChrNf4Dev, ChrNf4Plan

    assert [f[0] for f in ChrNf4Dev._fields_] == ["M", "K", "K_pad", "packed", "scale"]
    assert ChrNf4Dev.packed.offset == 16 and ChrNf4Dev.scale.offset == 24
    assert ctypes.sizeof(ChrNf4Dev) == 32
    assert ctypes.sizeof(ChrNf4Plan) == 48 and ChrNf4Plan.ws_floats.offset == 40


def test_peer_struct_matches_the_header(tmp_path):
    """sizeof / offsetof of the peer-exchange struct as the C compiler sees it."""
    import subprocess

    from gpu.nf4._lib import AR_MAX_CTAS, AR_MAX_RANKS, ChrNf4Peers

    src = tmp_path / "sz.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "chr_gpu.h"\n'
        'int main(void) { printf("%zu %zu %zu %zu %d %d\\n", sizeof(chr_nf4_peers_t), '
        "offsetof(chr_nf4_peers_t, capacity), offsetof(chr_nf4_peers_t, recv), "
        "offsetof(chr_nf4_peers_t, epoch), CHR_NF4_AR_MAX_RANKS, CHR_NF4_AR_MAX_CTAS); return 0; }\n")
    exe = tmp_path / "sz"
    subprocess.run(["gcc", f"-I{ROOT / 'include'}", str(src), "-o", str(exe)], check=True)
    got = [int(v) for v in subprocess.run([str(exe)], check=True, capture_output=True,
                                          text=True).stdout.split()]
    assert got == [ctypes.sizeof(ChrNf4Peers), ChrNf4Peers.capacity.offset, ChrNf4Peers.recv.offset,
                   ChrNf4Peers.epoch.offset, AR_MAX_RANKS, AR_MAX_CTAS]


@pytest.mark.parametrize("m,k,n", [(2048, 2048, 1), (256, 2048, 1), (11008, 2048, 32),
                                   (2048, 11008, 16), (151936, 2048, 1), (130, 65, 3),
                                   (5120, 27648, 64), (64, 64, 9)])
@pytest.mark.parametrize("have_ws", [True, False])
def test_python_planner_mirrors_the_library(m, k, n, have_ws):
    from gpu.nf4 import nf4_plan, nf4_set_tuning
    from gpu.nf4.plan import ONE_WAVE, plan

    nf4_set_tuning(0, 0, ONE_WAVE)
    try:
        got = nf4_plan(m, k, n, have_ws=have_ws)
    finally:
        nf4_set_tuning(0, 0, 0)
    want = plan(m, k, n, have_ws=have_ws, one_wave=ONE_WAVE).as_dict()
    assert got == want


def test_planner_rejects_bad_arguments():
    from gpu.nf4 import nf4_plan
    from gpu.nf4.plan import plan

    with pytest.raises(RuntimeError, match=r"\(-2\)"):
        nf4_plan(64, 64, 65)
    with pytest.raises(RuntimeError, match=r"\(-4\)"):
        nf4_plan(64, 65, 1, K_pad=64)
    with pytest.raises(RuntimeError, match=r"\(-3\)"):
        nf4_plan(0, 64, 1)
    with pytest.raises(ValueError):
        plan(64, 64, 0)
    with pytest.raises(ValueError):
        plan(64, 65, 1, K_pad=64)
    p = plan(2048, 2048, 16, have_ws=True)
    assert p.ctas == p.grid_x * p.grid_y and p.tiles_per_split * p.grid_y >= p.n_ktiles
    assert p.ws_floats == (p.grid_y * 2048 * 16 if p.grid_y > 1 else 0)


def test_host_codec_matches_oracle_and_reference(golden):
    import nf4_ref as o
    from gpu.host.codec import decode_nf4, encode_nf4

    g = golden("nf4_codec.npz")
    for tag, (m, k) in {"a": (48, 200), "b": (32, 256), "c": (130, 65)}.items():
        p, s = encode_nf4(g[f"{tag}_w"])
        assert np.array_equal(p, g[f"{tag}_packed"])
        assert np.array_equal(s.view(np.uint16), g[f"{tag}_scale"])
        w = decode_nf4(p, s, m, k)
        assert np.array_equal(w.view(np.uint32), g[f"{tag}_what"].view(np.uint32))
    rng = np.random.default_rng(9)
    w = (rng.standard_normal((257, 1000)) * 0.02).astype(np.float32)
    w[3] = 0.0
    w[5, :64] = 1.0e6            # scale overflows binary16 -> clamped like the Go writer
    w[6, :64] = 1.0e-9           # scale underflows -> treated as a zero group
    p, s = encode_nf4(w, threads=3)
    p1, s1 = encode_nf4(w, threads=1)
    assert np.array_equal(p, p1) and np.array_equal(s.view(np.uint16), s1.view(np.uint16))
    po, so = o.quantize(np.delete(w, [5, 6], axis=0))
    keep = np.delete(np.arange(257), [5, 6])
    assert np.array_equal(p[keep], po) and np.array_equal(s[keep].view(np.uint16), so.view(np.uint16))
    assert int(s.view(np.uint16)[5, 0]) == 0x7BFF and int(s.view(np.uint16)[6, 0]) == 0x3C00
    with pytest.raises(ValueError):
        encode_nf4(np.full((1, 64), np.inf, dtype=np.float32))
    with pytest.raises(TypeError):
        encode_nf4(np.zeros((4, 64), dtype=np.float64))


def test_ops_reject_cpu_tensors_before_any_launch():
    import torch

    from gpu.nf4 import nf4_gemm, nf4_gemv, nf4_rms

    packed = torch.zeros((4, 32), dtype=torch.uint8)
    scale = torch.ones((4, 1), dtype=torch.float16)
    x = torch.zeros(64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        nf4_gemv(packed, scale, x, 4, 64, 64)
    with pytest.raises(RuntimeError, match="CUDA"):
        nf4_gemm(packed, scale, x, 4, 64, 64)
    with pytest.raises(RuntimeError, match="CUDA"):
        nf4_rms(x, x, x, 1e-6)
    with pytest.raises(RuntimeError, match="max_n"):
        nf4_gemm(packed, scale, x, 4, 64, 64, max_n=65)


def test_no_entry_point_allocates_device_memory():
    """Source scan of the library for allocation calls (the reference gates its own
    kernels the same way, gpu/tests/oracle_gate.py:558-582): every buffer is the caller's."""
    import re

    banned = re.compile(r"\b(cudaMalloc\w*|cudaHostAlloc|cudaFree\w*|cuMemAlloc\w*|malloc|calloc|realloc)\s*\(")
    hits = []
    for src in sorted((ROOT / "deep-fold_b200" / "csrc").glob("*")):
        if src.suffix not in (".cu", ".cuh", ".cpp", ".h"):
            continue
        if src.name == "codec.cpp":
            continue  # the host-side codec works on host memory only (std::vector / threads)
        for no, line in enumerate(src.read_text().splitlines(), 1):
            code = line.split("//")[0]
            if banned.search(code):
                hits.append(f"{src.name}:{no}: {line.strip()}")
    assert not hits, "\n".join(hits)


def test_the_reference_binding_compiles_against_this_header(tmp_path):
    """gpu/nf4/bindings.cpp of the reference (its torch/pybind layer over the C ABI) must
    build unchanged against include/chr_gpu.h: same structs, entry names and signatures."""
    import os
    import subprocess
    import sysconfig

    sibling = ROOT.parent / "reference"
    where = os.environ.get("DEEPFOLD_REFERENCE") or (str(sibling) if sibling.is_dir() else None)
    src = None if where is None else Path(where) / "gpu" / "nf4" / "bindings.cpp"
    if src is None or not src.is_file():
        pytest.skip("no reference checkout here (DEEPFOLD_REFERENCE): nothing to compile")
    from torch.utils.cpp_extension import include_paths

    # the binding includes "chr_gpu.h" from its own include directory: point that name at ours
    inc = tmp_path / "inc"
    inc.mkdir()
    (inc / "chr_gpu.h").write_text((ROOT / "include" / "chr_gpu.h").read_text())
    cmd = ["g++", "-std=c++17", "-fsyntax-only", "-w", f"-I{inc}",
           f"-I{sysconfig.get_paths()['include']}", "-DTORCH_EXTENSION_NAME=chr_nf4_ext",
           "-DTORCH_API_INCLUDE_EXTENSION_H"]
    cmd += [f"-I{p}" for p in include_paths()]
    cuda_inc = Path("/usr/local/cuda/include")
    if cuda_inc.is_dir():
        cmd.append(f"-I{cuda_inc}")
    res = subprocess.run(cmd + [str(src)], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]


def test_workspace_queries_of_the_wide_gemm_and_the_multi_row_gemv():
    """Host-only arithmetic behind ``chr_nf4_gemm_rows_ws`` and ``chr_nf4_gemv_n_ws`` (no launch;
    without a GPU the planners assume 148 SMs). Split-K is taken where the tile grid alone
    leaves SMs idle and a cut does not just add a second wave; the workspace is
    ``splits * M * N`` floats."""
    from gpu.nf4 import _lib
    from gpu.nf4._lib import ChrNf4Dev

    lib = _lib.load()

    def gemm_ws(m, k, n):
        return int(lib.chr_nf4_gemm_rows_ws(ctypes.byref(ChrNf4Dev(m, k, k, 1, 1)), n))

    # stacked 32B gate/up: 432 row tiles fill the device, no split at any N
    for n in (16, 512, 4096):
        assert gemm_ws(55296, 5120, n) == 0
    # 32B down-proj at the chunk width: 80 CTAs on 148 SMs -> cut K, but not in two
    # (160 CTAs would be two waves of half the work each)
    ws = gemm_ws(5120, 27648, 512)
    assert ws > 0 and ws % (5120 * 512) == 0
    splits = ws // (5120 * 512)
    assert 3 <= splits <= 16
    # a short K is not worth a reduction pass at wide N
    assert gemm_ws(5120, 5120, 512) == 0
    # one decode-sized row block of a long-K matrix: many splits, each at least 8 K tiles
    ws16 = gemm_ws(5120, 27648, 16)
    assert ws16 % (5120 * 16) == 0 and 4 <= ws16 // (5120 * 16) <= 16

    def gemv_n_ws(m, k, n):
        return int(lib.chr_nf4_gemv_n_ws(ctypes.byref(ChrNf4Dev(m, k, k, 1, 1)), n))

    assert gemv_n_ws(2048, 5120, 4) == 0               # 5 chunks of 1024: one K slice
    assert gemv_n_ws(2048, 11264, 8) == 0              # 11 chunks: still one
    assert gemv_n_ws(64, 27648, 8) == 3 * 4 * 64       # 27 chunks -> 3 slices, 4 rows per pass
    assert gemv_n_ws(64, 27648, 3) == 3 * 3 * 64
    assert gemv_n_ws(64, 27648, 9) == 0                # more than 8 rows: refused (no workspace)
