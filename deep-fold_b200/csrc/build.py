"""Build ``libchr_nf4.so``: the C-ABI CUDA library for sm_100a.

    python deep-fold_b200/csrc/build.py [--force]

Plain ``nvcc`` invocations, no torch headers: the library's interface is
``include/chr_gpu.h`` only. Objects are compiled in parallel and linked into
``deep-fold_b200/gpu/nf4/libchr_nf4.so`` (git-ignored).
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import os
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
ROOT = CSRC.parents[1]
INCLUDE = ROOT / "include"
OUT_DIR = CSRC.parent / "gpu" / "nf4"
LIB = OUT_DIR / "libchr_nf4.so"
OBJ_DIR = CSRC / "build"

CUDA_SOURCES = ("gemv.cu", "decode_ops.cu", "prefill_ops.cu", "prefill_attn.cu", "gemm.cu", "gemm_tc.cu", "codec_dev.cu",
                "version.cu")
CXX_SOURCES = ("codec.cpp",)
HEADERS = ("nf4_common.cuh", "gemv_ring.cuh", "gemv_cols.cuh", "gemv_n.cuh", "attn_core.cuh", "attn_mma.cuh", "gemm_plan.h")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-ffp-contract=off",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else "nvcc"


def source_digest() -> str:
    h = hashlib.sha256()
    for name in CUDA_SOURCES + CXX_SOURCES + HEADERS:
        h.update((CSRC / name).read_bytes())
    h.update((INCLUDE / "chr_gpu.h").read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:12]


def _compile(src: str, tag: str, verbose: bool) -> Path:
    obj = OBJ_DIR / (src.rsplit(".", 1)[0] + ".o")
    cmd = [_nvcc(), *NVCC_FLAGS, f"-DCHR_BUILD_TAG=\"{tag}\"", f"-I{INCLUDE}", f"-I{CSRC}"]
    if verbose and src.endswith(".cu"):
        cmd += ["-Xptxas", "-v"]
    cmd += ["-c", str(CSRC / src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    tag = source_digest()
    stamp = OBJ_DIR / "stamp.txt"
    if not force and LIB.exists() and stamp.exists() and stamp.read_text().strip() == tag:
        return LIB
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as pool:
        objs = list(pool.map(lambda s: _compile(s, tag, verbose), CUDA_SOURCES + CXX_SOURCES))
    link = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-lpthread"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    stamp.write_text(tag + "\n")
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
