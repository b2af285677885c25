"""Build the oracle's native pieces (checker only; never loaded by the package).

* ``oracle/libnf4_ref_c.so`` from ``oracle/nf4_ref.c`` with gcc.
* ``oracle/_ref/libchr_nf4_ref.so``: the reference's own CUDA kernels
  (``gpu/nf4/nf4_gemv.cu`` and ``gpu/nf4/nf4_gemm.cu``, C ABI of
  ``gpu/include/chr_gpu.h``) compiled for sm_100a straight from the reference
  checkout when it is present. No reference source is copied; only the built
  library lands in ``oracle/_ref`` (git-ignored). Tests load it through ctypes as
  the GPU-side oracle for greedy-token and per-kernel comparisons.
"""

from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
C_LIB = HERE / "libnf4_ref_c.so"
REF_DIR = HERE / "_ref"
REF_LIB = REF_DIR / "libchr_nf4_ref.so"


def _run(cmd: list[str]) -> None:
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")


def build_c() -> Path:
    src = HERE / "nf4_ref.c"
    if not C_LIB.exists() or C_LIB.stat().st_mtime < src.stat().st_mtime:
        _run(["gcc", "-O2", "-ffp-contract=off", "-shared", "-fPIC", "-o", str(C_LIB), str(src), "-lm"])
    return C_LIB


def reference_checkout() -> Path | None:
    """Where the reference's sources are: ``--reference DIR`` on the command line or the
    ``DEEPFOLD_REFERENCE`` environment variable. There is no built-in default."""
    if "--reference" in sys.argv[1:-1]:
        return Path(sys.argv[sys.argv.index("--reference") + 1])
    env = os.environ.get("DEEPFOLD_REFERENCE")
    return Path(env) if env else None


def build_reference_kernels(reference_root: str | os.PathLike | None = None) -> Path | None:
    root = Path(reference_root) if reference_root is not None else reference_checkout()
    if root is None:
        return REF_LIB if REF_LIB.exists() else None
    srcs = [root / "gpu" / "nf4" / "nf4_gemv.cu", root / "gpu" / "nf4" / "nf4_gemm.cu"]
    if not all(s.is_file() for s in srcs):
        return REF_LIB if REF_LIB.exists() else None
    if REF_LIB.exists() and all(REF_LIB.stat().st_mtime >= s.stat().st_mtime for s in srcs):
        return REF_LIB
    REF_DIR.mkdir(exist_ok=True)
    nvcc = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    _run([nvcc, "-O3", "--expt-relaxed-constexpr", "-lineinfo",
          "-gencode", "arch=compute_100a,code=sm_100a",
          f"-I{root / 'gpu' / 'include'}", "-Xcompiler", "-fPIC", "-shared",
          "-o", str(REF_LIB), *map(str, srcs)])
    return REF_LIB


def build(reference_root: str | os.PathLike | None = None) -> list[str]:
    out = [f"built {build_c()}"]
    ref = build_reference_kernels(reference_root)
    out.append(f"reference kernels: {ref}" if ref else "reference kernels: checkout absent, not built")
    return out


if __name__ == "__main__":
    print("\n".join(build()))
    sys.exit(0)
