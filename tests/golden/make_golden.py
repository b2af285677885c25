"""Regenerate the golden fixtures in this folder from the reference tree.

Run where the reference checkout is available (it is not needed to *use* the
fixtures):

    python tests/golden/make_golden.py /path/to/deep-fold

Every array written here is an output of the reference's own Python code on
seeded inputs: the NF4 codec and float32 matmul of ``gpu/tests/nf4_oracle.py``,
the synthetic-decoder oracle of ``gpu/decodev2/oracle.py`` on the models
``gpu/decodev2/synth.py`` builds, the embedding row decode of
``gpu/host/embedding.py`` and the RoPE tables of ``gpu/decodev2/rope.py``.
The tests compare this repository's restatements, and through them the CUDA
kernels, against these files.
"""

from __future__ import annotations

import hashlib
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def bf16_as_f32(a: np.ndarray) -> np.ndarray:
    import torch

    return torch.from_numpy(a).to(torch.bfloat16).to(torch.float32).numpy()


def codec(ref) -> None:
    enc, dec, mm, toy = ref.encode_nf4, ref.decode_nf4, ref.matmul_f32, ref.toy_nf4
    out = {}
    for tag, (m, k, n, seed) in {
        "a": (48, 200, 3, 11),     # K tail: 200 -> K_pad 256
        "b": (32, 256, 1, 12),
        "c": (130, 65, 9, 13),     # M and K tails
    }.items():
        rng = np.random.default_rng(seed)
        w = (rng.standard_normal((m, k), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        x = bf16_as_f32(rng.standard_normal((k, n), dtype=np.float32))
        packed, scale = enc(w)
        w_hat = dec(packed, scale, m, k)
        out[f"{tag}_w"] = w
        out[f"{tag}_x"] = x
        out[f"{tag}_packed"] = packed
        out[f"{tag}_scale"] = scale.view(np.uint16)
        out[f"{tag}_what"] = w_hat
        out[f"{tag}_y"] = mm(w_hat, x)
    packed, scale = toy(130, 65, 5, pad_garbage=True)
    out["toy_packed"] = packed
    out["toy_scale"] = scale.view(np.uint16)
    out["toy_what"] = dec(packed, scale, 130, 65)
    np.savez_compressed(HERE / "nf4_codec.npz", **out)


def model_digest(model) -> str:
    h = hashlib.sha256()
    mats = []
    for ly in model.layers:
        mats += [ly.q, ly.k, ly.v, ly.wqkv, ly.o, ly.gate, ly.up, ly.down]
    mats.append(model.lm_head)
    for mat in mats:
        if mat is None:
            continue
        h.update(np.ascontiguousarray(mat.packed).tobytes())
        h.update(np.ascontiguousarray(mat.scale).tobytes())
    for ly in model.layers:
        h.update(ly.norm1.tobytes())
        h.update(ly.norm2.tobytes())
    h.update(model.final_norm.tobytes())
    h.update(np.ascontiguousarray(model.embed).tobytes())
    return h.hexdigest()


def decoder() -> None:
    from gpu.decodev2.oracle import greedy_ids, teacher_logits
    from gpu.decodev2.plan import MEDIUM_LLAMA, TINY_INTERNLM, TINY_LLAMA
    from gpu.decodev2.synth import build

    out = {}
    cases = {
        "tiny_llama_s0_p1357": (TINY_LLAMA, 0, [1, 3, 5, 7]),
        "tiny_llama_s0_p456": (TINY_LLAMA, 0, [4, 5, 6]),
        "tiny_internlm_s1_p1357": (TINY_INTERNLM, 1, [1, 3, 5, 7]),
        "medium_llama_s0_p1357": (MEDIUM_LLAMA, 0, [1, 3, 5, 7]),
    }
    for tag, (spec, seed, prompt) in cases.items():
        model = build(spec, seed)
        out[tag + "_digest"] = np.frombuffer(model_digest(model).encode(), dtype=np.uint8)
        out[tag + "_prompt"] = np.array(prompt, dtype=np.int64)
        out[tag + "_greedy"] = np.array(greedy_ids(model, prompt, 8), dtype=np.int64)
        out[tag + "_teacher"] = teacher_logits(model, prompt)
    np.savez_compressed(HERE / "decodev2_oracle.npz", **out)


def embedding(ref) -> None:
    import torch

    from gpu.host.embedding import dequant_nf4_rows

    packed, scale = ref.toy_nf4(40, 200, 21, pad_garbage=True)
    ids = np.array([0, 39, 7, 7, 13], dtype=np.int64)
    rows = dequant_nf4_rows(
        torch.from_numpy(packed), torch.from_numpy(scale), torch.from_numpy(ids), 200,
        dtype=torch.bfloat16,
    )
    np.savez_compressed(
        HERE / "embed_rows.npz",
        packed=packed,
        scale=scale.view(np.uint16),
        ids=ids,
        rows_bf16_bits=rows.view(torch.int16).numpy().view(np.uint16),
    )


def rope() -> None:
    from gpu.decodev2.rope import apply_rope_numpy, rope_tables_numpy

    cos, sin = rope_tables_numpy(16, 16, 10000.0)
    cos6, sin6 = rope_tables_numpy(8, 128, 1.0e6)
    rng = np.random.default_rng(3)
    t = rng.standard_normal((2, 3, 16), dtype=np.float32)
    np.savez_compressed(
        HERE / "rope.npz",
        cos=cos, sin=sin, cos6=cos6, sin6=sin6, t=t,
        t_rot=apply_rope_numpy(t, cos[4:6], sin[4:6]),
    )


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <reference checkout>")
    root = Path(sys.argv[1]).resolve()
    sys.path.insert(0, str(root))
    import gpu.tests.nf4_oracle as ref

    bad = [c for c in ref.selfcheck() if not c.ok]
    if bad:
        raise SystemExit(f"reference selfcheck failed: {bad}")
    codec(ref)
    decoder()
    embedding(ref)
    rope()
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
