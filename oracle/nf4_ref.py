"""CPU restatement of deep-fold's NF4 group-64 codec and dequant+matmul path.

TEST INFRASTRUCTURE ONLY. This module is the checker the CUDA kernels are
compared against; nothing in the shipped package imports it. Only the test
suite, the smoke entry and the benchmark's CPU-baseline leg may call it.

Parity is pinned: ``selfcheck()`` replays every golden vector the reference
holds for this path (LUT bit patterns, the 64-wide ramp, the 2x64 fixture with
its error caps, the pad-to-64 fixture, the nibble-order pairs and the scale bit
patterns), and ``tests/golden`` holds outputs of the reference's own Python
implementation on seeded inputs which the tests compare bit for bit.

What each function follows in the reference tree:

* ``LUT_BITS``            -- gpu/tests/nf4_oracle.py:42-59, docs/spec/nf4.md:37-54
* ``padded_k``            -- gpu/tests/nf4_oracle.py:84-88
* ``split_nibbles``       -- gpu/tests/nf4_oracle.py:104-116 (low nibble = even k)
* ``dequantize``          -- gpu/tests/nf4_oracle.py:119-135, internal/nf4/nf4.go:85-121
* ``quantize``            -- gpu/tests/nf4_oracle.py:157-187, internal/nf4/nf4.go:129-185,
                             docs/spec/nf4.md:76-106 (step order), :116-132 (midpoints)
* ``matmul``              -- gpu/tests/nf4_oracle.py:138-142
* ``dequantize_bf16``     -- gpu/nf4/nf4_gemm.cu:168-172,319-323 (A operand of the GEMM)
* ``embed_rows``          -- gpu/host/embedding.py:74-107
* ``random_blobs``        -- gpu/tests/nf4_oracle.py:295-319 (toy blobs with pad garbage)
"""

from __future__ import annotations

import struct

import numpy as np

GROUP = 64

# binary32 bit patterns of the sixteen levels; index 7 is +0.0.
LUT_BITS = (
    0xBF800000, 0xBF3239B1, 0xBF066B30, 0xBECA32A0,
    0xBE91A24D, 0xBE3D353F, 0xBDBA7871, 0x00000000,
    0x3DA2FAFF, 0x3E24CAE3, 0x3E7C04DD, 0x3EAD033A,
    0x3EE1A4B8, 0x3F1007AB, 0x3F3913B3, 0x3F800000,
)
LUT = np.array(LUT_BITS, dtype=np.uint32).view(np.float32)

# Midpoints between neighbouring levels, float32((L[j] + L[j+1]) * 0.5).
MID = ((LUT[:-1] + LUT[1:]) * np.float32(0.5)).astype(np.float32)
MID_BITS = (
    0xBF591CD8, 0xBF1C5270, 0xBEEB8480, 0xBEADEA76, 0xBE703CEC,
    0xBE0D38BC, 0xBD3A7871, 0x3D22FAFF, 0x3DF64862, 0x3E5067E0,
    0x3E9582D4, 0x3EC753F9, 0x3F006D04, 0x3F248DAF, 0x3F5C89DA,
)


def padded_k(k: int) -> int:
    if k < 1:
        raise ValueError(f"K must be positive, got {k}")
    return -(-k // GROUP) * GROUP


def blob_shapes(m: int, k: int) -> tuple[tuple[int, int], tuple[int, int]]:
    """Shapes of (packed uint8, scale float16) for a logical [m, k] matrix."""
    if m < 1:
        raise ValueError(f"M must be positive, got {m}")
    kp = padded_k(k)
    return (m, kp // 2), (m, kp // GROUP)


def split_nibbles(packed: np.ndarray) -> np.ndarray:
    """[M, K_pad/2] bytes -> [M, K_pad] codes. Even column sits in the low nibble."""
    if packed.dtype != np.uint8 or packed.ndim != 2:
        raise TypeError("packed must be a 2-D uint8 array")
    codes = np.empty((packed.shape[0], packed.shape[1] * 2), dtype=np.uint8)
    codes[:, 0::2] = packed & 0x0F
    codes[:, 1::2] = packed >> 4
    return codes


def join_nibbles(codes: np.ndarray) -> np.ndarray:
    if codes.dtype != np.uint8 or codes.shape[1] % 2:
        raise TypeError("codes must be uint8 with an even number of columns")
    return (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)


def _check_blobs(packed: np.ndarray, scale: np.ndarray, m: int, k: int) -> int:
    ps, ss = blob_shapes(m, k)
    if packed.shape != ps:
        raise ValueError(f"packed is {packed.shape}, want {ps}")
    if scale.shape != ss:
        raise ValueError(f"scale is {scale.shape}, want {ss}")
    if scale.dtype != np.float16:
        raise TypeError("scale must be IEEE binary16")
    return padded_k(k)


def dequantize(packed: np.ndarray, scale: np.ndarray, m: int, k: int) -> np.ndarray:
    """W_hat[m, k] float32 = float32(LUT[code]) * float32(scale of the code's group)."""
    kp = _check_blobs(packed, scale, m, k)
    w = LUT[split_nibbles(packed)].reshape(m, kp // GROUP, GROUP)
    w = w * scale.astype(np.float32)[:, :, None]
    return np.ascontiguousarray(w.reshape(m, kp)[:, :k])


def bf16_round(a: np.ndarray) -> np.ndarray:
    """float32 -> nearest-even bfloat16, returned widened back to float32."""
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (bits & 0x7FFFFFFF) > 0x7F800000
    rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    rounded = np.where(nan, bits | 0x00400000, rounded) & 0xFFFF0000
    return rounded.astype(np.uint32).view(np.float32)


def bf16_bits(a: np.ndarray) -> np.ndarray:
    return (bf16_round(a).view(np.uint32) >> 16).astype(np.uint16)


def dequantize_bf16(packed: np.ndarray, scale: np.ndarray, m: int, k: int) -> np.ndarray:
    """The tensor-core GEMM's A operand: bf16(LUT * scale), widened to float32."""
    return bf16_round(dequantize(packed, scale, m, k))


def matmul(w_hat: np.ndarray, x: np.ndarray) -> np.ndarray:
    """Y[m, n] = W_hat[m, k] @ x[k, n], float32 in, float32 out."""
    if w_hat.dtype != np.float32 or x.dtype != np.float32:
        raise TypeError("float32 only")
    return w_hat @ x


def quantize(w: np.ndarray, *, clamp_scale: bool = False) -> tuple[np.ndarray, np.ndarray]:
    """float32 [M, K] -> (packed, scale).

    Group max-abs -> binary16 (RNE) -> divide by the widened binary16 -> clip to
    [-1, 1] -> nearest level by squared float32 distance, ties to the lower
    index (see ``_nearest_code``; ``quantize_l2`` is the brute-force form).

    ``clamp_scale`` follows the Go writer (a scale that leaves binary16's
    finite-positive range is clamped to 65504 / 1.0); without it such a group
    raises, as the reference's Python oracle does.
    """
    if w.dtype != np.float32 or w.ndim != 2:
        raise TypeError("quantize wants a 2-D float32 array")
    if not np.isfinite(w).all():
        raise ValueError("non-finite value in quantize input")
    m, k = w.shape
    kp = padded_k(k)
    g = np.zeros((m, kp), dtype=np.float32)
    g[:, :k] = w
    g = g.reshape(m, kp // GROUP, GROUP)
    top = np.abs(g).max(axis=2)
    top = np.where(top == 0, np.float32(1), top).astype(np.float32)
    with np.errstate(over="ignore"):
        s16 = top.astype(np.float16)
    bad = ~np.isfinite(s16) | (s16 <= 0)
    if bad.any():
        if not clamp_scale:
            raise ValueError("group scale is not finite-positive in binary16")
        s16 = np.where(np.isfinite(s16), s16, np.float16(65504.0))
        s16 = np.where(s16 <= 0, np.float16(1.0), s16).astype(np.float16)
    s = s16.astype(np.float32)
    u = np.clip(g / s[:, :, None], np.float32(-1), np.float32(1)).astype(np.float32)
    return join_nibbles(_nearest_code(u).reshape(m, kp)), s16


def _nearest_code(u: np.ndarray) -> np.ndarray:
    """First minimum of float32 (u - L[j])**2 over j, found from three candidates.

    The count of midpoints strictly below u lands on the nearest level or, when
    u sits within rounding of a midpoint, next to it; comparing the squared
    float32 distances of that level and its two neighbours (lowest index wins a
    tie) reproduces the normative 16-way search exactly.
    """
    c = (u[..., None] > MID).sum(axis=-1).astype(np.int64)
    best = np.clip(c - 1, 0, 15)
    d = (u - LUT[best]).astype(np.float32)
    best_d2 = (d * d).astype(np.float32)
    for cand in (c, np.clip(c + 1, 0, 15)):
        d = (u - LUT[cand]).astype(np.float32)
        d2 = (d * d).astype(np.float32)
        take = (d2 < best_d2) | ((d2 == best_d2) & (cand < best))
        best = np.where(take, cand, best)
        best_d2 = np.where(take, d2, best_d2)
    return best.astype(np.uint8)


def quantize_l2(w: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Same as ``quantize`` with the normative squared-distance search (slow)."""
    m, k = w.shape
    kp = padded_k(k)
    g = np.zeros((m, kp), dtype=np.float32)
    g[:, :k] = w
    g = g.reshape(m, kp // GROUP, GROUP)
    top = np.abs(g).max(axis=2)
    top = np.where(top == 0, np.float32(1), top).astype(np.float32)
    s16 = top.astype(np.float16)
    s = s16.astype(np.float32)
    u = np.clip(g / s[:, :, None], np.float32(-1), np.float32(1)).astype(np.float32)
    d = (u[..., None] - LUT).astype(np.float32)
    codes = np.argmin((d * d).astype(np.float32), axis=-1).astype(np.uint8).reshape(m, kp)
    return join_nibbles(codes), s16


def embed_rows(packed: np.ndarray, scale: np.ndarray, ids, k: int) -> np.ndarray:
    """Rows ``ids`` of an NF4 table as bfloat16 bit patterns [n, k] (uint16)."""
    ids = np.asarray(ids, dtype=np.int64).reshape(-1)
    sub_p = packed[ids]
    sub_s = scale[ids]
    w = dequantize(sub_p, sub_s, sub_p.shape[0], k)
    return bf16_bits(w)


def random_blobs(m: int, k: int, seed: int, *, pad_garbage: bool = True):
    """Uniform random codes + weight-like scales; pad columns hold garbage."""
    (_, half), (_, groups) = blob_shapes(m, k)
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 16, size=(m, half * 2), dtype=np.uint8)
    if not pad_garbage and half * 2 > k:
        codes[:, k:] = 7
    scale = rng.uniform(0.012, 0.055, size=(m, groups)).astype(np.float16)
    return join_nibbles(codes), scale


# --------------------------------------------------------------------------- #
# Golden vectors held by the reference for this path
# --------------------------------------------------------------------------- #
RAMP64_HEX = "778788889999A9AAAABABBBBCBCCCCCCDDDDDDDDEDEEEEEEEEEEEEFEFFFFFFFF"
RAMP2_ROW1_HEX = "00001011111121222233434454556676878899AABABBCCCCDDDDEEEEEEFEFFFF"
RAMP2_CAPS = {"rmse": 0.05185, "maxabs": 0.14508, "mae": 0.03980}


def _bits(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", x))[0]


def selfcheck() -> dict[str, bool]:
    """Replay the reference's known-answer tests; every value must be True."""
    out: dict[str, bool] = {}
    out["lut_increasing_and_zero"] = bool(
        (np.diff(LUT) > 0).all() and LUT.view(np.uint32)[7] == 0
    )
    out["midpoint_bits"] = [int(v) for v in MID.view(np.uint32)] == list(MID_BITS)

    pairs = {(7, 15): 0xF7, (15, 7): 0x7F, (3, 12): 0xC3}
    out["nibble_order"] = all(
        int(join_nibbles(np.array([[a, b]], dtype=np.uint8))[0, 0]) == want
        for (a, b), want in pairs.items()
    )

    ramp = (np.arange(64, dtype=np.float32) / np.float32(63)).reshape(1, 64)
    for name, fn in (("", quantize), ("_l2", quantize_l2)):
        p, s = fn(ramp)
        out["ramp64_hex" + name] = p.tobytes().hex().upper() == RAMP64_HEX
        out["ramp64_scale" + name] = int(s.view(np.uint16)[0, 0]) == 0x3C00
        dec = dequantize(p, s, 1, 64)
        out["ramp64_decode_is_lut" + name] = bool(
            (dec.view(np.uint32) == LUT[split_nibbles(p)].view(np.uint32)).all()
        )

    i = np.arange(64, dtype=np.float32)
    two = np.stack([i / np.float32(63), (np.float32(2) * i - np.float32(63)) / np.float32(63)])
    two = two.astype(np.float32)
    p2, s2 = quantize(two)
    out["ramp2_hex"] = (
        p2[0].tobytes().hex().upper() == RAMP64_HEX
        and p2[1].tobytes().hex().upper() == RAMP2_ROW1_HEX
    )
    err = (dequantize(p2, s2, 2, 64) - two).astype(np.float64)
    out["ramp2_error_caps"] = bool(
        np.sqrt((err**2).mean()) <= RAMP2_CAPS["rmse"]
        and np.abs(err).max() <= RAMP2_CAPS["maxabs"]
        and np.abs(err).mean() <= RAMP2_CAPS["mae"]
    )

    p5, s5 = quantize(np.array([[0.0, 1.0]], dtype=np.float32))
    d5 = dequantize(p5, s5, 1, 2)
    out["pad_fixture"] = (
        p5.tobytes().hex().upper() == "F7" + "77" * 31
        and int(s5.view(np.uint16)[0, 0]) == 0x3C00
        and d5.shape == (1, 2)
        and float(d5[0, 0]) == 0.0
        and float(d5[0, 1]) == 1.0
    )

    # group max 1.0 / 2.25 / 0.5 -> binary16 0x3C00 / 0x4080 / 0x3800
    for top, want in ((1.0, 0x3C00), (2.25, 0x4080), (0.5, 0x3800)):
        w = np.zeros((1, 64), dtype=np.float32)
        w[0, 3] = top
        _, s = quantize(w)
        out[f"scale_bits_{want:04X}"] = int(s.view(np.uint16)[0, 0]) == want

    zero_p, zero_s = quantize(np.zeros((1, 64), dtype=np.float32))
    out["zero_group"] = (
        zero_p.tobytes() == b"\x77" * 32 and int(zero_s.view(np.uint16)[0, 0]) == 0x3C00
    )
    return out


if __name__ == "__main__":
    res = selfcheck()
    for key, ok in res.items():
        print(("PASS " if ok else "FAIL ") + key)
    raise SystemExit(0 if all(res.values()) else 1)
