"""The CPU oracle against the reference's golden vectors and recorded outputs."""

from __future__ import annotations

import numpy as np
import pytest

import nf4_ref as o


def test_selfcheck_all_green():
    res = o.selfcheck()
    assert all(res.values()), [k for k, v in res.items() if not v]


@pytest.mark.parametrize("tag,m,k", [("a", 48, 200), ("b", 32, 256), ("c", 130, 65)])
def test_codec_matches_reference_outputs(golden, tag, m, k):
    g = golden("nf4_codec.npz")
    packed, scale = o.quantize(g[f"{tag}_w"])
    assert np.array_equal(packed, g[f"{tag}_packed"])
    assert np.array_equal(scale.view(np.uint16), g[f"{tag}_scale"])
    w_hat = o.dequantize(packed, scale, m, k)
    assert np.array_equal(w_hat.view(np.uint32), g[f"{tag}_what"].view(np.uint32))
    y = o.matmul(w_hat, g[f"{tag}_x"])
    np.testing.assert_allclose(y, g[f"{tag}_y"], rtol=0, atol=1e-6)


def test_toy_blobs_and_pad_garbage(golden):
    g = golden("nf4_codec.npz")
    packed, scale = o.random_blobs(130, 65, 5, pad_garbage=True)
    assert np.array_equal(packed, g["toy_packed"])
    assert np.array_equal(scale.view(np.uint16), g["toy_scale"])
    assert np.array_equal(
        o.dequantize(packed, scale, 130, 65).view(np.uint32), g["toy_what"].view(np.uint32)
    )


def test_quantize_equals_bruteforce_on_midpoints():
    u = np.concatenate(
        [o.MID, np.nextafter(o.MID, np.float32(2)), np.nextafter(o.MID, np.float32(-2)), o.LUT]
    ).astype(np.float32)
    w = np.zeros((2, 64), dtype=np.float32)
    w[0, : len(u)] = u
    w[0, 63] = 1.0
    w[1] = np.random.default_rng(0).standard_normal(64).astype(np.float32)
    a, b = o.quantize(w), o.quantize_l2(w)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1].view(np.uint16), b[1].view(np.uint16))


def test_quantize_rejects_non_finite_and_zero_rows():
    with pytest.raises(ValueError):
        o.quantize(np.array([[np.nan] * 64], dtype=np.float32))
    p, s = o.quantize(np.zeros((3, 70), dtype=np.float32))
    assert (p == 0x77).all() and (s.view(np.uint16) == 0x3C00).all()
    with pytest.raises(ValueError):
        o.quantize(np.full((1, 64), 1e6, dtype=np.float32))
    p, s = o.quantize(np.full((1, 64), 1e6, dtype=np.float32), clamp_scale=True)
    assert int(s.view(np.uint16)[0, 0]) == 0x7BFF and (p == 0xFF).all()


def test_idempotent_reencode():
    rng = np.random.default_rng(4)
    w = (rng.standard_normal((16, 192)) * 0.02).astype(np.float32)
    p, s = o.quantize(w)
    p2, s2 = o.quantize(o.dequantize(p, s, 16, 192))
    assert np.array_equal(p, p2) and np.array_equal(s.view(np.uint16), s2.view(np.uint16))


def test_embed_rows_match_reference(golden):
    g = golden("embed_rows.npz")
    rows = o.embed_rows(g["packed"], g["scale"].view(np.float16), g["ids"], 200)
    assert np.array_equal(rows, g["rows_bf16_bits"])


def test_bf16_round_is_rne():
    import torch

    a = np.random.default_rng(1).standard_normal(4096).astype(np.float32)
    a[:4] = [0.0, -0.0, 1.0 + 2**-8, 1.0 + 3 * 2**-8]
    want = torch.from_numpy(a).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(o.bf16_round(a).view(np.uint32), want.view(np.uint32))
