"""CUDA kernels vs the CPU oracle, through the C ABI (ctypes) on the same inputs.

Tolerance for GEMV / GEMM outputs is the one the path's specification states:
max-abs-rel <= 1e-2, i.e. max|y - y_ref| / max|y_ref| (bf16 accumulate-order
tolerance); the reference's own floor (max(0.05, half a bf16 ulp), absolute) is
asserted as well. Integer / byte work (embedding rows, encoder, greedy pick) is
bit-exact.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import model_ref as mr
import nf4_ref as o

pytestmark = pytest.mark.gpu

DEV = "cuda"
REL_TOL = 1e-2
ABS_FLOOR = 0.05


def t_u8(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def bf16_vec(rng, *shape, std=1.0):
    a = (rng.standard_normal(shape) * std).astype(np.float32)
    t = torch.from_numpy(a).to(torch.bfloat16)
    return t.to(DEV), t.to(torch.float32).numpy()


def blobs(m, k, seed, weight_like=True):
    if weight_like:
        rng = np.random.default_rng(seed)
        w = (rng.standard_normal((m, k)) * 0.02).astype(np.float32)
        p, s = o.quantize(w)
    else:
        p, s = o.random_blobs(m, k, seed, pad_garbage=True)
    return p, s, t_u8(p), t_u8(s.view(np.uint16)).view(torch.float16)


def assert_close(got: torch.Tensor, want: np.ndarray, what=""):
    g = got.to(torch.float32).cpu().numpy().reshape(want.shape)
    err = np.abs(g - want).max()
    ref = np.abs(want).max()
    half_ulp = 2.0 ** (np.floor(np.log2(max(ref, 1e-30))) - 8)
    assert err <= REL_TOL * ref + 1e-30, f"{what}: max-abs-rel {err / ref:.3e} > {REL_TOL}"
    assert err <= max(ABS_FLOOR, half_ulp), f"{what}: abs err {err:.4f}"
    cos = float((g * want).sum() / (np.linalg.norm(g) * np.linalg.norm(want) + 1e-30))
    assert cos > 0.999, f"{what}: cosine {cos}"


GEMV_SHAPES = [
    (2048, 2048), (256, 2048), (11008, 2048), (2048, 11008), (5120, 5120), (1024, 5120),
    (5120, 13824), (6144, 16384), (5120, 27648), (130, 65), (7, 64), (1, 4096), (333, 1000),
    (4096, 4096), (64, 30080), (2051, 2752),
]


@pytest.mark.parametrize("m,k", GEMV_SHAPES)
def test_gemv_matches_oracle(m, k):
    from gpu.nf4 import nf4_gemv

    rng = np.random.default_rng(m * 31 + k)
    p, s, pt, st = blobs(m, k, m + k, weight_like=(m * k > 100000))
    xt, xf = bf16_vec(rng, k)
    y = nf4_gemv(pt, st, xt, m, k, o.padded_k(k))
    want = o.dequantize(p, s, m, k).astype(np.float64) @ xf.astype(np.float64)
    assert y.shape == (m, 1) and y.dtype is torch.bfloat16
    assert_close(y, want.astype(np.float32).reshape(m, 1), f"gemv {m}x{k}")
    # repeat is bit-identical
    y2 = nf4_gemv(pt, st, xt, m, k, o.padded_k(k))
    assert torch.equal(y, y2)


def test_gemv_rejects_k_beyond_what_a_cta_stages_and_reports_no_status():
    """x is staged in shared memory beside the lookup table: K up to 30080."""
    from gpu.nf4 import _lib, nf4_gemv

    k = 30144
    p, s, pt, st = blobs(8, k, 5)
    xt = torch.zeros(k, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match=r"\(-3\)"):
        nf4_gemv(pt, st, xt, 8, k, o.padded_k(k))
    assert _lib.load().chr_nf4_gemv_status() == 0


def test_gemv_with_scales_off_the_16_byte_grid():
    """A scale blob that starts 2 bytes past a 16-byte boundary cannot ride the bulk
    copies: the kernel fetches scales from global memory instead, same results."""
    from gpu.nf4 import _lib
    from gpu.nf4._lib import ChrNf4Dev

    m, k = 515, 4096
    rng = np.random.default_rng(77)
    p, s, pt, st = blobs(m, k, 3, weight_like=True)
    xt, xf = bf16_vec(rng, k)
    shifted = torch.empty(st.numel() + 8, dtype=st.dtype, device="cuda")
    off = shifted[1:1 + st.numel()].view(st.shape)
    off.copy_(st)
    assert off.data_ptr() % 16 == 2
    y = torch.empty(m, dtype=torch.bfloat16, device="cuda")
    w = ChrNf4Dev(m, k, o.padded_k(k), pt.data_ptr(), off.data_ptr())
    rc = _lib.load().chr_nf4_gemv(w, xt.data_ptr(), y.data_ptr(),
                                  torch.cuda.current_stream().cuda_stream, None, None, 1e-6)
    assert rc == 0
    want = o.dequantize(p, s, m, k).astype(np.float64) @ xf.astype(np.float64)
    assert_close(y.reshape(m, 1), want.astype(np.float32).reshape(m, 1), "gemv, unaligned scales")
    assert _lib.load().chr_nf4_gemv_status() == 0


def test_gemv_pad_garbage_is_ignored():
    from gpu.nf4 import nf4_gemv

    m, k = 130, 65
    p, s = o.random_blobs(m, k, 5, pad_garbage=True)
    clean = o.split_nibbles(p)
    clean[:, k:] = 7
    p_clean = o.join_nibbles(clean)
    xt, _ = bf16_vec(np.random.default_rng(0), k)
    st = t_u8(s.view(np.uint16)).view(torch.float16)
    a = nf4_gemv(t_u8(p), st, xt, m, k, 128)
    b = nf4_gemv(t_u8(p_clean), st, xt, m, k, 128)
    assert torch.equal(a, b)


def test_gemv_residual_alias_and_out():
    from gpu.nf4 import nf4_gemv

    m, k = 2048, 2048
    rng = np.random.default_rng(3)
    p, s, pt, st = blobs(m, k, 77)
    xt, xf = bf16_vec(rng, k)
    rt, rf = bf16_vec(rng, m)
    dest = rt.clone()
    ret = nf4_gemv(pt, st, xt, m, k, k, dest, dest)
    assert ret.data_ptr() == dest.data_ptr()
    want = o.dequantize(p, s, m, k).astype(np.float64) @ xf.astype(np.float64) + rf
    assert_close(dest, want.astype(np.float32), "gemv+residual")
    # fused residual equals separate add of the un-rounded sum: check against plain gemv + add
    plain = nf4_gemv(pt, st, xt, m, k, k).view(-1).float() + rt.float()
    assert (dest.float() - plain).abs().max().item() <= 2 * 2.0 ** -8 * max(1.0, plain.abs().max().item())


def test_gemv_fused_rms_equals_rms_then_gemv():
    from gpu.nf4 import nf4_gemv, nf4_rms

    m, k = 1024, 2048
    rng = np.random.default_rng(5)
    _, _, pt, st = blobs(m, k, 9)
    xt, _ = bf16_vec(rng, k, std=3.0)
    wt, _ = bf16_vec(rng, k, std=0.5)
    h = torch.empty_like(xt)
    nf4_rms(xt, wt, h, 1e-6)
    a = nf4_gemv(pt, st, h, m, k, k)
    b = nf4_gemv(pt, st, xt, m, k, k, rms_w=wt, rms_eps=1e-6)
    assert torch.equal(a, b)


@pytest.mark.parametrize("n", [64, 2048, 5120, 6144, 1000])
def test_rms_matches_oracle(n):
    from gpu.nf4 import nf4_rms

    rng = np.random.default_rng(n)
    xt, xf = bf16_vec(rng, n, std=2.0)
    wt, wf = bf16_vec(rng, n, std=0.5)
    y = torch.empty_like(xt)
    nf4_rms(xt, wt, y, 1e-6)
    want = mr.rms(xf[None], wf, 1e-6)[0]
    g = y.float().cpu().numpy()
    assert np.abs(g - want).max() <= 2.0 ** -8 * np.abs(want).max() + 1e-6
    ref = torch.nn.functional.rms_norm(xt.float(), (n,), wt.float(), 1e-6)
    assert (y.float() - ref).abs().max().item() <= 2.0 ** -7 * ref.abs().max().item()


@pytest.mark.parametrize("mq,mkv,k,bias", [(2048, 256, 2048, True), (5120, 1024, 5120, True),
                                            (64, 32, 64, False), (512, 128, 512, True),
                                            (96, 40, 200, True)])
def test_qkv_equals_three_gemvs(mq, mkv, k, bias):
    from gpu.nf4 import nf4_gemv, nf4_qkv

    rng = np.random.default_rng(mq + k)
    kp = o.padded_k(k)
    mats = [blobs(m, k, 100 + i, weight_like=False) for i, m in enumerate((mq, mkv, mkv))]
    xt, xf = bf16_vec(rng, k)
    biases = [bf16_vec(rng, m, std=0.02) if bias else (None, None) for m in (mq, mkv, mkv)]
    outs = [torch.empty(m, dtype=torch.bfloat16, device=DEV) for m in (mq, mkv, mkv)]
    nf4_qkv(mats[0][2], mats[0][3], mats[1][2], mats[1][3], mats[2][2], mats[2][3], xt, mq, mkv,
            mkv, k, kp, *outs, biases[0][0], biases[1][0], biases[2][0])
    for (p, s, pt, st), (bt, bf), out, m in zip(mats, biases, outs, (mq, mkv, mkv)):
        want = o.dequantize(p, s, m, k).astype(np.float64) @ xf.astype(np.float64)
        if bf is not None:
            want = want + bf
        assert_close(out, want.astype(np.float32), "qkv")
        single = nf4_gemv(pt, st, xt, m, k, kp, add=bt).view(-1)
        assert (out.float() - single.float()).abs().max().item() <= 1e-3 * max(
            1.0, single.float().abs().max().item())


@pytest.mark.parametrize("m,k", [(11008, 2048), (13824, 5120), (128, 64), (1024, 512),
                                  (16384, 6144), (27648, 5120), (77, 200)])
def test_swiglu_matches_oracle(m, k):
    from gpu.nf4 import nf4_swiglu

    rng = np.random.default_rng(m + 7 * k)
    kp = o.padded_k(k)
    pg, sg, pgt, sgt = blobs(m, k, 11, weight_like=(m * k > 100000))
    pu, su, put, sut = blobs(m, k, 12, weight_like=(m * k > 100000))
    xt, xf = bf16_vec(rng, k)
    out = torch.empty(m, dtype=torch.bfloat16, device=DEV)
    nf4_swiglu(pgt, sgt, put, sut, xt, m, k, kp, out)
    g = o.dequantize(pg, sg, m, k).astype(np.float64) @ xf.astype(np.float64)
    u = o.dequantize(pu, su, m, k).astype(np.float64) @ xf.astype(np.float64)
    want = (g / (1.0 + np.exp(-g))) * u
    assert_close(out, want.astype(np.float32), f"swiglu {m}x{k}")


def _attn_case(n_q, n_kv, hd, max_seq, vl, seed):
    rng = np.random.default_rng(seed)
    qt, qf = bf16_vec(rng, n_q, hd)
    kt, kf = bf16_vec(rng, max_seq, n_kv, hd)
    vt, vf = bf16_vec(rng, max_seq, n_kv, hd)
    return qt, qf, kt, kf, vt, vf


class _Spec:
    def __init__(self, n_q, n_kv, hd):
        self.n_q, self.n_kv, self.head_dim = n_q, n_kv, hd
        self.n_rep = n_q // n_kv
        self.q_dim = n_q * hd
        self.attn_scale = hd ** -0.5


@pytest.mark.parametrize("n_q,n_kv,hd,max_seq,vl", [
    (16, 2, 128, 2048, 513), (40, 8, 128, 1024, 1024), (48, 8, 128, 256, 1), (4, 2, 16, 16, 5),
    (8, 2, 64, 32, 32), (8, 8, 256, 64, 40), (40, 8, 128, 512, 0), (12, 1, 128, 128, 77),
    # the tensor-core form's 128-row tiles: exactly one, one row over, one short of two,
    # many tiles per split, and a group of seven heads
    (40, 8, 128, 256, 128), (40, 8, 128, 256, 129), (7, 1, 64, 300, 255), (16, 2, 32, 4608, 4500),
])
def test_attention_plain_matches_oracle(n_q, n_kv, hd, max_seq, vl):
    from gpu.nf4 import ATTN_SPLIT, nf4_attn

    qt, qf, kt, kf, vt, vf = _attn_case(n_q, n_kv, hd, max_seq, vl, n_q * hd + vl)
    # poison the tail beyond valid_len: it must be ignored
    kt[vl:] = 1.0e4
    vt[vl:] = 1.0e4
    out = torch.zeros(n_q * hd, dtype=torch.bfloat16, device=DEV)
    valid = torch.tensor(vl, dtype=torch.int32, device=DEV)
    nf4_attn(qt, kt, vt, out, valid, hd ** -0.5, None, ATTN_SPLIT)
    if vl == 0:
        assert float(out.float().abs().max()) == 0.0
        return
    want = mr.attend(qf[None], kf, vf, _Spec(n_q, n_kv, hd), vl)[0]
    g = out.float().cpu().numpy()
    assert np.abs(g - want).max() <= 0.02, np.abs(g - want).max()
    # any split count gives the same answer within rounding
    out2 = torch.zeros_like(out)
    nf4_attn(qt, kt, vt, out2, valid, hd ** -0.5, None, 7)
    assert (out.float() - out2.float()).abs().max().item() <= 0.01


@pytest.mark.parametrize("n_q,n_kv,hd,max_seq,pos", [(16, 2, 128, 2048, 512), (40, 8, 128, 64, 0),
                                                      (4, 2, 16, 16, 15), (8, 2, 64, 32, 9),
                                                      # the current row is the last / the first row of a tile
                                                      (40, 8, 128, 256, 127), (40, 8, 128, 256, 128)])
def test_attention_fused_rope_and_cache_write(n_q, n_kv, hd, max_seq, pos):
    from gpu.nf4 import ATTN_SPLIT, nf4_attn, nf4_rope_kv

    rng = np.random.default_rng(pos + hd)
    qt, qf, kt, kf, vt, vf = _attn_case(n_q, n_kv, hd, max_seq, pos, 3 * pos + n_q)
    kat, kaf = bf16_vec(rng, n_kv, hd)
    vat, vaf = bf16_vec(rng, n_kv, hd)
    cos, sin = mr.rope_tables(max_seq, hd, 1.0e6)
    cos_t = torch.from_numpy(cos).to(DEV, torch.bfloat16)
    sin_t = torch.from_numpy(sin).to(DEV, torch.bfloat16)
    cos_b, sin_b = cos_t.float().cpu().numpy(), sin_t.float().cpu().numpy()
    position = torch.tensor(pos, dtype=torch.int64, device=DEV)
    valid = torch.tensor(pos + 1, dtype=torch.int32, device=DEV)
    k_cache, v_cache = kt.clone(), vt.clone()
    out = torch.zeros(n_q * hd, dtype=torch.bfloat16, device=DEV)
    nf4_attn(qt, k_cache, v_cache, out, valid, hd ** -0.5, None, ATTN_SPLIT, kat, vat, cos_t, sin_t,
             position)
    q_rot = mr.rotate(qf[None], cos_b[pos:pos + 1], sin_b[pos:pos + 1])
    k_rot = mr.rotate(kaf[None], cos_b[pos:pos + 1], sin_b[pos:pos + 1])[0]
    kf2, vf2 = kf.copy(), vf.copy()
    kf2[pos], vf2[pos] = k_rot, vaf
    want = mr.attend(q_rot, kf2, vf2, _Spec(n_q, n_kv, hd), pos + 1)[0]
    assert np.abs(out.float().cpu().numpy() - want).max() <= 0.02
    # the cache row holds bf16(rotated k) and v; every other row is untouched
    assert np.array_equal(o.bf16_bits(k_rot), k_cache[pos].view(torch.int16).cpu().numpy().view(np.uint16))
    assert torch.equal(v_cache[pos], vat)
    keep = [t for t in range(max_seq) if t != pos]
    assert torch.equal(k_cache[keep], kt[keep]) and torch.equal(v_cache[keep], vt[keep])
    # standalone rope_kv writes the same row and rotates q/k in place (bf16)
    q2, k2, kc2, vc2 = qt.clone(), kat.clone(), kt.clone(), vt.clone()
    nf4_rope_kv(q2, k2, vat, kc2, vc2, cos_t, sin_t, position)
    assert torch.equal(kc2[pos], k_cache[pos]) and torch.equal(vc2[pos], vat)
    assert np.array_equal(o.bf16_bits(q_rot[0]), q2.view(torch.int16).cpu().numpy().view(np.uint16))


def test_embed_rows_bit_exact(golden):
    from gpu.nf4 import nf4_embed_rows

    g = golden("embed_rows.npz")
    pt = t_u8(g["packed"])
    st = t_u8(g["scale"]).view(torch.float16)
    ids = torch.from_numpy(g["ids"]).to(DEV)
    rows = nf4_embed_rows(pt, st, ids, 40, 200, 256)
    assert np.array_equal(rows.view(torch.int16).cpu().numpy().view(np.uint16), g["rows_bf16_bits"])
    # big table, K multiple of 8, against the oracle; bad id -> zero row + status
    p, s, pt, st = blobs(5000, 6144, 21)
    ids = torch.tensor([0, 4999, 17, 5000, -1], dtype=torch.int64, device=DEV)
    status = torch.zeros((), dtype=torch.int32, device=DEV)
    pos = torch.tensor(41, dtype=torch.int64, device=DEV)
    vl = torch.zeros((), dtype=torch.int32, device=DEV)
    rows = nf4_embed_rows(pt, st, ids, 5000, 6144, 6144, status=status, position=pos, valid_len=vl)
    want = o.embed_rows(p, s, [0, 4999, 17], 6144)
    got = rows.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got[:3], want)
    assert (got[3:] == 0).all() and int(status.item()) == 1 and int(vl.item()) == 42


def test_device_encoder_bit_exact():
    from gpu.host.codec import encode_nf4, encode_nf4_device

    rng = np.random.default_rng(8)
    w = (rng.standard_normal((513, 1000)) * 0.02).astype(np.float32)
    w[4] = 0
    w[9, :64] = 1e6
    w[10, :64] = 1e-9
    u = np.concatenate([o.MID, np.nextafter(o.MID, np.float32(2)), np.nextafter(o.MID, np.float32(-2))])
    w[11, : len(u)] = u
    w[11, 63] = 1.0
    p, s = encode_nf4(w)
    pd, sd = encode_nf4_device(torch.from_numpy(w).to(DEV))
    assert np.array_equal(pd.cpu().numpy(), p)
    assert np.array_equal(sd.view(torch.int16).cpu().numpy().view(np.uint16), s.view(np.uint16))
    with pytest.raises(ValueError):
        encode_nf4_device(torch.full((2, 64), float("nan"), device=DEV))


def test_pick_commit():
    from gpu.nf4 import nf4_pick_commit

    rng = np.random.default_rng(2)
    for n in (32, 1000, 151936):
        logits = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).to(DEV, torch.bfloat16)
        logits[n // 3] = logits.max()          # a tie: lowest index must win
        want = int(torch.argmax(logits.float()).item())
        scratch = torch.zeros(16, dtype=torch.uint8, device=DEV)
        nxt = torch.zeros((), dtype=torch.int64, device=DEV)
        tok = torch.zeros((), dtype=torch.int64, device=DEV)
        pos = torch.tensor(5, dtype=torch.int64, device=DEV)
        fin = torch.zeros((), dtype=torch.uint8, device=DEV)
        nf4_pick_commit(logits, nxt, scratch, tok, pos, fin, eos=want)
        first = int((logits == logits.max()).nonzero()[0].item())
        assert int(nxt.item()) == first == want
        assert int(tok.item()) == want and int(pos.item()) == 6 and int(fin.item()) == 1
        assert int(scratch.sum().item()) == 0
        nf4_pick_commit(logits, nxt, scratch)   # pick only, scratch reusable
        assert int(nxt.item()) == want and int(pos.item()) == 6
    logits = torch.tensor([0.5, float("nan"), 3.0, -0.0, 0.0], dtype=torch.bfloat16, device=DEV)
    nf4_pick_commit(logits, nxt, scratch)
    assert int(nxt.item()) == 1
    logits = torch.tensor([-1.0, -0.0, 0.0, -2.0], dtype=torch.bfloat16, device=DEV)
    nf4_pick_commit(logits, nxt, scratch)
    assert int(nxt.item()) == 1


GEMM_CASES = [(128, 256, 16), (130, 65, 3), (2048, 2048, 32), (256, 2048, 9), (11008, 2048, 17),
              (2048, 11008, 32), (4096, 4096, 32), (4096, 4096, 1), (300, 1000, 33), (512, 512, 64)]


@pytest.mark.parametrize("m,k,n", GEMM_CASES)
def test_gemm_matches_oracle(m, k, n):
    from gpu.nf4 import PLAN_MAX_N, nf4_gemm

    rng = np.random.default_rng(m + k + n)
    p, s, pt, st = blobs(m, k, m * 3 + n, weight_like=(m * k > 100000))
    xt, xf = bf16_vec(rng, k, n)
    y = nf4_gemm(pt, st, xt, m, k, o.padded_k(k), max_n=PLAN_MAX_N if n > 32 else 32)
    assert y.shape == (m, n) and y.dtype is torch.bfloat16
    want = o.dequantize_bf16(p, s, m, k).astype(np.float64) @ xf.astype(np.float64)
    assert_close(y, want.astype(np.float32), f"gemm {m}x{k}x{n}")
    assert torch.equal(y, nf4_gemm(pt, st, xt, m, k, o.padded_k(k), max_n=PLAN_MAX_N if n > 32 else 32))


ROWS_CASES = [(128, 64, 16), (130, 72, 3), (2048, 2048, 512), (300, 1000, 33), (11008, 2048, 300),
              (2048, 11008, 64), (4096, 4096, 1), (512, 512, 257)]


@pytest.mark.parametrize("m,k,n", ROWS_CASES)
def test_gemm_rows_matches_oracle(m, k, n):
    from gpu.nf4 import nf4_gemm_rows, nf4_gemm_status

    rng = np.random.default_rng(m + k + n)
    p, s, pt, st = blobs(m, k, m * 3 + n, weight_like=(m * k > 100000))
    xt, xf = bf16_vec(rng, n, k)
    y = nf4_gemm_rows(pt, st, xt, m, k, o.padded_k(k))
    assert y.shape == (n, m) and y.dtype is torch.bfloat16
    want = xf.astype(np.float64) @ o.dequantize_bf16(p, s, m, k).astype(np.float64).T
    assert_close(y, want.astype(np.float32), f"gemm_rows {m}x{k}x{n}")
    assert torch.equal(y, nf4_gemm_rows(pt, st, xt, m, k, o.padded_k(k)))
    assert nf4_gemm_status() == 0


@pytest.mark.parametrize("m,k,n", [(2048, 2048, 37), (5120, 13824, 64), (300, 1000, 5), (22016, 2048, 512)])
def test_gemm_rows_bias_and_residual_ride_the_epilogue(m, k, n):
    """``chr_nf4_gemm_rows_add``: bias[m] and add[n, m] join the FP32 sum before its one rounding,
    with and without split-K, and with the residual aliasing the output."""
    from gpu.nf4 import nf4_gemm_rows

    rng = np.random.default_rng(m + k + n)
    kp = o.padded_k(k)
    p, s, pt, st = blobs(m, k, 21, weight_like=True)
    xt = torch.from_numpy(rng.standard_normal((n, k)).astype(np.float32)).to(torch.bfloat16).to(DEV)
    bt, bf = bf16_vec(rng, m, std=0.05)
    at, af = bf16_vec(rng, n, m, std=0.5)
    plain = nf4_gemm_rows(pt, st, xt, m, k, kp).float()
    want = plain + bt.float()[None, :] + at.float()
    got = nf4_gemm_rows(pt, st, xt, m, k, kp, bias=bt, add=at)
    # the fused result is the unrounded sum rounded once: within one bf16 ulp of the
    # twice-rounded reference, plus the rounding of `plain` itself
    tol = 2.0 ** -7 * want.abs().max().item()
    assert (got.float() - want).abs().max().item() <= tol
    dest = at.clone()
    nf4_gemm_rows(pt, st, xt, m, k, kp, out=dest, bias=bt, add=dest)
    assert torch.equal(dest, got)


def test_gemm_rows_rejects_unaligned_k():
    from gpu.nf4 import nf4_gemm_rows

    _, _, pt, st = blobs(64, 65, 1, weight_like=False)
    with pytest.raises(RuntimeError, match="K % 8"):
        nf4_gemm_rows(pt, st, torch.zeros((4, 65), dtype=torch.bfloat16, device=DEV), 64, 65, 128)


def test_gemm_no_column_leak_and_pad_garbage():
    from gpu.nf4 import nf4_gemm

    m, k = 130, 65
    p, s = o.random_blobs(m, k, 5, pad_garbage=True)
    st = t_u8(s.view(np.uint16)).view(torch.float16)
    clean = o.split_nibbles(p)
    clean[:, k:] = 7
    rng = np.random.default_rng(1)
    x4, _ = bf16_vec(rng, k, 4)
    x4[:, 3] = 1.0e30                       # a wild extra column must not leak into 0..2
    x3 = x4[:, :3].contiguous()
    y3 = nf4_gemm(t_u8(p), st, x3, m, k, 128)
    y4 = nf4_gemm(t_u8(p), st, x4, m, k, 128)
    assert torch.equal(y3, y4[:, :3].contiguous())
    y3c = nf4_gemm(t_u8(o.join_nibbles(clean)), st, x3, m, k, 128)
    assert torch.equal(y3, y3c)


def test_gemm_split_k_agrees_within_one_ulp():
    from gpu.nf4 import nf4_gemm, nf4_set_tuning

    m, k, n = 512, 4096, 16
    _, _, pt, st = blobs(m, k, 4)
    xt, _ = bf16_vec(np.random.default_rng(6), k, n)
    outs = []
    try:
        for split in (1, 2, 5, 64):
            nf4_set_tuning(0, split, 0)
            outs.append(nf4_gemm(pt, st, xt, m, k, k).float())
    finally:
        nf4_set_tuning(0, 0, 0)
    for y in outs[1:]:
        assert (y - outs[0]).abs().max().item() <= 2.0 ** -7 * outs[0].abs().max().item()


def test_bad_arguments_are_rejected_without_launch():
    from gpu.nf4 import nf4_gemm, nf4_gemv

    _, _, pt, st = blobs(64, 128, 1, weight_like=False)
    x = torch.zeros(128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="packed has"):
        nf4_gemv(pt[:32], st, x, 64, 128, 128)
    with pytest.raises(RuntimeError, match="scale has"):
        nf4_gemm(pt, st[:10], x, 64, 128, 128)
    with pytest.raises(RuntimeError, match="K_pad"):
        nf4_gemv(pt, st, x, 64, 128, 192)
    with pytest.raises(RuntimeError, match="bfloat16"):
        nf4_gemm(pt, st, x.float(), 64, 128, 128)
    with pytest.raises(RuntimeError, match=r"N=40"):
        nf4_gemm(pt, st, torch.zeros((128, 40), dtype=torch.bfloat16, device=DEV), 64, 128, 128)
    with pytest.raises(RuntimeError, match="out too small"):
        nf4_gemv(pt, st, x, 64, 128, 128, out=torch.zeros(8, dtype=torch.bfloat16, device=DEV))
    # misaligned x (offset by one element) is the C ABI's -5
    xx = torch.zeros(129, dtype=torch.bfloat16, device=DEV)[1:]
    with pytest.raises(RuntimeError, match=r"\(-5\)"):
        nf4_gemv(pt, st, xx, 64, 128, 128)
    torch.cuda.synchronize()


def test_nan_does_not_bleed_across_rows():
    from gpu.nf4 import nf4_gemv

    m, k = 256, 512
    _, s, pt, _ = blobs(m, k, 2, weight_like=False)
    s = s.copy()
    s.view(np.uint16)[7, 0] = 0x7E00         # NaN scale in row 7 only
    st = t_u8(s.view(np.uint16)).view(torch.float16)
    xt, _ = bf16_vec(np.random.default_rng(0), k)
    y = nf4_gemv(pt, st, xt, m, k, k).view(-1).float()
    assert torch.isnan(y[7]) and torch.isfinite(torch.cat([y[:7], y[8:]])).all()


def test_prefill_row_kernels_match_the_torch_ops_bit_for_bit():
    import torch.nn.functional as F

    from gpu.decodev2.rope import apply_rope_torch, rope_tables_torch
    from gpu.nf4 import nf4_rms, nf4_rms_rows, nf4_rope_kv_rows, nf4_silu_mul

    gen = torch.Generator(device="cuda").manual_seed(3)
    n, n_q, n_kv, hd, max_seq, start = 37, 8, 2, 64, 96, 11
    wide = torch.randn((n, (n_q + 2 * n_kv) * hd + 8), generator=gen, device="cuda").to(torch.bfloat16)
    q, k, v = wide[:, : n_q * hd], wide[:, n_q * hd:(n_q + n_kv) * hd], wide[:, (n_q + n_kv) * hd:-8]
    cos, sin = rope_tables_torch(max_seq, hd, 10000.0, device="cuda", dtype=torch.bfloat16)
    k_cache = torch.zeros((max_seq, n_kv, hd), dtype=torch.bfloat16, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    q_out = nf4_rope_kv_rows(q, k, v, k_cache, v_cache, cos, sin, start, n_q, n_kv, hd)
    c, s_ = cos[start:start + n], sin[start:start + n]
    assert torch.equal(q_out, apply_rope_torch(q.reshape(n, n_q, hd), c, s_))
    assert torch.equal(k_cache[start:start + n], apply_rope_torch(k.reshape(n, n_kv, hd), c, s_))
    assert torch.equal(v_cache[start:start + n], v.reshape(n, n_kv, hd))
    assert not k_cache[:start].any() and not k_cache[start + n:].any()
    with pytest.raises(RuntimeError):
        nf4_rope_kv_rows(q, k, v, k_cache, v_cache, cos, sin, max_seq - 3, n_q, n_kv, hd)

    inter = 176
    gu = (torch.randn((n, 2 * inter), generator=gen, device="cuda") * 3).to(torch.bfloat16)
    assert torch.equal(nf4_silu_mul(gu, inter), F.silu(gu[:, :inter]) * gu[:, inter:])

    kdim = 520
    x = torch.randn((n, kdim + 8), generator=gen, device="cuda").to(torch.bfloat16)[:, :kdim]
    w = torch.randn(kdim, generator=gen, device="cuda").to(torch.bfloat16)
    y = nf4_rms_rows(x, w, 1e-6)
    for r in (0, 5, n - 1):
        row = torch.empty(kdim, dtype=torch.bfloat16, device="cuda")
        nf4_rms(x[r].contiguous(), w, row, 1e-6)
        assert torch.equal(y[r], row)
    ref = F.rms_norm(x.float(), (kdim,), w.float(), 1e-6)
    assert (y.float() - ref).abs().max() <= 2 ** -7 * ref.abs().max()


PREFILL_ATTN_CASES = [
    # n, start, n_q, n_kv, hd, max_seq
    (37, 11, 8, 2, 64, 96),        # ragged chunk in the middle of the cache
    (1, 0, 4, 4, 16, 8),           # one query, one key, no grouping
    (64, 0, 5, 1, 128, 64),        # exactly one tile, five heads on one kv head
    (130, 200, 10, 2, 128, 512),   # several key tiles before the diagonal one
    (512, 512, 10, 2, 128, 1024),  # the benchmark's chunk width against a 512-row prefix
    (33, 95, 6, 3, 32, 128),       # the chunk ends on the last cache row
]


@pytest.mark.parametrize("n,start,n_q,n_kv,hd,max_seq", PREFILL_ATTN_CASES)
def test_prefill_attention_matches_masked_softmax_in_f32(n, start, n_q, n_kv, hd, max_seq):
    """``chr_nf4_attn_prefill`` against softmax(scale * q k^T + causal mask) v evaluated in
    float32 on the same bf16 inputs (the reference's per-chunk attention,
    gpu/decodev2/prefill.py:50-92). Tolerance: 0.02 of the largest output, the bound the
    model oracle puts on attention."""
    from gpu.nf4 import nf4_attn_prefill

    gen = torch.Generator(device="cuda").manual_seed(n * 131 + start)
    wide = torch.randn((n, n_q * hd + 16), generator=gen, device="cuda").to(torch.bfloat16)
    q = wide[:, : n_q * hd]                     # rows with a stride, as a slice of a GEMM output
    k_cache = torch.randn((max_seq, n_kv, hd), generator=gen, device="cuda").to(torch.bfloat16)
    v_cache = torch.randn((max_seq, n_kv, hd), generator=gen, device="cuda").to(torch.bfloat16)
    # rows past the prefix must not matter, whatever they hold
    k_cache[start + n:] = float("nan")
    v_cache[start + n:] = float("nan")
    scale = hd ** -0.5
    got = nf4_attn_prefill(q, k_cache, v_cache, start, scale).float().reshape(n, n_q, hd)

    seq = start + n
    qf = q.float().reshape(n, n_q, hd)
    kf = k_cache[:seq].float().repeat_interleave(n_q // n_kv, dim=1)
    vf = v_cache[:seq].float().repeat_interleave(n_q // n_kv, dim=1)
    scores = torch.einsum("ihd,thd->hit", qf, kf) * scale
    allowed = torch.arange(seq, device="cuda")[None, :] <= (start + torch.arange(n, device="cuda"))[:, None]
    scores = scores.masked_fill(~allowed[None], float("-inf"))
    want = torch.einsum("hit,thd->ihd", torch.softmax(scores, dim=-1), vf)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() <= 0.02 * want.abs().max()
    # 3-D query tensors take the same path
    again = nf4_attn_prefill(q.reshape(n, n_q, hd).contiguous(), k_cache, v_cache, start, scale)
    assert torch.equal(again.float().reshape(n, n_q, hd), got)


def test_prefill_attention_rejects_what_it_does_not_cover():
    from gpu.nf4 import nf4_attn_prefill

    k = torch.zeros((32, 2, 48), dtype=torch.bfloat16, device="cuda")
    q = torch.zeros((4, 4 * 48), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        nf4_attn_prefill(q, k, k, 0, 0.1)                      # head_dim 48
    k = torch.zeros((32, 2, 64), dtype=torch.bfloat16, device="cuda")
    q = torch.zeros((4, 4 * 64), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        nf4_attn_prefill(q, k, k, 30, 0.1)                     # 30 + 4 rows in a 32-row cache


GEMV_N_CASES = [
    (2048, 2048, 2), (2560, 5120, 3), (1024, 5120, 8), (520, 13824, 4), (300, 27648, 8),
    (6144, 6144, 4), (130, 65, 3), (333, 1000, 8), (64, 16384, 5), (7, 64, 1),
]


@pytest.mark.parametrize("m,k,n", GEMV_N_CASES)
def test_gemv_n_matches_oracle_with_gemv_numerics(m, k, n):
    """N activation rows against the float64 product with FP32-dequantized weights."""
    from gpu.nf4 import nf4_gemv_n

    rng = np.random.default_rng(m * 7 + k + n)
    p, s, pt, st = blobs(m, k, m + k + n, weight_like=(m * k > 100000))
    xt, xf = bf16_vec(rng, n, k)
    bias_t, bias_f = bf16_vec(rng, m, std=0.1)
    add_t, add_f = bf16_vec(rng, n, m, std=0.1)
    w = o.dequantize(p, s, m, k).astype(np.float64)
    y = nf4_gemv_n(pt, st, xt, m, k, o.padded_k(k))
    assert y.shape == (n, m) and y.dtype is torch.bfloat16
    assert_close(y, (xf.astype(np.float64) @ w.T).astype(np.float32), f"gemv_n {m}x{k} N={n}")
    # bias + residual, written in place over the residual; and bit-stable on repeat
    want = (xf.astype(np.float64) @ w.T + bias_f[None, :] + add_f).astype(np.float32)
    buf = add_t.clone()
    nf4_gemv_n(pt, st, xt, m, k, o.padded_k(k), out=buf, add=buf, bias=bias_t)
    assert_close(buf, want, f"gemv_n+bias+add {m}x{k} N={n}")
    buf2 = add_t.clone()
    nf4_gemv_n(pt, st, xt, m, k, o.padded_k(k), out=buf2, add=buf2, bias=bias_t)
    assert torch.equal(buf, buf2)


def test_gemv_n_rows_are_independent_and_track_the_one_row_gemv():
    from gpu.nf4 import nf4_gemv, nf4_gemv_n

    m, k = 1536, 4096
    rng = np.random.default_rng(3)
    p, s, pt, st = blobs(m, k, 9)
    xt, xf = bf16_vec(rng, 4, k)
    y4 = nf4_gemv_n(pt, st, xt, m, k, k)
    # a row does not depend on its neighbours (same row alone, or repeated, gives the same bits)
    y1 = nf4_gemv_n(pt, st, xt[2:3].contiguous(), m, k, k)
    assert torch.equal(y4[2], y1[0])
    rep = nf4_gemv_n(pt, st, xt[1:2].repeat(8, 1).contiguous(), m, k, k)
    assert all(torch.equal(rep[0], rep[i]) for i in range(8)) and torch.equal(rep[0], y4[1])
    # and agrees with the one-row kernel to within the last bf16 place
    g = nf4_gemv(pt, st, xt[0], m, k, k).view(-1).float()
    d = (y4[0].float() - g).abs().max().item()
    assert d <= 2.0 ** -7 * g.abs().max().item()
    # NaN in one row of x stays in that row
    bad = xt.clone()
    bad[3, 17] = float("nan")
    yb = nf4_gemv_n(pt, st, bad, m, k, k)
    assert torch.equal(yb[:3], y4[:3]) and torch.isnan(yb[3].float()).all()


def test_gemv_n_argument_errors():
    from gpu.nf4 import _lib, nf4_gemv_n
    from gpu.nf4._lib import ChrNf4Dev

    p, s, pt, st = blobs(64, 27648, 1, weight_like=False)
    xt = torch.zeros(9, 27648, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        nf4_gemv_n(pt, st, xt, 64, 27648, 27648)          # more than 8 rows
    lib = _lib.load()
    w = ChrNf4Dev(64, 27648, 27648, pt.data_ptr(), st.data_ptr())
    # 27 chunks of 1024 -> 3 K slices of 9; a launch carries at most 4 activation rows
    assert lib.chr_nf4_gemv_n_ws(w, 8) == 3 * 4 * 64
    assert lib.chr_nf4_gemv_n_ws(w, 2) == 3 * 2 * 64
    y = torch.empty(8, 64, dtype=torch.bfloat16, device="cuda")
    rc = lib.chr_nf4_gemv_n(w, xt.data_ptr(), y.data_ptr(), 8, None, None, None, 0, None)
    assert rc == -7                                         # split-K workspace missing
    assert lib.chr_nf4_gemv_n(w, xt.data_ptr(), y.data_ptr(), 9, None, None, None, 0, None) == -2


def test_peer_waits_run_out_and_report_instead_of_hanging():
    """One GPU plays rank 0 of a 2-rank group whose peer never raises its flags: the fused
    GEMV exchange and the split pick both return after their (shortened) poll budget with the
    status word set, and later calls skip the wait until the host clears it."""
    from gpu.nf4 import _lib, nf4_gemv_allreduce, nf4_pick_commit_tp
    from gpu.nf4._lib import AR_MAX_CTAS, ChrNf4Peers

    lib = _lib.load()
    m, k = 512, 2048
    rng = np.random.default_rng(11)
    p, s, pt, st = blobs(m, k, 4)
    xt, xf = bf16_vec(rng, k)

    def peers_for(capacity):
        n_recv = 2 * 2 * capacity * 2      # halves x ranks x rows, 8-byte words, in floats
        bufs = [torch.zeros(n_recv + 2 * AR_MAX_CTAS, dtype=torch.float32, device="cuda")
                for _ in range(2)]
        epoch = torch.zeros(2, dtype=torch.int32, device="cuda")
        status = torch.zeros((), dtype=torch.int32, device="cuda")
        pr = ChrNf4Peers()
        pr.rank, pr.world, pr.capacity = 0, 2, capacity
        for r, b in enumerate(bufs):
            pr.recv[r] = b.data_ptr()
            pr.flags[r] = b.data_ptr() + 4 * n_recv
        pr.epoch, pr.status = epoch.data_ptr(), status.data_ptr()
        return pr, (bufs, epoch, status)

    lib.chr_nf4_set_peer_polls(2000)
    try:
        pr, keep = peers_for(m)
        y = torch.zeros(m, dtype=torch.bfloat16, device="cuda")
        nf4_gemv_allreduce(pt, st, xt, m, k, k, y, pr)
        torch.cuda.synchronize()
        assert int(keep[2].item()) == 1                       # the wait ran out and said so
        # the sum holds this rank's partial (the absent peer's slot is still zero)
        want = o.dequantize(p, s, m, k).astype(np.float64) @ xf.astype(np.float64)
        assert_close(y.reshape(m, 1), want.astype(np.float32).reshape(m, 1), "partial after a timed-out wait")
        nf4_gemv_allreduce(pt, st, xt, m, k, k, y, pr)        # sticky status: no second wait
        torch.cuda.synchronize()
        assert int(keep[2].item()) == 1 and int(keep[1][0].item()) == 2
        # capacity is enforced
        small, keep2 = peers_for(m - 1)
        with pytest.raises(RuntimeError, match=r"\(-7\)"):
            nf4_gemv_allreduce(pt, st, xt, m, k, k, y, small)
        # split pick
        pk, keep3 = peers_for(2)
        logits = torch.randn(4096, device="cuda").to(torch.bfloat16)
        nxt = torch.zeros((), dtype=torch.int64, device="cuda")
        scratch = torch.zeros(16, dtype=torch.uint8, device="cuda")
        nf4_pick_commit_tp(logits, 4096, pk, nxt, scratch)
        torch.cuda.synchronize()
        assert int(keep3[2].item()) == 1
        assert int(nxt.item()) == 4096 + int(logits.float().argmax().item())
    finally:
        lib.chr_nf4_set_peer_polls(0)
    assert lib.chr_nf4_gemv_status() == 0
