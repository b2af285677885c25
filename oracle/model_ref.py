"""CPU float32 restatement of deep-fold's synthetic-decoder oracle.

TEST INFRASTRUCTURE ONLY: the checker for the greedy-step executor. Nothing in
the shipped package imports it.

Parity is pinned by ``tests/golden/decodev2_*.npz``: token ids and logits that
the reference's own ``gpu/decodev2/oracle.py`` produced for its published
(spec, seed, prompt) triples; the CPU tests compare this module against them.

The model argument is duck-typed: ``spec`` (hidden, n_q, n_kv, head_dim,
n_rep, q_dim, attn_scale, rms_eps, rope_theta, max_seq, family, eos_id,
vocab), ``embed`` float32 [vocab, hidden], ``final_norm``, ``lm_head`` and
``layers`` whose matrices carry ``packed, scale, M, K, bias``.

Reference functions followed:

* ``rms``, ``silu``          -- gpu/decodev2/oracle.py:27-37
* ``linear``                 -- gpu/decodev2/oracle.py:40-48
* ``split_fused_qkv``        -- gpu/decodev2/oracle.py:51-57 (InternLM packing)
* ``attend``                 -- gpu/decodev2/oracle.py:60-82
* ``step_logits``            -- gpu/decodev2/oracle.py:113-138
* ``teacher_logits``         -- gpu/decodev2/oracle.py:141-146
* ``greedy_ids``             -- gpu/decodev2/oracle.py:149-166
* ``rope_tables``, ``rotate``-- gpu/decodev2/rope.py:20-43
"""

from __future__ import annotations

import numpy as np

from nf4_ref import dequantize

_MASKED = np.float32(-1.0e9)


def rope_tables(max_seq: int, head_dim: int, theta: float):
    """cos, sin float32 [max_seq, head_dim], halves duplicated (rotate-half layout)."""
    if head_dim % 2:
        raise ValueError("head_dim must be even")
    idx = np.arange(0, head_dim, 2, dtype=np.float32)
    inv = (1.0 / (np.float32(theta) ** (idx / np.float32(head_dim)))).astype(np.float32)
    ang = np.outer(np.arange(max_seq, dtype=np.float32), inv).astype(np.float32)
    ang = np.concatenate([ang, ang], axis=-1)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def rotate(t: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """t [n, heads, hd]; cos/sin [n, hd]. t*cos + cat(-t_hi, t_lo)*sin."""
    cos = cos[:, None, :]
    sin = sin[:, None, :]
    half = t.shape[-1] // 2
    swapped = np.concatenate((-t[..., half:], t[..., :half]), axis=-1)
    return (t * cos + swapped * sin).astype(np.float32)


def rms(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    v = x.astype(np.float32, copy=False)
    ms = (v * v).mean(axis=-1, keepdims=True)
    return (v * np.reciprocal(np.sqrt(ms + np.float32(eps))) * w.astype(np.float32)).astype(
        np.float32
    )


def silu(x: np.ndarray) -> np.ndarray:
    v = x.astype(np.float32, copy=False)
    return (v * (1.0 / (1.0 + np.exp(-v)))).astype(np.float32)


def linear(mat, x: np.ndarray) -> np.ndarray:
    """x [n, K] float32 -> [n, M] float32 (+ bias)."""
    w = dequantize(mat.packed, mat.scale, mat.M, mat.K)
    y = (w @ np.ascontiguousarray(x.astype(np.float32, copy=False).T)).T
    if getattr(mat, "bias", None) is not None:
        y = y + mat.bias.astype(np.float32)
    return y.astype(np.float32)


def split_fused_qkv(y: np.ndarray, spec):
    n = y.shape[0]
    grouped = y.reshape(n, spec.n_kv, spec.n_rep + 2, spec.head_dim)
    q = grouped[:, :, : spec.n_rep, :].reshape(n, spec.n_q, spec.head_dim)
    return q, grouped[:, :, -2, :], grouped[:, :, -1, :]


def attend(q: np.ndarray, k: np.ndarray, v: np.ndarray, spec, valid: int) -> np.ndarray:
    """q [n, n_q, hd]; k, v [max_seq, n_kv, hd]; slots >= valid are masked out."""
    n = q.shape[0]
    q4 = q.reshape(n, spec.n_kv, spec.n_rep, spec.head_dim)
    k4 = np.broadcast_to(np.transpose(k, (1, 0, 2))[None], (n,) + (k.shape[1], k.shape[0], k.shape[2]))
    v4 = np.broadcast_to(np.transpose(v, (1, 0, 2))[None], k4.shape)
    sc = np.einsum("bhrd,bhtd->bhrt", q4, k4).astype(np.float32)
    sc *= np.float32(spec.attn_scale)
    sc[..., int(valid):] = _MASKED
    sc = sc - sc.max(axis=-1, keepdims=True)
    p = np.exp(sc)
    p /= p.sum(axis=-1, keepdims=True)
    return np.einsum("bhrt,bhtd->bhrd", p, v4).astype(np.float32).reshape(n, spec.q_dim)


class Cache:
    def __init__(self, spec) -> None:
        shape = (spec.n_layers, spec.max_seq, spec.n_kv, spec.head_dim)
        self.k = np.zeros(shape, dtype=np.float32)
        self.v = np.zeros(shape, dtype=np.float32)
        self.pos = 0
        self.cos, self.sin = rope_tables(spec.max_seq, spec.head_dim, spec.rope_theta)


def _qkv(layer, h: np.ndarray, spec):
    if spec.family == "internlm_gqa":
        return split_fused_qkv(linear(layer.wqkv, h), spec)
    n = h.shape[0]
    return (
        linear(layer.q, h).reshape(n, spec.n_q, spec.head_dim),
        linear(layer.k, h).reshape(n, spec.n_kv, spec.head_dim),
        linear(layer.v, h).reshape(n, spec.n_kv, spec.head_dim),
    )


def step_logits(model, cache: Cache, token: int) -> np.ndarray:
    spec = model.spec
    pos = cache.pos
    if pos >= spec.max_seq:
        raise ValueError("position past max_seq")
    x = model.embed[int(token): int(token) + 1].astype(np.float32)
    cos = cache.cos[pos: pos + 1]
    sin = cache.sin[pos: pos + 1]
    for li, layer in enumerate(model.layers):
        h = rms(x, layer.norm1, spec.rms_eps)
        q, k, v = _qkv(layer, h, spec)
        q = rotate(q, cos, sin)
        k = rotate(k, cos, sin)
        cache.k[li, pos] = k[0]
        cache.v[li, pos] = v[0]
        a = attend(q, cache.k[li], cache.v[li], spec, pos + 1)
        x = x + linear(layer.o, a)
        h = rms(x, layer.norm2, spec.rms_eps)
        x = x + linear(layer.down, silu(linear(layer.gate, h)) * linear(layer.up, h))
    out = linear(model.lm_head, rms(x, model.final_norm, spec.rms_eps))[0]
    cache.pos = pos + 1
    return out.astype(np.float32)


def teacher_logits(model, tokens) -> np.ndarray:
    cache = Cache(model.spec)
    rows = [step_logits(model, cache, int(t)) for t in tokens]
    if not rows:
        return np.zeros((0, model.spec.vocab), dtype=np.float32)
    return np.stack(rows)


def greedy_ids(model, prompt, n_new: int) -> list[int]:
    if not len(prompt):
        raise ValueError("prompt must be non-empty")
    cache = Cache(model.spec)
    last = None
    for t in prompt:
        last = step_logits(model, cache, int(t))
    out: list[int] = []
    tok = int(last.argmax())
    for _ in range(int(n_new)):
        out.append(tok)
        if tok == int(model.spec.eos_id):
            break
        last = step_logits(model, cache, tok)
        tok = int(last.argmax())
    return out
