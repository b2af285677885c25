"""The allocation-free attention entry point against the regular one.

Hosts that cannot allocate device memory (a binding that only forwards pointers,
a plugin shut out of the process's memory pool, code under a no-allocation rule)
call ``chr_nf4_attn_noalloc``; its split partials live in an array built into
the library. This file is collected last on purpose: if the new entry point ever
breaks, a run that stops at the first failure has already run everything else.
The check goes straight through the C ABI, twice in a row, because the built-in
scratch keeps whatever the previous call left in it.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _case(n_q, n_kv, hd, max_seq, pos, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g, device="cuda").to(torch.bfloat16)
    ang = torch.rand(max_seq, hd, generator=g, device="cuda") * 6.28
    return dict(q=rnd(n_q, hd), k=rnd(max_seq, n_kv, hd), v=rnd(max_seq, n_kv, hd),
                k_act=rnd(n_kv, hd), v_act=rnd(n_kv, hd), cos=torch.cos(ang).to(torch.bfloat16),
                sin=torch.sin(ang).to(torch.bfloat16),
                position=torch.tensor(pos, dtype=torch.int64, device="cuda"),
                valid=torch.tensor(pos + 1, dtype=torch.int32, device="cuda"))


def _run(lib, c, n_q, n_kv, hd, max_seq, n_split, static: bool):
    k, v = c["k"].clone(), c["v"].clone()
    out = torch.zeros(n_q * hd, dtype=torch.bfloat16, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    tail = (n_q, n_kv, hd, n_split, ctypes.c_float(hd ** -0.5), stream, _p(c["k_act"]),
            _p(c["v_act"]), _p(c["cos"]), _p(c["sin"]), _p(c["position"]), max_seq)
    if static:
        before = torch.cuda.memory_stats()["allocation.all.allocated"]
        rc = lib.chr_nf4_attn_noalloc(_p(c["q"]), _p(k), _p(v), _p(out), _p(c["valid"]), *tail)
        assert torch.cuda.memory_stats()["allocation.all.allocated"] == before
    else:
        ws = torch.empty(n_q * n_split * (hd + 2), dtype=torch.float32, device="cuda")
        rc = lib.chr_nf4_attn(_p(c["q"]), _p(k), _p(v), _p(out), _p(c["valid"]), _p(ws), *tail)
    assert rc == 0, rc
    torch.cuda.synchronize()
    return out, k, v


def test_noalloc_attention_matches_regular_entry_twice_in_a_row():
    from gpu.nf4 import _lib

    lib = _lib.load()
    shapes = [(16, 2, 128, 2048, 700, 32), (40, 8, 128, 512, 511, 32), (8, 2, 64, 32, 9, 7)]
    for rep in range(2):                       # second pass reuses the dirty built-in scratch
        for i, (n_q, n_kv, hd, max_seq, pos, n_split) in enumerate(shapes):
            c = _case(n_q, n_kv, hd, max_seq, pos, 100 * rep + i)
            got, gk, gv = _run(lib, c, n_q, n_kv, hd, max_seq, n_split, static=True)
            want, wk, wv = _run(lib, c, n_q, n_kv, hd, max_seq, n_split, static=False)
            # same kernel, same inputs: equal to the last bit, well inside the 0.02 the
            # attention tests allow against the CPU oracle
            assert torch.equal(got, want)
            assert torch.equal(gk, wk) and torch.equal(gv, wv)


def test_noalloc_attention_refuses_sizes_beyond_its_scratch():
    from gpu.nf4 import _lib

    lib = _lib.load()
    n_q, n_kv, hd, max_seq = 128, 8, 256, 16       # 128 * 16 * 258 floats > 262144
    c = _case(n_q, n_kv, hd, max_seq, 3, 5)
    out = torch.zeros(n_q * hd, dtype=torch.bfloat16, device="cuda")
    rc = lib.chr_nf4_attn_noalloc(
        _p(c["q"]), _p(c["k"]), _p(c["v"]), _p(out), _p(c["valid"]), n_q, n_kv, hd, 32,
        ctypes.c_float(0.1), None, None, None, None, None, None, max_seq)
    assert rc == -7
    assert float(out.float().abs().max()) == 0.0
