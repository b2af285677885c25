"""Batched greedy decode: ``B`` independent sequences advance together, one set of
weight reads per step.

Not in the reference, whose executor holds one sequence
(gpu/decodev2/state.py:19-107, step.py:162-187); the per-sequence semantics are
kept: every sequence has its own token / position / valid_len / finished
registers and its own ``[max_seq, n_kv, head_dim]`` KV block, and the operation
sequence of a step is the single-sequence one with ``B`` rows: embedding rows ->
per layer [RMSNorm rows, q/k/v linear, attention of B sequences in one launch,
o-proj + residual, RMSNorm rows, gate/up linear, SiLU*up, down-proj + residual]
-> final RMSNorm -> lm_head -> greedy pick + commit of all sequences in one launch.

Linears: up to ``GEMV_ROWS`` (4) sequences run through the CUDA-core multi-row GEMV
(``chr_nf4_gemv_n``: FP32 weights, the numerics of the one-sequence step; one launch
carries four rows for the price of one pass over the weights); larger batches through
the tensor-core GEMM on activation rows (bf16 weight operand, as in prefill), whose
pass over the weights costs less than two GEMV launches. Single GPU only.
"""

from __future__ import annotations

from collections.abc import Sequence

import torch

from gpu.nf4 import (ATTN_SPLIT, GEMV_MAX_N, nf4_attn_batch, nf4_gemm_rows, nf4_gemv_n,
                     nf4_pick_commit_batch, nf4_rms_rows, nf4_silu_mul)

from .embed import PackedEmbed
from .graph import capture_on_side_stream
from .linear import DeviceLinear, DeviceWeights
from .runner import consume_prompt
from .state import DecodeState, GraphSafeKV

__all__ = ["BatchState", "BatchLoop", "batched_greedy_decode", "GEMV_ROWS"]

#: sequences up to which the linears take the CUDA-core GEMV (one launch of four rows)
GEMV_ROWS = min(4, GEMV_MAX_N)


class BatchState:
    """Registers, KV blocks and activation rows of ``batch`` sequences."""

    def __init__(self, weights: DeviceWeights, batch: int, dtype: torch.dtype = torch.bfloat16):
        spec = weights.spec
        if spec.tp != 1:
            raise RuntimeError("batched decode is single-GPU")
        if batch < 1:
            raise ValueError("batch must be >= 1")
        self.spec, self.batch = spec, int(batch)
        b = self.batch
        dev = weights.lm_head.packed.device
        self.device = dev
        i64 = lambda: torch.zeros(b, dtype=torch.int64, device=dev)
        self.token, self.position, self.next_token = i64(), i64(), i64()
        self.valid_len = torch.zeros(b, dtype=torch.int32, device=dev)
        self.finished = torch.zeros(b, dtype=torch.uint8, device=dev)
        shape = (spec.n_layers, b, spec.max_seq, spec.n_kv, spec.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=dev)
        self.v = torch.zeros(shape, dtype=dtype, device=dev)
        z = lambda *s: torch.zeros((b, *s), dtype=dtype, device=dev)
        self.x = z(spec.hidden)
        self.q = z(spec.n_q, spec.head_dim)
        self.k_act, self.v_act = z(spec.n_kv, spec.head_dim), z(spec.n_kv, spec.head_dim)
        self.attn = z(spec.q_dim)
        self.logits = z(spec.vocab)
        self.attn_ws = torch.zeros(b * spec.n_q * ATTN_SPLIT * (spec.head_dim + 2), dtype=torch.float32,
                                   device=dev)
        self.pick_scratch = torch.zeros((b, 16), dtype=torch.uint8, device=dev)
        self.status = torch.zeros((), dtype=torch.int32, device=dev)
        # one single-sequence state per row for the prompt: its KV tensors are this
        # batch's blocks, so the chunked prefill writes straight into them
        self._seq: list[DecodeState] = []
        first = None
        for i in range(b):
            st = DecodeState.allocate(spec, weights.embed, dtype=dtype,
                                      cos=None if first is None else first.cos,
                                      sin=None if first is None else first.sin)
            kv = GraphSafeKV.__new__(GraphSafeKV)
            kv.n_layers, kv.max_seq, kv.n_kv, kv.head_dim = (spec.n_layers, spec.max_seq, spec.n_kv,
                                                           spec.head_dim)
            kv.k, kv.v, kv.valid_len = self.k[:, i], self.v[:, i], st.valid_len
            st.kv = kv
            if first is None:
                first = st
            self._seq.append(st)
        self.cos, self.sin = first.cos, first.sin

    def reset(self) -> None:
        for t in (self.token, self.position, self.next_token, self.valid_len, self.finished):
            t.zero_()
        for st in self._seq:
            st.reset()

    def prefill(self, weights: DeviceWeights, prompts: Sequence[Sequence[int]],
                chunk: int | None = None) -> None:
        """Ingest one prompt per sequence (chunked GEMM prefill of the single-sequence
        executor, one sequence after the other) and load the batch registers."""
        if len(prompts) != self.batch:
            raise ValueError(f"{len(prompts)} prompts for a batch of {self.batch}")
        self.reset()
        for i, (st, ids) in enumerate(zip(self._seq, prompts)):
            consume_prompt(st, weights, ids, chunk=chunk)
            self.next_token[i].copy_(st.next_token)
            self.token[i].copy_(st.next_token)
            self.position[i].copy_(st.position)
            self.valid_len[i].copy_(st.valid_len)


def _linear(mat: DeviceLinear, rows: torch.Tensor, out: torch.Tensor | None = None,
            add: torch.Tensor | None = None) -> torch.Tensor:
    """``rows [B, K] @ W.T (+ bias) (+ add)`` -> ``[B, M]``."""
    n = int(rows.size(0))
    if n <= GEMV_ROWS:
        return nf4_gemv_n(mat.packed, mat.scale, rows, mat.M, mat.K, mat.K_pad, out=out, add=add,
                          bias=mat.bias)
    # bias and residual ride the GEMM epilogue (one rounding); ``add`` may be ``out`` itself
    return nf4_gemm_rows(mat.packed, mat.scale, rows, mat.M, mat.K, mat.K_pad,
                         out=None if out is None else out.view(n, mat.M), bias=mat.bias,
                         add=None if add is None else add.view(n, mat.M))


def batched_forward(state: BatchState, weights: DeviceWeights) -> None:
    spec, b = state.spec, state.batch
    if isinstance(weights.embed, PackedEmbed):
        weights.embed.gather(state.token, out=state.x, status=state.status)
    else:
        torch.index_select(weights.embed, 0, state.token, out=state.x)
    state.valid_len.copy_(state.position)
    state.valid_len.add_(1)
    for li, layer in enumerate(weights.layers):
        h = nf4_rms_rows(state.x, layer.norm1, spec.rms_eps)
        if layer.wqkv is None and layer.qkv_rows is not None:
            # q, k, v stacked in memory: one pass over the activations instead of three
            y = _linear(layer.qkv_rows, h)
            mq, mk = layer.q.M, layer.k.M
            state.q.view(b, -1).copy_(y[:, :mq])
            state.k_act.view(b, -1).copy_(y[:, mq:mq + mk])
            state.v_act.view(b, -1).copy_(y[:, mq + mk:])
        elif layer.wqkv is None:
            _linear(layer.q, h, out=state.q)
            _linear(layer.k, h, out=state.k_act)
            _linear(layer.v, h, out=state.v_act)
        else:
            grouped = _linear(layer.wqkv, h).view(b, spec.n_kv, spec.n_rep + 2, spec.head_dim)
            state.q.view(b, spec.n_kv, spec.n_rep, spec.head_dim).copy_(grouped[:, :, : spec.n_rep])
            state.k_act.copy_(grouped[:, :, -2])
            state.v_act.copy_(grouped[:, :, -1])
        nf4_attn_batch(state.q, state.k[li], state.v[li], state.attn, state.valid_len,
                       spec.attn_scale, state.attn_ws, ATTN_SPLIT, state.k_act, state.v_act,
                       state.cos, state.sin, state.position)
        _linear(layer.o, state.attn, out=state.x, add=state.x)
        h = nf4_rms_rows(state.x, layer.norm2, spec.rms_eps)
        if layer.gate_up is not None:
            act = nf4_silu_mul(_linear(layer.gate_up, h), spec.intermediate)
        else:
            g, u = _linear(layer.gate, h), _linear(layer.up, h)
            act = nf4_silu_mul(torch.cat([g, u], dim=1), spec.intermediate)
        _linear(layer.down, act, out=state.x, add=state.x)
    h = nf4_rms_rows(state.x, weights.final_norm, spec.rms_eps)
    _linear(weights.lm_head, h, out=state.logits)


def batched_greedy_decode(state: BatchState, weights: DeviceWeights) -> None:
    """Forward for every sequence, then pick + commit per sequence on the device."""
    batched_forward(state, weights)
    nf4_pick_commit_batch(state.logits, state.next_token, state.pick_scratch, state.token,
                          state.position, state.finished, int(state.spec.eos_id))


class BatchLoop:
    """Prefill ``B`` prompts, then decode them together (optionally as one CUDA graph per step)."""

    def __init__(self, weights: DeviceWeights, batch: int) -> None:
        self.weights = weights
        self.state = BatchState(weights, batch)
        self._graph = None

    def capture_graph(self) -> None:
        body = lambda: batched_greedy_decode(self.state, self.weights)
        snap = [t.clone() for t in (self.state.token, self.state.position, self.state.valid_len,
                                    self.state.next_token, self.state.finished)]
        self._graph = capture_on_side_stream(body, warm_runs=2)
        for t, s in zip((self.state.token, self.state.position, self.state.valid_len,
                         self.state.next_token, self.state.finished), snap):
            t.copy_(s)

    def step(self) -> None:
        if self._graph is not None:
            self._graph.replay()
        else:
            batched_greedy_decode(self.state, self.weights)

    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], n_new: int,
                 chunk: int | None = None) -> list[list[int]]:
        """``n_new`` greedy ids per sequence (EOS ignored), read back once at the end."""
        st = self.state
        st.prefill(self.weights, prompts, chunk=chunk)
        trace = torch.zeros((max(1, int(n_new)), st.batch), dtype=torch.int64, device=st.device)
        trace[0].copy_(st.next_token)
        for i in range(1, int(n_new)):
            self.step()
            trace[i].copy_(st.token)
        torch.cuda.synchronize()
        return [[int(t) for t in trace[:, j].tolist()] for j in range(st.batch)]
