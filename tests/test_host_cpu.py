"""Host-side seats and request objects that need no GPU: construction, shape checks,
the no-fallback rule (nothing computes on the CPU)."""

from __future__ import annotations

import pytest
import torch

from gpu.chr0.loader import ChrMatrix
from gpu.decodev2 import Generation
from gpu.host.embedding import Nf4Embedding, dequant_nf4_rows
from gpu.host.linear import CompressedLinear, nf4_linear


def _matrix(m: int, k: int, name: str = "w") -> ChrMatrix:
    kp = 64 * ((k + 63) // 64)
    return ChrMatrix(name, m, k, kp, torch.zeros((m, kp // 2), dtype=torch.uint8),
                     torch.ones((m, kp // 64), dtype=torch.float16))


def test_compressed_linear_is_an_empty_seat_until_attached():
    seat = CompressedLinear(128, 64, bias=True)
    assert (seat.in_features, seat.out_features, seat.M, seat.K, seat.K_pad) == (128, 64, 64, 128, 128)
    assert not seat.is_loaded and seat.weight.numel() == 0 and seat.nbytes == 0
    assert "loaded=False" in repr(seat)
    assert not list(seat.parameters()) and "packed" not in seat.state_dict()
    with pytest.raises(RuntimeError, match="attach"):
        seat(torch.zeros(1, 128, dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        seat.attach(_matrix(64, 192))
    with pytest.raises(ValueError):
        CompressedLinear(128, 64, bias=False).attach(_matrix(64, 128), torch.zeros(64))
    seat.attach(_matrix(64, 128, "layers.0.q"), torch.ones(64))
    assert seat.is_loaded and seat.chr_name == "layers.0.q" and seat.nbytes == 64 * 64 + 64 * 2 * 2
    # attached on the CPU there is still nothing to run it: the ops are CUDA-only
    with pytest.raises(RuntimeError):
        seat(torch.zeros(1, 128, dtype=torch.bfloat16))


def test_nf4_linear_checks_features_and_empty_batches_before_any_launch():
    m = _matrix(64, 128)
    with pytest.raises(ValueError, match="K=128"):
        nf4_linear(torch.zeros(2, 64), m.packed, m.scale, 64, 128, 128)
    with pytest.raises(ValueError, match="empty"):
        nf4_linear(torch.zeros(0, 128), m.packed, m.scale, 64, 128, 128)


def test_nf4_embedding_seat_and_row_decoder_checks():
    emb = Nf4Embedding(40, 200)
    assert not emb.is_loaded and emb.weight.numel() == 0
    with pytest.raises(RuntimeError, match="attach"):
        emb(torch.tensor([1, 2]))
    with pytest.raises(ValueError):
        emb.attach(_matrix(41, 200))
    emb.attach(_matrix(40, 200, "embed"))
    assert emb.is_loaded and emb.chr_name == "embed"
    with pytest.raises(TypeError):
        dequant_nf4_rows(emb.packed.to(torch.int8), emb.scale, torch.tensor([0]), 200)
    with pytest.raises(TypeError):
        dequant_nf4_rows(emb.packed, emb.scale.float(), torch.tensor([0]), 200)
    with pytest.raises(ValueError):
        dequant_nf4_rows(emb.packed, emb.scale[:, :2], torch.tensor([0]), 200)
    with pytest.raises(RuntimeError):  # CPU ids: no CPU path
        dequant_nf4_rows(emb.packed, emb.scale, torch.tensor([0]), 200)


def test_generation_rates_keep_prefill_and_decode_apart():
    g = Generation(prompt_len=512, tokens=list(range(65)), prefill_ms=16.0, decode_ms=128.0,
                   decode_steps=64)
    assert g.decode_tok_s == pytest.approx(500.0) and g.ms_per_token == pytest.approx(2.0)
    assert g.prefill_tok_s == pytest.approx(32000.0)
    assert g.eval_tok_s == pytest.approx(65 / 0.128)
    assert Generation(prompt_len=1).decode_tok_s == 0.0


def test_token_loop_shares_the_request_api():
    from gpu.decodev2 import DecodeV2Loop
    from gpu.loop import TokenLoop

    for name in ("generate", "prefill_from", "decode_from_logits", "step", "warmup",
                 "capture_graphs", "reset", "seal_last"):
        assert callable(getattr(TokenLoop, name))
    assert issubclass(TokenLoop, DecodeV2Loop)
