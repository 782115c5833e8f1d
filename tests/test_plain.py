"""The plain implementation against stored outputs of the upstream model (CPU)."""

from __future__ import annotations

from pathlib import Path

import pytest
import torch
from safetensors.torch import load_file

import plain_qwen3 as plain

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize(
    "name,raw,seed", [("tiny_a", plain.TINY_A, 0), ("tiny_b", plain.TINY_B, 2), ("tiny_c", plain.TINY_C, 5)]
)
def test_plain_matches_upstream_outputs(name: str, raw: dict, seed: int) -> None:
    golden = load_file(str(GOLDEN / f"{name}.safetensors"))
    cfg = plain.PlainConfig.from_dict(raw)
    weights = plain.seeded_weights(cfg, seed)
    ids = golden["ids"].long()
    last, layers = plain.hidden_states(ids, weights, cfg, torch.float32)
    for index, hidden in enumerate(layers):
        torch.testing.assert_close(hidden, golden[f"layer_{index}"], atol=2e-6, rtol=1e-5)
    logits = plain.forward_logits(ids, weights, cfg)
    torch.testing.assert_close(logits, golden["logits"], atol=5e-6, rtol=1e-5)
    # upstream fed the same tokens in portions through its tuple cache
    torch.testing.assert_close(logits, golden["chunked_logits"], atol=2e-5, rtol=1e-5)


def test_rms_norm_formula() -> None:
    x = torch.tensor([[1.0, -2.0, 3.0, -4.0]])
    w = torch.tensor([1.0, 2.0, 3.0, 4.0])
    expected = x * torch.rsqrt(x.square().mean(-1, keepdim=True) + 1e-6) * w
    torch.testing.assert_close(plain.rms_norm(x, w, 1e-6), expected)


def test_rotation_pairs_halves() -> None:
    x = torch.arange(8.0).view(1, 1, 8)
    cosine, sine = plain.rotary_tables(torch.tensor([3]), 8, 10000.0, torch.float32)
    y = plain.apply_rotary(x, cosine, sine)[0, 0]
    for j in range(4):
        angle = 3.0 * 10000.0 ** (-2 * j / 8)
        c, s = torch.cos(torch.tensor(angle)), torch.sin(torch.tensor(angle))
        assert abs(float(y[j]) - float(x[0, 0, j] * c - x[0, 0, j + 4] * s)) < 1e-5
        assert abs(float(y[j + 4]) - float(x[0, 0, j + 4] * c + x[0, 0, j] * s)) < 1e-5


def test_prefix_logits_do_not_depend_on_later_tokens() -> None:
    cfg = plain.PlainConfig.from_dict(plain.TINY_C)
    weights = plain.seeded_weights(cfg, 5)
    ids = torch.randint(0, cfg.vocab_size, (19,), generator=torch.Generator().manual_seed(9))
    whole = plain.forward_logits(ids, weights, cfg)
    prefix = plain.forward_logits(ids[:11], weights, cfg)
    torch.testing.assert_close(whole[:11], prefix, atol=2e-6, rtol=1e-5)


def test_filters_keep_expected_survivors() -> None:
    logits = torch.log(torch.tensor([[0.5, 0.25, 0.15, 0.07, 0.03]]))
    assert torch.isfinite(plain.filter_logits(logits, 1.0, top_k=2)).sum() == 2
    # cumulative mass before token 2 is 0.75 > 0.7, so tokens 0 and 1 survive
    assert torch.isfinite(plain.filter_logits(logits, 1.0, top_p=0.7)).sum() == 2
    # min_p 0.2: threshold 0.1, keeps 0.5, 0.25, 0.15
    assert torch.isfinite(plain.filter_logits(logits, 1.0, min_p=0.2)).sum() == 3
    assert int(plain.greedy(logits)) == 0


def test_bfloat16_flow_stays_close_to_float32() -> None:
    cfg = plain.PlainConfig.from_dict(plain.TINY_A)
    weights = plain.seeded_weights(cfg, 0)
    ids = torch.randint(0, cfg.vocab_size, (16,), generator=torch.Generator().manual_seed(1))
    full = plain.forward_logits(ids, weights, cfg, torch.float32)
    half = plain.forward_logits(ids, weights, cfg, torch.bfloat16)
    assert float((full - half).abs().max()) < 0.05 * float(full.abs().max())
