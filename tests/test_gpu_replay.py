"""Trace replay on the GPU against the plain implementation, in 32-bit and bfloat16.

The same requests are replayed whole, with the last 32 tokens one by one, in portions of
changing size, and mixed (up to four live, portions beside decoded tokens, a pool so
small that pages are used again).  Everything goes through ``bin/trace_run``.
"""

from __future__ import annotations

import json

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import trace_modes
from helpers import make_model_folder, random_ids, run_trace

pytestmark = pytest.mark.gpu

# 32-bit: the budget upstream's own cached-vs-whole test uses (tests/test_qwen3.py:61-63).
F32_ATOL = 2e-5
# bfloat16: inputs of every matrix product are rounded to 8 mantissa bits (relative
# 2^-9 each); through a few layers this gives logit errors of a few 1e-3 on logits of
# size ~1.  The bound is 3e-2 of the largest logit; the distributions must also agree.
BF16_REL = 3e-2
BF16_TV = 2e-2

CONFIGS = {
    "A": (plain.TINY_A, 0, 4),
    "B": (plain.TINY_B, 2, 16),
    "C": (plain.TINY_C, 5, 8),
    "D": (plain.TINY_D, 6, 4),
    "E": (plain.TINY_E, 7, 16),
}
LENGTHS = {"A": (70, 41, 97, 33, 52, 64), "B": (1 + 32, 7 + 32, 75, 40, 129, 48),
           "C": (66, 35, 50, 81, 34, 47), "D": (90, 37, 58, 44, 71, 33),
           "E": (200, 150, 170, 140, 260, 130)}


def total_variation(a: np.ndarray, b: np.ndarray) -> float:
    pa = torch.softmax(torch.from_numpy(a).double(), -1)
    pb = torch.softmax(torch.from_numpy(b).double(), -1)
    return float(0.5 * (pa - pb).abs().sum(-1).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_replay_modes_match_plain(name: str, dtype: str, tmp_path) -> None:
    raw, seed, page = CONFIGS[name]
    cfg, weights = make_model_folder(tmp_path / "model", raw, seed)
    sequences = {f"s{i}": random_ids(cfg.vocab_size, n, 100 + i) for i, n in enumerate(LENGTHS[name])}
    expected = {k: plain.forward_logits(v, weights, cfg).numpy() for k, v in sequences.items()}

    trace = trace_modes.Trace()
    for key in ("s0", "s1"):
        trace_modes.whole(trace, key, sequences[key])
    trace_modes.bulk_then_tail(trace, "s0", sequences["s0"])
    trace_modes.bulk_then_tail(trace, "s3", sequences["s3"])
    trace_modes.portions(trace, "s2", sequences["s2"])
    trace_modes.portions(trace, "s1", sequences["s1"], sizes=(2, 2, 3, 2, 17, 2))
    trace_modes.mixed(trace, sequences)
    # the pool holds just what the trace's live requests need, so pages are leased again
    got = run_trace(tmp_path / "model", tmp_path / "out", dtype, trace.peak_tokens, trace.steps,
                    ("--page-size", str(page), "--page-log", str(tmp_path / "pages.json")))
    assert len(trace.rows) > 300
    # ... and they were: some physical page was held by different requests at different times,
    # in every layer group (a windowed group gives pages back while its request lives)
    held = json.loads((tmp_path / "pages.json").read_text())
    assert len(held) == len(trace.steps and {e["id"] for s in trace.steps for e in s["entries"]})
    for group in range(len(held[0]["pages"])):
        owners: dict = {}
        for record in held:
            for page_id in record["pages"][group]:
                owners.setdefault(page_id, set()).add(record["id"])
        assert max(len(ids) for ids in owners.values()) >= 2, "no page was leased a second time"
    worst, worst_at = 0.0, None
    for step, row, key, position in trace.rows:
        mine, ref = got[step][row], expected[key][position]
        err = float(np.abs(mine - ref).max())
        bound = F32_ATOL if dtype == "float32" else BF16_REL * max(1.0, float(np.abs(ref).max()))
        if err > worst:
            worst, worst_at = err, (step, row, key, position)
        assert err <= bound, f"{key}[{position}] in step {step}: error {err:.3e} > {bound:.1e}"
        if dtype == "bfloat16":
            assert total_variation(mine, ref) <= BF16_TV
            # greedy choice agrees unless the plain logits are nearly tied
            top2 = np.sort(ref)[-2:]
            if top2[1] - top2[0] > 2 * bound:
                assert int(mine.argmax()) == int(ref.argmax())
    print(f"{name} {dtype}: {len(trace.rows)} rows, worst error {worst:.3e} at {worst_at}")


def test_sharp_attention_shows_cache_faults(tmp_path) -> None:
    """Random weights give near-uniform attention, which hides a wrong key among many.
    Scaling the q-norm weights makes every query pick out few keys, so a key read from a
    wrong page or slot changes the logits visibly.  32-bit only: the point is the cache."""
    raw, seed, page = CONFIGS["B"]
    cfg = plain.PlainConfig.from_dict(raw)
    weights = plain.seeded_weights(cfg, seed)
    for layer in range(cfg.num_hidden_layers):
        weights[f"model.layers.{layer}.self_attn.q_norm.weight"] *= 8.0
    import json
    from safetensors.torch import save_file

    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(raw))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    ids = random_ids(cfg.vocab_size, 300, 77)
    ref = plain.forward_logits(ids, weights, cfg).numpy()
    # sanity: attention really is sharp - dropping the first page's keys would change a lot
    trace = trace_modes.Trace()
    trace_modes.whole(trace, "x", ids)
    trace_modes.bulk_then_tail(trace, "x", ids)
    trace_modes.portions(trace, "x", ids, sizes=(16, 15, 17, 2, 31, 33, 1, 64))
    got = run_trace(folder, tmp_path / "out", "float32", trace.peak_tokens, trace.steps, ("--page-size", "16"))
    for step, row, _, position in trace.rows:
        err = float(np.abs(got[step][row] - ref[position]).max())
        assert err <= 5 * F32_ATOL, f"position {position} in step {step}: {err:.3e}"
