"""Random runs: schedules and cuts drawn from seeds, where the hand-made traces of the other
tests have fixed ones.

Scheduler runs first: the same requests with steps replayed from CUDA graphs and launched
eagerly must give the same tokens.

Every trial draws a tiny configuration, a page size, a token budget, a portion size, a batch
bound, look-ahead or not, how often a bucket must be seen before it is captured, and 6 to 20
requests of 1 to 70 prompt tokens with 1 to 12 new tokens each, with so few pages that requests
wait for one another.  In 32-bit the tokens must be equal (a replayed step runs the same kernels
on the same numbers; only filler entries are added); in bfloat16 a padded step may pick another
split of the keys, so requests whose tokens differ are only counted.  After every run no page
may be leased.
"""

from __future__ import annotations

import random

import pytest

import plain_qwen3 as plain
from helpers import make_model_folder, random_ids

pytestmark = pytest.mark.gpu

CONFIGS = {"A": (plain.TINY_A, 0), "B": (plain.TINY_B, 2), "C": (plain.TINY_C, 5), "D": (plain.TINY_D, 6),
           "E": (plain.TINY_E, 7)}


@pytest.mark.parametrize("seed", [3, 17])
def test_random_runs_with_and_without_graphs(seed, tmp_path) -> None:
    from forge_engine_b200.config import EngineConfig, SchedulerConfig
    from forge_engine_b200.engine import Engine, ModelRunner
    from forge_engine_b200.sampling import SamplingParams

    rng = random.Random(seed)
    folders = {}
    for name, (raw, weight_seed) in CONFIGS.items():
        cfg, _ = make_model_folder(tmp_path / name, dict(raw, eos_token_id=None), weight_seed)
        folders[name] = (tmp_path / name, cfg)
    differing = 0
    for trial in range(10):
        name = rng.choice(sorted(CONFIGS))
        folder, cfg = folders[name]
        page = rng.choice([4, 8, 16])
        dtype = rng.choice(["float32", "float32", "bfloat16"])
        requests = rng.randint(6, 20)
        prompts = [random_ids(cfg.vocab_size, rng.randint(1, 70), rng.randint(0, 10 ** 6)) for _ in range(requests)]
        news = [rng.randint(1, 12) for _ in range(requests)]
        pages = sum(-(-(len(p) + n) // page) + 1 for p, n in zip(prompts, news)) // 2 + 40
        scheduler = SchedulerConfig(max_requests=requests + 1, max_batch_size=rng.choice([2, 3, 4, 6]),
                                    token_budget=rng.choice([8, 12, 24, 48, 100]), chunk_size=rng.choice([None, 5, 8, 16]),
                                    block_size=page, block_capacity=pages, lookahead=rng.random() < 0.5)
        after = rng.choice([0, 1, 3])
        outputs = {}
        for graphs in (False, True):
            runner = ModelRunner.from_folder(folder, dtype=dtype, page_size=page, num_pages=pages,
                                             max_requests=requests + 1, use_graphs=graphs)
            runner.graphs.capture_after = after
            engine = Engine(runner, EngineConfig(dtype=dtype), scheduler)
            outputs[graphs] = engine.generate(prompts, [SamplingParams(max_new_tokens=n) for n in news])
            runner.cache.check_consistency()
            assert all(n == 0 for n in runner.cache.leased_pages())
        what = f"trial {trial}: {name} {dtype}, pages of {page}, {scheduler}"
        if dtype == "float32":
            assert outputs[True] == outputs[False], what
        else:
            differing += sum(a != b for a, b in zip(outputs[True], outputs[False]))
    assert differing <= 4, f"{differing} bfloat16 requests differ between replayed and eager steps"


@pytest.mark.parametrize("seed", [5, 23])
def test_random_replays_at_the_benchmark_layer_sizes(seed) -> None:
    """Random replays through ``ModelRunner.step`` at the benchmark model's layer sizes (two
    layers; the tcgen05 products and attention kernels, the split and the balanced decode
    kernels, the library product above 64 tokens) against the plain implementation: 3 to 8
    requests of up to 1,200 tokens, up to 4 or 8 live, cut into single tokens, portions of 2
    to 5 and portions of up to 900 tokens, requests left out of steps now and then, logits
    wanted at random places, in 32-bit and bfloat16, replayed from graphs or launched eagerly."""
    import torch

    import test_gpu_real_sizes as sizes
    from forge_engine_b200.engine import StepEntry

    rng = random.Random(seed)
    model = sizes.Model(sizes.TWO_LAYERS, 11)
    for trial in range(6):
        dtype = rng.choice(["float32", "bfloat16", "bfloat16"])
        sequences = {f"r{i}": random_ids(5003, rng.randint(2, rng.choice([60, 300, 1200])), rng.randint(0, 10 ** 6))
                     for i in range(rng.randint(3, 8))}
        expected = {k: model.plain_logits(v) for k, v in sequences.items()}
        live_max = rng.choice([4, 4, 8])
        pages = sum(-(-len(v) // 16) for v in sequences.values()) + 1
        runner = model.runner(dtype, pages=pages, requests=live_max, graphs=rng.random() < 0.7)
        runner.graphs.capture_after = rng.choice([0, 2])
        waiting = sorted(sequences)
        rng.shuffle(waiting)
        live, fed = [], {}
        while waiting or live:
            while waiting and len(live) < live_max and rng.random() < 0.7:
                key = waiting.pop()
                runner.begin(key)
                live.append(key)
                fed[key] = 0
            entries = []
            for key in live:
                if rng.random() < 0.15 and len(live) > 1:
                    continue
                left = len(sequences[key]) - fed[key]
                kind = rng.random()
                count = 1 if kind < 0.45 else (rng.randint(2, 5) if kind < 0.65 else rng.randint(2, rng.choice([40, 70, 300, 900])))
                count = max(1, min(count, left))
                want = sorted(rng.sample(range(count), rng.randint(0, min(count, 3))))
                entries.append(StepEntry(key, sequences[key][fed[key] : fed[key] + count], want))
            if not entries:
                continue
            out = runner.step(entries).float().cpu()
            row = 0
            for entry in entries:
                for j in entry.want:
                    at = fed[entry.key] + j
                    sizes.check_rows(dtype, out[row : row + 1], expected[entry.key][at : at + 1],
                                     f"trial {trial}, {dtype}: {entry.key}[{at}] beside {[(e.key, len(e.tokens)) for e in entries]}")
                    row += 1
                fed[entry.key] += len(entry.tokens)
            for key in [k for k in live if fed[k] == len(sequences[k])]:
                runner.end(key)
                live.remove(key)
        runner.check_status()
        runner.cache.check_consistency()
        assert all(n == 0 for n in runner.cache.leased_pages())
        del runner
        torch.cuda.empty_cache()


def test_random_sampled_runs_with_end_tokens_and_tight_pools(tmp_path) -> None:
    """Sampled requests (temperature, top-k, top-p, min-p, each with a seed of its own), an end
    token in half of the models, and pools from just the largest request's pages upwards, so
    that requests are put back and run again: with and without graphs, with and without
    look-ahead, the four runs give the same tokens in 32-bit (a request's random stream is keyed
    by its seed and its position, not by the step it is sampled in)."""
    from forge_engine_b200.config import EngineConfig, SchedulerConfig
    from forge_engine_b200.engine import Engine, ModelRunner
    from forge_engine_b200.sampling import SamplingParams

    rng = random.Random(29)
    for trial in range(8):
        name = rng.choice(sorted(CONFIGS))
        raw, weight_seed = CONFIGS[name]
        end = rng.choice([None, rng.randint(0, raw["vocab_size"] - 1)])
        folder = tmp_path / f"{name}{trial}"
        cfg, _ = make_model_folder(folder, dict(raw, eos_token_id=end), weight_seed)
        page = rng.choice([4, 8, 16])
        requests = rng.randint(5, 16)
        prompts = [random_ids(cfg.vocab_size, rng.randint(1, 60), rng.randint(0, 10 ** 6)) for _ in range(requests)]
        params = [SamplingParams(temperature=rng.choice([0.0, 0.0, 0.7, 1.0, 1.5]), top_k=rng.choice([None, 1, 5, 50]),
                                 top_p=rng.choice([1.0, 0.9, 0.5]), min_p=rng.choice([0.0, 0.05]),
                                 max_new_tokens=rng.randint(1, 14), seed=rng.randint(0, 10 ** 9)) for _ in range(requests)]
        largest = max(-(-(len(p) + q.max_new_tokens) // page) + 1 for p, q in zip(prompts, params))
        pages = largest + rng.choice([0, 2, 5, 20, 60])
        outputs = {}
        for graphs in (False, True):
            for lookahead in (False, True):
                scheduler = SchedulerConfig(max_requests=requests + 1, max_batch_size=4, token_budget=24, block_size=page,
                                            block_capacity=pages, lookahead=lookahead)
                runner = ModelRunner.from_folder(folder, dtype="float32", page_size=page, num_pages=pages,
                                                 max_requests=requests + 1, use_graphs=graphs)
                runner.graphs.capture_after = 1
                engine = Engine(runner, EngineConfig(dtype="float32"), scheduler)
                outputs[(graphs, lookahead)] = engine.generate(prompts, params)
                runner.cache.check_consistency()
                assert all(n == 0 for n in runner.cache.leased_pages())
        first = outputs[(False, False)]
        differ = [key for key, tokens in outputs.items() if tokens != first]
        assert not differ, f"trial {trial}: {name}, pages of {page}, pool {pages} (largest request {largest}), end token {end}: {differ}"


def test_random_configurations_of_the_architecture(tmp_path) -> None:
    """Configurations drawn from a seed - head sizes in steps of 16 up to 256, 1 to 4 key/value
    heads with 1 to 8 query heads each, widths and feed-forward widths in steps of 8, 1 to 4
    layers, any vocabulary from 20 to 700, windows on none, some or all layers, tied or untied
    embeddings, with and without projection bias, several eps and theta - each built from a
    model folder and stepped in 32-bit and in bfloat16 with three requests cut at random,
    against the plain implementation."""
    from forge_engine_b200.engine import ModelRunner, StepEntry

    rng = random.Random(53)
    for trial in range(8):
        d = 16 * rng.randint(1, 8) if rng.random() < 0.7 else rng.choice([64, 128, 256])
        nkv, groups, layers = rng.choice([1, 2, 3, 4]), rng.choice([1, 2, 3, 4, 6, 8]), rng.randint(1, 4)
        window = rng.choice([None, None, 5, 11, 33, 70, 130])
        raw = dict(plain.TINY_A, vocab_size=rng.randint(20, 700), hidden_size=8 * rng.randint(2, 40),
                   intermediate_size=8 * rng.randint(2, 60), num_hidden_layers=layers, num_attention_heads=nkv * groups,
                   num_key_value_heads=nkv, head_dim=d, rms_norm_eps=rng.choice([1e-6, 1e-5, 3e-4]),
                   rope_theta=rng.choice([1e4, 5e5, 1e6, 1234.5]), tie_word_embeddings=rng.random() < 0.5,
                   attention_bias=rng.random() < 0.3, eos_token_id=None)
        if window is not None:
            raw.update(use_sliding_window=True, sliding_window=window, max_window_layers=rng.randint(0, layers))
        described = {k: raw[k] for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                         "num_attention_heads", "num_key_value_heads", "head_dim", "sliding_window")}
        cfg, weights = make_model_folder(tmp_path / f"m{trial}", raw, trial)
        sequences = {f"r{i}": random_ids(cfg.vocab_size, rng.randint(2, 220), rng.randint(0, 10 ** 6)) for i in range(3)}
        expected = {k: plain.forward_logits(v, weights, cfg) for k, v in sequences.items()}
        for dtype in ("float32", "bfloat16"):
            page = rng.choice([4, 8, 16, 32])
            pages = sum(-(-len(v) // page) for v in sequences.values()) + 2
            runner = ModelRunner.from_folder(tmp_path / f"m{trial}", dtype=dtype, page_size=page, num_pages=pages,
                                             max_requests=3, use_graphs=rng.random() < 0.6)
            runner.graphs.capture_after = 0
            fed = {k: 0 for k in sequences}
            for key in sequences:
                runner.begin(key)
            while any(fed[k] < len(sequences[k]) for k in sequences):
                entries = []
                for key in sequences:
                    left = len(sequences[key]) - fed[key]
                    if left:
                        count = min(left, rng.choice([1, 1, 2, 3, 17, 64, 100, 200]))
                        entries.append(StepEntry(key, sequences[key][fed[key] : fed[key] + count], sorted({0, count - 1})))
                out = runner.step(entries).float().cpu()
                row = 0
                for entry in entries:
                    for j in entry.want:
                        ref = expected[entry.key][fed[entry.key] + j]
                        limit = 3e-5 if dtype == "float32" else 3e-2 * max(1.0, float(ref.abs().max()))
                        error = float((out[row] - ref).abs().max())
                        assert error <= limit, f"trial {trial} {described}, {dtype}, pages of {page}: {entry.key}[{fed[entry.key] + j}] {error:.3e}"
                        row += 1
                    fed[entry.key] += len(entry.tokens)
            for key in sequences:
                runner.end(key)
            runner.check_status()
