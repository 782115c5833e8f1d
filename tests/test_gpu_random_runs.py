"""Random scheduler runs: the same requests with steps replayed from CUDA graphs and launched
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
