#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the Qwen3-4B shape, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 with
2,048-token contexts (device time of K decode steps through the step function);
``e2e`` is the same through the Python entry point (``Engine.step``: host token ids in,
sampled ids out, every step); ``prefill`` is one 2,048-token prompt in one step;
``points`` holds decode at batch 1 and 64; ``roofline`` relates the decode step to the
bytes it has to read.  Weights are random (seeded), token ids synthetic (seed 5).
The contexts of the device-timed decode are cache pages filled with random numbers: a
decode step's work does not depend on what the cached keys are.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CONFIG_4B = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "hidden_act": "silu",
    "vocab_size": 151936,
    "hidden_size": 2560,
    "intermediate_size": 9728,
    "num_hidden_layers": 36,
    "num_attention_heads": 32,
    "num_key_value_heads": 8,
    "head_dim": 128,
    "max_position_embeddings": 8192,
    "rms_norm_eps": 1e-6,
    "rope_theta": 5000000.0,
    "tie_word_embeddings": True,
    "attention_bias": False,
    "sliding_window": None,
    "eos_token_id": None,
}
CONTEXT = 2048
PAGE = 16

# Two further shapes, run through the scheduler from prompts to the last token
# (`--workload`): requests, prompt lengths (uniform range, ids from the given seed), new
# tokens per request.
WORKLOADS = {
    "mixed-8b": {
        "config": dict(CONFIG_4B, hidden_size=4096, intermediate_size=12288, rope_theta=1000000.0,
                       max_position_embeddings=32768, tie_word_embeddings=False),
        "requests": 64, "prompt_range": (16, 4096), "new_tokens": 256, "seed": 6, "token_budget": 2048,
    },
    "long-32b": {
        "config": dict(CONFIG_4B, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64,
                       num_attention_heads=64, rope_theta=1000000.0, max_position_embeddings=16384,
                       tie_word_embeddings=False),
        "requests": 32, "prompt_range": (8192, 8192), "new_tokens": 128, "seed": 7, "token_budget": 2048,
    },
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            return float(raw["hbm_gbs"]), float(raw["bf16_tflops"]), "measured"
        except (KeyError, ValueError):
            pass
    return FALLBACK_PEAKS["hbm_gbs"], FALLBACK_PEAKS["bf16_tflops"], "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self) -> None:
        self.proc = None
        self.lines: list = []

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        clocks, max_clock, reasons = [], None, set()
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                max_clock = float(parts[1])
            except ValueError:
                continue
            for name, flag in zip(self.NAMES, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


def reference_arm(args) -> int:
    """Decode tokens per second of the unmodified upstream engine at the same shape.

    Upstream's loader only accepts its pinned Hub checkpoint (src/forge_engine/weights.py:55-70
    downloads it; there is no network here) and it has no random-weights mode.  What it
    does expose publicly is ``ConcurrentGenerationEngine(tokenizer, model, sampling params,
    scheduler config)`` (src/forge_engine/scheduler.py:137-170) and its own
    ``Qwen3ForCausalLM(Qwen3Config(...))``; its tests drive exactly this constructor with a
    stub tokenizer (tests/test_scheduler.py:42-68).  So the arm builds upstream's model
    class with the benchmark's sizes (torch's default random initialisation, bfloat16),
    a stub tokenizer that returns synthetic ids, and times upstream's own ``step()``.
    """
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "forge_engine").is_dir():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed (pip --target install of the reference)"}))
        return 0
    try:
        import torch

        sys.path.insert(0, str(ref_root))
        from forge_engine.qwen3 import Qwen3Config, Qwen3ForCausalLM
        from forge_engine.sampling import SamplingParams
        from forge_engine.scheduler import ConcurrentGenerationEngine, SchedulerConfig

        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device")
        raw = dict(CONFIG_4B)
        if args.layers:
            raw["num_hidden_layers"] = args.layers
        batch, steps, warmup = args.batch, args.steps, max(3, args.warmup)
        config = Qwen3Config(
            vocab_size=raw["vocab_size"], hidden_size=raw["hidden_size"], intermediate_size=raw["intermediate_size"],
            num_hidden_layers=raw["num_hidden_layers"], num_attention_heads=raw["num_attention_heads"],
            num_key_value_heads=raw["num_key_value_heads"], head_dim=raw["head_dim"],
            max_position_embeddings=raw["max_position_embeddings"], rms_norm_eps=raw["rms_norm_eps"],
            rope_theta=raw["rope_theta"], eos_token_id=0, tie_word_embeddings=True, attention_bias=False)
        torch.manual_seed(0)
        with torch.device("cuda:0"):
            model = Qwen3ForCausalLM(config).to(torch.bfloat16).eval()
        generator = torch.Generator().manual_seed(5)

        class StubTokenizer:
            eos_token_id = None

            def apply_chat_template(self, conversation, *, tokenize, add_generation_prompt, return_tensors):
                return torch.randint(0, raw["vocab_size"], (1, CONTEXT), generator=generator)

            def decode(self, token_ids, *, skip_special_tokens):
                return " ".join(str(t) for t in token_ids)

        total = CONTEXT + warmup + steps + 8
        engine = ConcurrentGenerationEngine(
            StubTokenizer(), model, SamplingParams(max_new_tokens=warmup + steps + 4),
            SchedulerConfig(max_requests=batch, max_batch_size=batch, token_budget=batch * CONTEXT,
                            block_size=PAGE, block_capacity=batch * (-(-total // PAGE))))
        for i in range(batch):
            engine.submit([{"role": "user", "content": str(i)}])
        engine.step()                              # all prompts (one length, one forward)
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        sampler = ClockSampler()
        sampler.start()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        t0 = time.perf_counter()
        for _ in range(steps):
            engine.step()
        end.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        ms = begin.elapsed_time(end) / steps
        clocks = sampler.stop()
        print(json.dumps({
            "impl": "reference",
            "metric": "decode tok/s (Qwen3-4B shape, bf16, batch 8, 2048-token contexts)",
            "value": round(batch / (ms / 1e3), 2), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
            "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic token ids (seed 5), upstream model class with torch default init (seed 0)",
            "config": {"model": "Qwen3-4B shape", "layers": raw["num_hidden_layers"], "layers_full": CONFIG_4B["num_hidden_layers"],
                       "hidden": raw["hidden_size"], "q_heads": raw["num_attention_heads"],
                       "kv_heads": raw["num_key_value_heads"], "head_dim": raw["head_dim"],
                       "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"],
                       "global_batch": batch, "seq_len": CONTEXT, "max_context": raw["max_position_embeddings"],
                       "page_size": PAGE, "tied_embeddings": True, "parallelism": "single GPU",
                       "l2": "inputs larger than L2 (weights 8.0 GB read every step)", "peaks": peaks()[2]},
            "api": "ConcurrentGenerationEngine.step with a stub tokenizer",
            "clocks": clocks,
            # upstream keeps the pending token on the device and reads every request's sampled id
            # back with .item() (an int64 each, src/forge_engine/scheduler.py:472-482)
            "e2e": {"value": round(batch * steps / wall, 2), "unit": "tokens/s", "ms_per_step": round(1e3 * wall / steps, 4),
                    "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 8 * batch},
        }))
        return 0
    except Exception as error:  # the arm must never fail the run
        print(json.dumps({"impl": "reference", "unavailable": f"{type(error).__name__}: {str(error)[:200]}"}))
        return 0


def scheduler_workload(name: str, layers: int | None) -> int:
    """All requests of the workload submitted at once; the scheduler cuts the prompts into
    portions under its token budget beside the decoding requests.  Wall-clock time from
    the first submit to the last token, host token ids in and out."""
    import torch

    from forge_engine_b200.config import EngineConfig, SchedulerConfig
    from forge_engine_b200.engine import Engine
    from forge_engine_b200.sampling import SamplingParams

    work = WORKLOADS[name]
    raw = dict(work["config"])
    layers_full = raw["num_hidden_layers"]
    if layers:
        raw["num_hidden_layers"] = layers
    gen = torch.Generator().manual_seed(work["seed"])
    low, high = work["prompt_range"]
    count, new = work["requests"], work["new_tokens"]
    lengths = torch.randint(low, high + 1, (count,), generator=gen).tolist()
    prompts = [torch.randint(0, raw["vocab_size"], (n,), generator=gen).tolist() for n in lengths]
    pages = sum(-(-(n + new) // PAGE) + 1 for n in lengths) + 64
    engine = Engine.from_random(
        raw, 0, engine_config=EngineConfig(max_new_tokens=new, dtype="bfloat16"),
        scheduler_config=SchedulerConfig(max_requests=count, max_batch_size=count, token_budget=work["token_budget"],
                                         block_size=PAGE, block_capacity=pages),
        device="cuda:0")
    # warm-up: builds, first launches, and one prompt step of the full token budget (the library's
    # choice of kernels for that many rows, the allocator's growth: 0.2 s the first time)
    warm = torch.randint(0, raw["vocab_size"], (work["token_budget"] + 64,), generator=gen).tolist()
    engine.generate([warm], SamplingParams(max_new_tokens=4))
    torch.cuda.synchronize()
    warmed = engine.scheduler.snapshot()          # the counters below are those of the timed run alone
    sampler = ClockSampler()
    sampler.start()
    begin = time.perf_counter()
    outputs = engine.generate(prompts, SamplingParams(max_new_tokens=new, temperature=0.0))
    torch.cuda.synchronize()
    seconds = time.perf_counter() - begin
    clocks = sampler.stop()
    made = sum(len(o) for o in outputs)
    # what a roofline needs: the products' flops over all tokens run (prompt tokens and every
    # generated token but each request's last, which is never fed back), the attention flops
    # over the contexts, and the bytes read if every model step streams the weights once and
    # every decoded token its request's cache
    hbm_gbs, bf16_tflops, peak_source = peaks()
    snapshot = engine.scheduler.snapshot()
    h, q = raw["hidden_size"], raw["num_attention_heads"] * raw["head_dim"]
    kv, inter = raw["num_key_value_heads"] * raw["head_dim"], raw["intermediate_size"]
    per_token = 2 * raw["num_hidden_layers"] * (h * (q + 2 * kv) + q * h + 3 * h * inter)
    steps_run = snapshot.model_steps - warmed.model_steps
    prefill_run = snapshot.prefill_tokens - warmed.prefill_tokens
    decode_run = snapshot.decode_tokens - warmed.decode_tokens
    tokens_run = prefill_run + decode_run
    attention = sum(4 * raw["num_hidden_layers"] * q * (n + new) * (n + new + 1) // 2 for n in lengths)
    flops = per_token * tokens_run + attention + 2 * raw["vocab_size"] * h * (made + count)
    weight_bytes = engine.runner.model.weight_bytes()
    kv_bytes = engine.runner.cache.bytes_per_token() * sum((n + new // 2) * new for n in lengths)
    bytes_read = weight_bytes * steps_run + kv_bytes
    sm_mhz = clocks.get("sm_mhz") or 0.0
    print(json.dumps({
        "metric": f"generated tok/s through the scheduler ({name})", "value": round(made / seconds, 1), "unit": "tokens/s",
        "n_gpus": 1, "higher_is_better": True, "dtype": "bf16", "impl": "ours",
        "data": f"synthetic token ids (seed {work['seed']}), random weights (seed 0)",
        "seconds": round(seconds, 3), "generated": made, "prompt_tokens": sum(lengths),
        "all_tokens_per_second": round((made + sum(lengths)) / seconds, 1),
        "config": {"workload": name, "layers": raw["num_hidden_layers"], "layers_full": layers_full,
                   "hidden": raw["hidden_size"], "q_heads": raw["num_attention_heads"],
                   "kv_heads": raw["num_key_value_heads"], "head_dim": raw["head_dim"],
                   "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"], "requests": count,
                   "prompt_min": low, "prompt_max": high, "new_tokens": new, "token_budget": work["token_budget"],
                   "page_size": PAGE, "peaks": peak_source},
        "clocks": clocks,
        "model_steps": steps_run, "prefill_tokens": prefill_run, "decode_tokens": decode_run,
        "roofline": {"flops": flops, "compute_floor_s": round(flops / (bf16_tflops * 1e12), 3),
                     "bytes": int(bytes_read), "hbm_floor_s": round(bytes_read / (hbm_gbs * 1e9), 3),
                     "frac": round((flops / (bf16_tflops * 1e12) + bytes_read / (hbm_gbs * 1e9)) / seconds, 4),
                     "note": "frac = (compute floor + memory floor) / time: prompt steps are bound by flops, decode steps by bytes"},
        "seconds_x_sm_ghz": round(seconds * sm_mhz / 1e3, 3),
    }))
    return 0


def kernel_shapes() -> int:
    """The three kernel shapes upstream publishes (docs/benchmarks.md:27-29, measured there on
    an L4 with 10 warm-up and 50 timed iterations, CUDA events, median): this repository's
    kernels at the same shapes, same method."""
    import torch

    from forge_engine_b200.ops import native

    native.lib()
    device = "cuda:0"
    gen = torch.Generator().manual_seed(5)

    def median_ms(run) -> float:
        for _ in range(10):
            run()
        torch.cuda.synchronize()
        times = []
        for _ in range(50):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            run()
            end.record()
            torch.cuda.synchronize()
            times.append(begin.elapsed_time(end))
        return statistics.median(times)

    status = torch.zeros(1, dtype=torch.int32, device=device)
    results = {}
    # fused residual add + RMSNorm, [512, 2560] bfloat16
    residual = torch.randn((512, 2560), generator=gen).to(device)
    update = torch.randn((512, 2560), generator=gen).bfloat16().to(device)
    weight = torch.ones(2560, device=device)
    out = torch.empty((512, 2560), dtype=torch.bfloat16, device=device)
    results["add_rmsnorm_512x2560_ms"] = round(median_ms(lambda: native.add_rmsnorm(residual, update, weight, out, 1e-6)), 4)
    # paged single-token decode attention: 127 cached keys, 32 q heads, 8 kv heads, head size 128, one request
    nq, nkv, d, page = 32, 8, 128, 16
    k_cache = torch.randn((16, nkv, page, d), generator=gen).bfloat16().to(device)
    v_cache = torch.randn((16, nkv, page, d), generator=gen).bfloat16().to(device)
    table = torch.arange(8, dtype=torch.int32, device=device).view(1, 8)
    q = torch.randn((1, (nq + 2 * nkv) * d), generator=gen).bfloat16().to(device)
    o = torch.empty((1, nq * d), dtype=torch.bfloat16, device=device)
    cu = torch.tensor([0, 1], dtype=torch.int32, device=device)
    starts = torch.tensor([127], dtype=torch.int32, device=device)
    results["paged_decode_past127_ms"] = round(median_ms(lambda: native.attention_mma(
        q, q.shape[1], k_cache, v_cache, table, cu, starts, 1, 1, None, d ** -0.5, o, nq, status, False, True, 1)), 4)
    # causal prefill attention, 128 tokens, 8 heads of 128 (8 kv heads)
    q2 = torch.randn((128, 3 * 8 * d), generator=gen).bfloat16().to(device)
    o2 = torch.empty((128, 8 * d), dtype=torch.bfloat16, device=device)
    k2 = torch.randn((16, 8, page, d), generator=gen).bfloat16().to(device)
    v2 = torch.randn((16, 8, page, d), generator=gen).bfloat16().to(device)
    cu2 = torch.tensor([0, 128], dtype=torch.int32, device=device)
    starts2 = torch.tensor([0], dtype=torch.int32, device=device)
    results["causal_prefill_8x128x128_ms"] = round(median_ms(lambda: native.attention_mma(
        q2, q2.shape[1], k2, v2, table, cu2, starts2, 1, 128, None, d ** -0.5, o2, 8, status, True, False, 1)), 4)
    assert int(status.item()) == 0
    print(json.dumps({"metric": "kernel time at the shapes upstream publishes", "unit": "ms", "impl": "ours", **results,
                      "upstream_on_L4": {"add_rmsnorm_512x2560_ms": 0.0850, "paged_decode_past127_ms": 0.1004,
                                         "causal_prefill_8x128x128_ms": 0.0891}}))
    return 0


def decode_attention(spec: str) -> int:
    """Decode attention alone at given context lengths, e.g. ``2048x64`` or ``32768x1,2048x7``
    (length x requests): the split kernel with the split count the engine would pick, and the
    kernel that spreads all key tiles evenly over the GPU's blocks.  32 query heads, 8 kv heads,
    head size 128, pages of 16; 12 launches over 4 caches in a replayed CUDA graph, so that the
    keys come from DRAM; CUDA events around the replay."""
    import torch

    from forge_engine_b200.ops import native
    from forge_engine_b200.parts.attention import choose_splits

    native.lib()
    device = "cuda:0"
    nq, nkv, d, page, layers, launches = 32, 8, 128, 16, 4, 12
    contexts = []
    for item in spec.split(","):
        length, _, count = item.partition("x")
        contexts += [int(length)] * int(count or 1)
    batch = len(contexts)
    pages_per = [-(-c // page) for c in contexts]
    num_pages = sum(pages_per)
    caches = [(torch.randn((num_pages, nkv, page, d), device=device).bfloat16(),
               torch.randn((num_pages, nkv, page, d), device=device).bfloat16()) for _ in range(layers)]
    order = torch.randperm(num_pages).to(torch.int32)
    table = torch.full((batch, max(pages_per)), -1, dtype=torch.int32)
    at = 0
    for r, n in enumerate(pages_per):
        table[r, :n] = order[at:at + n]
        at += n
    table = table.to(device)
    q = torch.randn((batch, (nq + 2 * nkv) * d), device=device).bfloat16()
    out = torch.empty((batch, nq * d), dtype=torch.bfloat16, device=device)
    cu = torch.arange(batch + 1, dtype=torch.int32, device=device)
    starts = torch.tensor([c - 1 for c in contexts], dtype=torch.int32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    kv_bytes = sum(contexts) * nkv * d * 2 * 2
    tiles = [-(-c // 64) for c in contexts]
    results = {"requests": batch, "longest": max(contexts), "tiles": sum(tiles) * nkv,
               "picked": choose_splits(tiles, nkv, batch <= 256)}
    for name, splits in (("split", choose_splits(tiles, nkv)), ("balanced", 0)):
        if splits == 0 and batch > 256:
            continue

        def run(i):
            k, v = caches[i % layers]
            native.attention_mma(q, q.shape[1], k, v, table, cu, starts, batch, 1, None, d ** -0.5, out, nq, status,
                                 False, True, splits)

        for i in range(3):
            run(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(launches):
                run(i)
        graph.replay()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        us = begin.elapsed_time(end) / launches * 1e3
        results[name] = {"splits": splits, "us": round(us, 1), "gb_per_s": round(kv_bytes / us / 1e3)}
    assert int(status.item()) == 0
    print(json.dumps({"metric": "decode attention alone", "impl": "ours", **results}))
    return 0


def chain_timeline(tokens: int) -> int:
    """The output projection, the norm + gate/up projection with SiLU*mul and the down
    projection of one layer (4B shape, ``tokens`` rows): as the one persistent kernel
    (``native.decode_chain``) and as the separate kernels the engine launches, 12 layers'
    worth of distinct weights back to back in a replayed CUDA graph so that the weights come
    from DRAM; then the persistent kernel's own timeline (nanosecond stamps of every block,
    taken in one launch in the middle of such a sequence)."""
    import ctypes

    import torch

    from forge_engine_b200.ops import native

    handle = native.lib()
    device = "cuda:0"
    hidden, heads, inter, sets = 2560, 4096, 9728, 12

    def rnd(*shape, scale=0.02):
        return (torch.randn(*shape, device=device) * scale).bfloat16()

    weights = [dict(o=rnd(hidden, heads), gu=rnd(2 * inter, hidden), d=rnd(hidden, inter)) for _ in range(sets)]
    norm_w = torch.ones(hidden, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    x = rnd(tokens, heads, scale=1.0)
    h = torch.randn(tokens, hidden, device=device)
    act = torch.empty(tokens, inter, dtype=torch.bfloat16, device=device)
    normed = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=device)

    def chain_one(w):
        native.decode_chain([dict(w=w["o"], x=x, out=h, src=native.CHAIN_SRC_ACTIVATIONS, epi=native.CHAIN_ADD),
                             dict(w=w["gu"], x=h, norm_w=norm_w, eps=1e-6, out=act, src=native.CHAIN_SRC_NORM,
                                  epi=native.CHAIN_SILU_MUL),
                             dict(w=w["d"], x=act, out=h, src=native.CHAIN_SRC_ACTIVATIONS, epi=native.CHAIN_ADD)],
                            tokens, status)

    def separate_one(w):
        native.gemm_tc5(x, w["o"], h, native.TC5_ADD_F32, status, ksplit=native.tc5_ksplit_add(hidden, heads))
        native.add_rmsnorm(h, None, norm_w, normed, 1e-6)
        native.gemm_tc5(normed, w["gu"], act, native.TC5_SILU_MUL, status, ksplit=native.tc5_ksplit(2 * inter, hidden))
        native.gemm_tc5(act, w["d"], h, native.TC5_ADD_F32, status, ksplit=native.tc5_ksplit_add(hidden, inter))

    result = {"metric": "o-projection + norm + gate/up + down of one layer, 4B shape", "tokens": tokens, "impl": "ours",
              "bytes": (hidden * heads + 3 * inter * hidden) * 2}
    for name, one in (("chain_us", chain_one), ("separate_us", separate_one)):
        for w in weights:
            one(w)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for w in weights:
                one(w)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(10):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
        result[name] = round(begin.elapsed_time(end) * 1e3 / 10 / sets, 2)
    handle.fe_decode_chain_blocks.restype = ctypes.c_int
    blocks = handle.fe_decode_chain_blocks()
    trace = torch.zeros(blocks * 16, dtype=torch.int64, device=device)
    for w in weights[:6]:
        chain_one(w)
    handle.fe_decode_chain_trace.argtypes = [ctypes.c_void_p]
    handle.fe_decode_chain_trace(trace.data_ptr())
    chain_one(weights[6])
    handle.fe_decode_chain_trace(None)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    stamps = trace.view(blocks, 16).cpu().double()
    origin = stamps[:, 0].min()
    names = ["block starts"] + [f"projection {j}: {what}" for j in range(3)
                                for what in ("input complete", "token tiles in shared memory", "last product issued",
                                             "share published", "last weight tile requested")]
    print(json.dumps(result))
    for index, name in enumerate(names):
        column = (stamps[:, index] - origin) / 1e3
        print(f"# {name:48s} min {column.min():7.2f}  median {column.median():7.2f}  max {column.max():7.2f} us")
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None,
                        help="timed steps (default 200; 20 for --impl reference, whose step takes a third of a second)")
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--layers", type=int, default=None, help="run fewer layers than the model has")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--shape", default="4b", choices=("4b", "8b", "32b"),
                        help="layer sizes of the decode benchmark: the 4B shape of the headline, or the 8B / 32B "
                             "shapes of the workloads (use --layers to keep it short)")
    parser.add_argument("--skip-points", action="store_true", help="skip batch 1/64, prefill and e2e")
    parser.add_argument("--prefill-only", action="store_true",
                        help="time only the 2,048-token prefill (small cases for profiling)")
    parser.add_argument("--workload", choices=sorted(WORKLOADS),
                        help="instead of the decode benchmark: a whole workload through the scheduler")
    parser.add_argument("--decode-attention", metavar="LENxN[,LENxN...]",
                        help="instead: decode attention alone at these context lengths, split and balanced kernel")
    parser.add_argument("--kernels", action="store_true",
                        help="instead: this repository's kernels at the three kernel shapes upstream publishes")
    parser.add_argument("--chain-timeline", type=int, metavar="TOKENS",
                        help="instead: the persistent kernel for a layer's last three projections against the "
                             "separate kernels, and its per-block timeline")
    parser.add_argument("--step-timeline", action="store_true",
                        help="also print, per kernel of one replayed decode step, the time from the end of the kernel "
                             "before it to its own end (for profiles/)")
    parser.add_argument("--mixed-only", type=int, metavar="TOKENS",
                        help="only the mixed step: 8 requests decoding beside a prompt portion, TOKENS tokens in all "
                             "(with --kernel-times: the kernels of one such step)")
    parser.add_argument("--kernel-times", action="store_true",
                        help="also print the device time of every kernel of one more step (for profiles/)")
    args = parser.parse_args()
    if args.steps is None:
        args.steps = 20 if args.impl == "reference" else 200
    if args.impl == "reference":
        if args.gpus != 1:
            print(f"bench.py measures one GPU; --gpus {args.gpus} is not supported by this single-GPU engine")
            return 2
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not supported by this single-GPU engine")
        return 2
    args.warmup = max(3, args.warmup)
    if args.workload:
        return scheduler_workload(args.workload, args.layers)
    if args.kernels:
        return kernel_shapes()
    if args.decode_attention:
        return decode_attention(args.decode_attention)
    if args.chain_timeline:
        return chain_timeline(args.chain_timeline)

    import torch

    from forge_engine_b200.config import EngineConfig, SchedulerConfig
    from forge_engine_b200.engine import Engine, ModelRunner, StepEntry
    from forge_engine_b200.ops import native

    raw = dict(CONFIG_4B)
    if args.shape != "4b":
        raw = dict(WORKLOADS["mixed-8b" if args.shape == "8b" else "long-32b"]["config"])
    layers_full = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    layers = raw["num_hidden_layers"]
    hbm_gbs, bf16_tflops, peak_source = peaks()
    device = "cuda:0"
    torch.cuda.set_device(0)
    gen = torch.Generator().manual_seed(5)

    max_batch = 64 if not args.skip_points else args.batch
    # the end-to-end run feeds one prompt a step, so requests start decoding up to `batch`
    # steps apart; nobody may reach its length limit inside the timed region
    steps_total = args.warmup + args.steps + 64 + 16
    pages_per_request = -(-(CONTEXT + steps_total) // PAGE) + 1
    num_pages = max_batch * pages_per_request + 8
    runner = main_runner = ModelRunner.from_random(raw, 0, dtype="bfloat16", device=device, page_size=PAGE,
                                                   num_pages=num_pages, max_requests=max_batch)
    for group in runner.cache.groups:        # contexts: pages of random numbers
        group.storage.normal_(0.0, 1.0)
    weight_bytes = runner.model.weight_bytes()
    kv_bytes_per_token = runner.cache.bytes_per_token()

    def decode_run(batch: int, steps: int, warmup: int, context: int = CONTEXT, runner=None) -> tuple:
        runner = runner or main_runner
        keys = [f"d{batch}-{i}" for i in range(batch)]
        for key in keys:
            runner.begin(key)
            runner.cache.reserve(key, context)
            runner.cache.advance(key, context)
        tokens = torch.randint(0, raw["vocab_size"], (batch,), generator=gen).tolist()

        def one_step():
            return runner.step([StepEntry(k, [t], [0]) for k, t in zip(keys, tokens)])

        for _ in range(warmup):
            one_step()
        torch.cuda.synchronize()
        launches_before = native.LAUNCHES
        sampler = ClockSampler()
        sampler.start()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        for _ in range(steps):
            one_step()
        end.record()
        torch.cuda.synchronize()
        ms = begin.elapsed_time(end) / steps
        clocks = sampler.stop()
        launches = native.LAUNCHES - launches_before
        runner.check_status()
        for key in keys:
            runner.end(key)
        return ms, clocks, launches

    def mixed_run(tokens: int, decoders: int, steps: int, warmup: int) -> dict:
        """A step as the scheduler makes it under a token budget of ``tokens``: ``decoders``
        requests with 2,048-token contexts decode one token each beside a prompt portion of
        the remaining tokens (the first portion of a fresh request, every step).  Wall time
        per step - host work, launch and the device, synchronised every step - beside the
        device time alone: replayed from a CUDA graph the two are about the same."""
        keys = [f"m{i}" for i in range(decoders)]
        for key in keys:
            runner.begin(key)
            runner.cache.reserve(key, CONTEXT)
            runner.cache.advance(key, CONTEXT)
        ids = torch.randint(0, raw["vocab_size"], (decoders,), generator=gen).tolist()
        portion = torch.randint(0, raw["vocab_size"], (tokens - decoders,), generator=gen).tolist()
        wall, dev = [], []
        for i in range(warmup + steps):
            key = f"mp{i}"
            runner.begin(key)
            entries = [StepEntry(k, [t], [0]) for k, t in zip(keys, ids)] + [StepEntry(key, portion, [])]
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            begin.record()
            runner.step(entries)
            end.record()
            torch.cuda.synchronize()
            if i >= warmup:
                wall.append((time.perf_counter() - t0) * 1e3)
                dev.append(begin.elapsed_time(end))
            runner.end(key)
        runner.check_status()
        for key in keys:
            runner.end(key)
        return {"ms_wall": statistics.median(wall), "ms_device": statistics.median(dev)}

    def prefill_run(repeats: int) -> dict:
        """One 2,048-token prompt in one step, logits at its last place."""
        prompt = torch.randint(0, raw["vocab_size"], (CONTEXT,), generator=gen).tolist()
        times = []
        for i in range(3 + repeats):
            key = f"p{i}"
            runner.begin(key)
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            begin.record()
            runner.step([StepEntry(key, prompt, [CONTEXT - 1])])
            end.record()
            torch.cuda.synchronize()
            if i >= 3:
                times.append(begin.elapsed_time(end))
            runner.end(key)
        ms_prefill = statistics.median(times)
        h, q = raw["hidden_size"], raw["num_attention_heads"] * raw["head_dim"]
        kv, inter = raw["num_key_value_heads"] * raw["head_dim"], raw["intermediate_size"]
        linear = 2 * CONTEXT * layers * (h * (q + 2 * kv) + q * h + 3 * h * inter) + 2 * raw["vocab_size"] * h
        attention = layers * 4 * raw["num_attention_heads"] * raw["head_dim"] * CONTEXT * (CONTEXT + 1) // 2
        flops = linear + attention
        return {"value": round(CONTEXT / (ms_prefill / 1e3), 1), "tokens": CONTEXT, "ms": round(ms_prefill, 3),
                "frac": round(flops / (ms_prefill / 1e3) / (bf16_tflops * 1e12), 4), "flops": flops}

    def kernel_times(step) -> None:
        """Device time of the kernels of one call of ``step`` (CUPTI through torch.profiler;
        shares for reading, never a bench value)."""
        from torch.profiler import ProfilerActivity, profile

        step()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step()
            torch.cuda.synchronize()
        rows = {}
        for event in prof.events():
            if event.device_type == torch.autograd.DeviceType.CUDA and "Memcpy" not in event.name:
                count, total = rows.get(event.name, (0, 0.0))
                rows[event.name] = (count + 1, total + event.time_range.end - event.time_range.start)
        whole = sum(total for _, total in rows.values())
        print(f"# kernels of one step: {whole:.0f} us summed over {sum(c for c, _ in rows.values())} launches")
        for name, (count, total) in sorted(rows.items(), key=lambda kv: -kv[1][1]):
            print(f"# {total:9.1f} us {100 * total / whole:5.1f}%  x{count:<4d} {total / count:7.1f} us each  {name[:90]}")

    def step_timeline(step) -> None:
        """Kernels of a replayed step overlap (programmatic dependent launch), so a kernel's own
        duration says little; the time from the end of the kernel before it to its own end adds
        up to the step.  CUPTI through torch.profiler: shares for reading, never a bench value."""
        from torch.profiler import ProfilerActivity, profile

        step()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step()
            torch.cuda.synchronize()
        events = [e for e in prof.events()
                  if e.device_type == torch.autograd.DeviceType.CUDA and "emcpy" not in e.name and "emset" not in e.name]
        events.sort(key=lambda e: e.time_range.end)
        previous = events[0].time_range.start
        rows: dict = {}
        for event in events:
            name = event.name.replace("(anonymous namespace)::", "").replace("void ", "")[:70]
            count, total = rows.get(name, (0, 0.0))
            rows[name] = (count + 1, total + event.time_range.end - previous)
            previous = event.time_range.end
        whole = sum(total for _, total in rows.values())
        print(f"# end-to-end shares of one step: {whole:.0f} us over {len(events)} kernels, {whole / layers:.1f} us per layer")
        for name, (count, total) in rows.items():
            print(f"# {total:9.1f} us {100 * total / whole:5.1f}%  x{count:<4d} {total / count:7.2f} us each  {name}")

    if args.prefill_only:
        record = {"prefill": prefill_run(max(1, args.steps)), "layers": layers, "impl": "ours"}
        if args.kernel_times:
            prompt = torch.randint(0, raw["vocab_size"], (CONTEXT,), generator=gen).tolist()

            def one_prefill():
                runner.begin("kt")
                runner.step([StepEntry("kt", prompt, [CONTEXT - 1])])
                runner.end("kt")

            kernel_times(one_prefill)
        print(json.dumps(record))
        return 0

    if args.mixed_only:
        tokens, decoders = args.mixed_only, 8
        mixed = mixed_run(tokens, decoders, max(1, args.steps if args.steps != 200 else 20), 24)
        record = {"mixed": {"tokens": tokens, "decoding": decoders, "ms_wall": round(mixed["ms_wall"], 3),
                            "ms_device": round(mixed["ms_device"], 3),
                            "value": round(tokens / (mixed["ms_device"] / 1e3), 1)}, "layers": layers, "impl": "ours"}
        if args.kernel_times:
            keys = [f"mk{i}" for i in range(decoders)]
            for key in keys:
                runner.begin(key)
                runner.cache.reserve(key, CONTEXT)
                runner.cache.advance(key, CONTEXT)
            portion = torch.randint(0, raw["vocab_size"], (tokens - decoders,), generator=gen).tolist()

            def one_mixed():
                runner.begin("mkp")
                runner.step([StepEntry(k, [7], [0]) for k in keys] + [StepEntry("mkp", portion, [])])
                runner.end("mkp")

            for _ in range(20):        # let the step's bucket be captured: the table is of a replayed step
                one_mixed()
            kernel_times(one_mixed)
        print(json.dumps(record))
        return 0

    ms_step, clocks, launches = decode_run(args.batch, args.steps, args.warmup)
    if args.kernel_times:
        keys = [f"kt{i}" for i in range(args.batch)]
        for key in keys:
            runner.begin(key)
            runner.cache.reserve(key, CONTEXT)
            runner.cache.advance(key, CONTEXT)
        kernel_times(lambda: runner.step([StepEntry(k, [7], [0]) for k in keys]))
        for key in keys:
            runner.end(key)
    if args.step_timeline:
        keys = [f"tl{i}" for i in range(args.batch)]
        for key in keys:
            runner.begin(key)
            runner.cache.reserve(key, CONTEXT)
            runner.cache.advance(key, CONTEXT)
        step_timeline(lambda: runner.step([StepEntry(k, [7], [0]) for k in keys]))
        for key in keys:
            runner.end(key)
    value = args.batch / (ms_step / 1e3)
    step_bytes = weight_bytes + args.batch * (CONTEXT + args.warmup + args.steps / 2) * kv_bytes_per_token
    achieved = step_bytes / (ms_step / 1e3) / 1e9
    record = {
        "metric": f"decode tok/s (Qwen3-{args.shape.upper()} shape, bf16, batch {args.batch}, 2048-token contexts)",
        "value": round(value, 2),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic token ids (seed 5), random weights (seed 0), contexts are random cache pages",
        "impl": "ours",
        "config": {
            "model": f"Qwen3-{args.shape.upper()} shape",
            "layers": layers,
            "layers_full": layers_full,
            "hidden": raw["hidden_size"],
            "q_heads": raw["num_attention_heads"],
            "kv_heads": raw["num_key_value_heads"],
            "head_dim": raw["head_dim"],
            "intermediate": raw["intermediate_size"],
            "vocab": raw["vocab_size"],
            "global_batch": args.batch,
            "seq_len": CONTEXT,
            "max_context": raw["max_position_embeddings"],
            "page_size": PAGE,
            "tied_embeddings": bool(raw["tie_word_embeddings"]),
            "parallelism": "single GPU",
            "l2": "inputs larger than L2 (weights %.1f GB read every step)" % (weight_bytes / 1e9),
            "peaks": peak_source,
        },
        "clocks": clocks,
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4), "bytes_per_step": int(step_bytes)},
    }

    if not args.skip_points:
        points = {}
        for batch in (1, 64):
            ms, _, _ = decode_run(batch, max(10, args.steps // 2), args.warmup)
            points[f"decode_b{batch}"] = round(batch / (ms / 1e3), 2)
        mixed = mixed_run(256, 8, 20, 24)      # the warm-up lets the step's bucket be captured (17th sighting)
        points["mixed_256"] = round(256 / (mixed["ms_wall"] / 1e3), 1)         # tokens a second, wall clock
        points["mixed_256_ms_wall"] = round(mixed["ms_wall"], 3)
        points["mixed_256_ms_device"] = round(mixed["ms_device"], 3)
        record["points"] = points

        record["prefill"] = prefill_run(3)

        # decode at longer contexts (the model's own position limit, 262,144, instead of the
        # benchmark's 8,192): 8,192 and 32,768 cached tokens per request, batch 1 and 8
        del runner, main_runner
        torch.cuda.empty_cache()
        long_raw = dict(raw, max_position_embeddings=262144)
        long_steps = 30
        long_runner = ModelRunner.from_random(long_raw, 0, dtype="bfloat16", device=device, page_size=PAGE,
                                              num_pages=8 * (-(-(32768 + 64) // PAGE) + 1) + 8, max_requests=8)
        for group in long_runner.cache.groups:
            group.storage.normal_(0.0, 1.0)
        for context, label in ((8192, "8k"), (32768, "32k")):
            for batch in (1, 8):
                ms, _, _ = decode_run(batch, long_steps, args.warmup, context, long_runner)
                points[f"decode_b{batch}_ctx{label}"] = round(batch / (ms / 1e3), 2)
                bytes_read = weight_bytes + batch * (context + args.warmup + long_steps / 2) * kv_bytes_per_token
                points[f"decode_b{batch}_ctx{label}_hbm_frac"] = round(bytes_read / (ms / 1e3) / 1e9 / hbm_gbs, 4)
        del long_runner
        torch.cuda.empty_cache()

        # end to end through the Python entry point: host ids in, sampled ids out, every step
        e2e_steps = args.steps
        engine = Engine.from_random(
            raw, 0,
            engine_config=EngineConfig(max_new_tokens=steps_total, dtype="bfloat16"),
            scheduler_config=SchedulerConfig(max_requests=args.batch, max_batch_size=args.batch,
                                             token_budget=CONTEXT + args.batch, block_size=PAGE,
                                             block_capacity=args.batch * pages_per_request + 8),
            device=device,
        )
        for i in range(args.batch):
            engine.submit(torch.randint(0, raw["vocab_size"], (CONTEXT,), generator=gen).tolist())
        while engine.scheduler.snapshot().running < args.batch:
            engine.step()
        for _ in range(args.warmup):
            engine.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        produced = 0
        for _ in range(e2e_steps):
            produced += sum(len(e.tokens) for e in engine.step())
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
        last = engine.runner.cache
        h2d = 4 * (args.batch * 8 + 16 + args.batch * (-(-(CONTEXT + args.warmup + e2e_steps) // PAGE)))
        record["e2e"] = {"value": round(produced / elapsed, 2), "unit": "tokens/s",
                         "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch,
                         "ms_per_step": round(1e3 * elapsed / e2e_steps, 4)}
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
