"""What stands in for a memory checker and a fault injector on the GPU, and the engine's
own instruments: a bounded wait that runs out and is reported, canary words round the
cache pool and the scratch buffers, loading without a second copy of the weights, and the
per-part timers of the step function."""

from __future__ import annotations

import json

import pytest
import torch

import plain_qwen3 as plain
from helpers import make_model_folder, random_ids, run_trace

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def native():
    from forge_engine_b200.ops import native as module

    module.require_cuda()
    module.lib()
    return module


def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable(native, tmp_path) -> None:
    """The producer of the tcgen05 product is told to leave out one load and every wait is
    cut to 20,000 polls: the block waiting for that tile gives up, sets status bit 8 and
    returns on its own (tensor memory freed, nothing left spinning).  The host turns the bit
    into an exception, and the next ordinary launch gives the right product."""
    from forge_engine_b200.engine import ModelRunner
    from forge_engine_b200.errors import ForgeEngineError

    g = torch.Generator().manual_seed(0)
    x = (torch.randn((8, 512), generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn((256, 512), generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    want = x.float() @ w.float().t()
    cfg, _ = make_model_folder(tmp_path / "m", plain.TINY_A, 0)
    runner = ModelRunner.from_folder(tmp_path / "m", dtype="bfloat16", page_size=4, num_pages=8, max_requests=1)
    status = runner.ctx.status
    for ksplit in (1, 2):
        out = torch.zeros((8, 256), dtype=torch.float32, device=DEV)
        native.gemm_tc5_set_test_fault(20000, 5)          # k-block 5 of 8 never arrives
        try:
            native.gemm_tc5(x, w, out, native.TC5_STORE_F32, status, ksplit=ksplit)
            torch.cuda.synchronize()
        finally:
            native.gemm_tc5_set_test_fault(0, -1)
        assert int(status.item()) & 8
        with pytest.raises(ForgeEngineError, match="bounded wait"):
            runner.check_status()
        assert int(status.item()) == 0                     # reading it cleared it
        native.gemm_tc5(x, w, out, native.TC5_STORE_F32, status, ksplit=ksplit)
        torch.cuda.synchronize()
        torch.testing.assert_close(out, want, atol=2e-2, rtol=2e-2)
        runner.check_status()


def test_canary_words_show_a_write_beside_the_pool_or_the_scratch(native, tmp_path) -> None:
    from forge_engine_b200.engine import ModelRunner, StepEntry
    from forge_engine_b200.errors import ForgeEngineError

    cfg, _ = make_model_folder(tmp_path / "m", plain.TINY_E, 7)
    runner = ModelRunner.from_folder(tmp_path / "m", dtype="bfloat16", page_size=16, num_pages=40, max_requests=2)
    runner.begin("a")
    runner.step([StepEntry("a", random_ids(cfg.vocab_size, 300, 1), [])])
    for token in random_ids(cfg.vocab_size, 5, 2):
        runner.step([StepEntry("a", [token], [0])])       # split decode attention: uses the scratch
    runner.check_status()                                  # a whole run leaves every canary alone
    assert len(runner.cache.guarded) == 2                  # full and windowed layer group
    assert native.damaged_canaries(runner.cache.guarded) == []
    pool = runner.cache.guarded[0]
    saved = pool._guards[1][0].clone()
    pool._guards[1][0] = 0                                 # what a write just past the last page does
    with pytest.raises(ForgeEngineError, match="cache pool of layer group 0"):
        runner.check_status()
    pool._guards[1][0] = saved
    scratch = native._scratch.all[0]
    saved = scratch._guards[0][-1].clone()
    scratch._guards[0][-1] = 7                             # ... and one just before a scratch buffer
    assert native.damaged_canaries() == [scratch.name]
    scratch._guards[0][-1] = saved
    runner.check_status()


def test_loading_holds_no_second_copy_of_the_weights(native, tmp_path) -> None:
    """Weights reach the device tensor by tensor as the model is assembled; what a part
    fuses (q/k/v, gate/up) exists twice only for the layer being built.  Peak memory while
    loading stays within 5 % of what the finished runner holds."""
    from forge_engine_b200.config import read_model_config
    from forge_engine_b200.engine import ModelRunner
    from forge_engine_b200.weights import RandomTensors, write_model_folder

    raw = dict(plain.TINY_B, hidden_size=1024, intermediate_size=3072, num_hidden_layers=12, num_attention_heads=16,
               num_key_value_heads=4, head_dim=64, vocab_size=8192, eos_token_id=None)
    arch, _, spec = read_model_config(raw)
    lazy = RandomTensors(arch.expected_tensors(spec), 1, dtype=torch.bfloat16, device="cpu")
    write_model_folder(tmp_path / "mid", raw, {name: lazy[name] for name in lazy})
    for build in ("folder", "random"):
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        before = torch.cuda.memory_allocated()
        torch.cuda.reset_peak_memory_stats()
        if build == "folder":
            runner = ModelRunner.from_folder(tmp_path / "mid", dtype="bfloat16", page_size=16, num_pages=4, max_requests=1)
        else:
            runner = ModelRunner.from_random(raw, 1, dtype="bfloat16", page_size=16, num_pages=4, max_requests=1)
        torch.cuda.synchronize()
        held = torch.cuda.memory_allocated() - before
        peak = torch.cuda.max_memory_allocated() - before
        weights = runner.model.weight_bytes()
        # what stays: the weights a step reads, the embedding table (untied here), a tiny cache
        assert weights > 150e6 and held < 1.10 * weights
        assert peak <= 1.05 * held, f"{build}: peak {peak / 1e6:.1f} MB while loading, {held / 1e6:.1f} MB held"
        del runner


def test_step_timers_and_the_timing_dump(native, tmp_path) -> None:
    from forge_engine_b200.engine import ModelRunner, StepEntry
    from forge_engine_b200.errors import ForgeEngineError

    cfg, _ = make_model_folder(tmp_path / "m", plain.TINY_B, 2)
    runner = ModelRunner.from_folder(tmp_path / "m", dtype="bfloat16", page_size=16, num_pages=16, max_requests=2,
                                     timing=True)
    assert not runner.use_graphs                           # timed steps are launched eagerly
    runner.begin("a")
    runner.step([StepEntry("a", random_ids(cfg.vocab_size, 40, 1), [39])])
    for token in (5, 6, 7):
        runner.step([StepEntry("a", [token], [0])])
    report = runner.timings()
    layers, steps = cfg.num_hidden_layers, 4
    assert report["steps"] == steps and report["tokens"] == 43
    parts = report["parts"]
    assert set(parts) == {"embedding", "input_norm", "mixer", "mixer.qkv_rope_cache", "mixer.attention", "mixer.o_proj",
                          "post_norm", "ffn", "final_norm", "head"}
    assert parts["mixer"]["calls"] == layers * steps and parts["head"]["calls"] == steps
    for figures in parts.values():
        assert 0.0 < figures["minimum"] <= figures["median"] <= figures["maximum"] < 1e3
        assert figures["total_ms"] >= figures["maximum"]
    inner = sum(parts[name]["total_ms"] for name in ("mixer.qkv_rope_cache", "mixer.attention", "mixer.o_proj"))
    assert inner <= parts["mixer"]["total_ms"] * 1.001
    untimed = ModelRunner.from_folder(tmp_path / "m", dtype="bfloat16", page_size=16, num_pages=16, max_requests=2)
    with pytest.raises(ForgeEngineError, match="timing"):
        untimed.timings()
    # the replay tool writes the same figures as JSON
    steps_in = [{"step": 0, "entries": [{"id": "x", "tokens": random_ids(cfg.vocab_size, 9, 3), "want": [8]}], "end": []},
                {"step": 1, "entries": [{"id": "x", "tokens": [4], "want": [0]}], "end": ["x"]}]
    run_trace(tmp_path / "m", tmp_path / "out", "float32", 64, steps_in, ("--timings", str(tmp_path / "t.json")))
    dumped = json.loads((tmp_path / "t.json").read_text())
    assert dumped["steps"] == 2 and dumped["parts"]["ffn"]["calls"] == 2 * layers
