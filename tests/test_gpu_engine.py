"""The engine in-process on the GPU: parts alone, first tokens, long decoding, generation
through the entry point, and a toy architecture registered from this file."""

from __future__ import annotations

from dataclasses import dataclass

import pytest
import torch

import plain_qwen3 as plain
from helpers import make_model_folder, random_ids

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32 = dict(atol=2e-5, rtol=1e-5)


def bound(dtype: str, ref: torch.Tensor) -> dict:
    if dtype == "float32":
        return F32
    return dict(atol=3e-2 * max(1.0, float(ref.abs().max())), rtol=0.0)


@pytest.fixture(scope="module")
def fe():
    import forge_engine_b200
    from forge_engine_b200.ops import native

    native.require_cuda()
    native.lib()
    return forge_engine_b200


def runner_for(tmp_path, raw, seed, dtype, page=8, pages=64, requests=4):
    from forge_engine_b200.engine import ModelRunner

    cfg, weights = make_model_folder(tmp_path / f"m{seed}{dtype}", raw, seed)
    runner = ModelRunner.from_folder(tmp_path / f"m{seed}{dtype}", dtype=dtype, page_size=page,
                                     num_pages=pages, max_requests=requests)
    return cfg, weights, runner


# ---------------------------------------------------------------------------
# parts alone
# ---------------------------------------------------------------------------

def build_ctx(dtype):
    from forge_engine_b200.parts import BuildContext

    return BuildContext(dtype=dtype, device=torch.device(DEV), status=torch.zeros(1, dtype=torch.int32, device=DEV))


def one_request_batch(cache, key, tokens, want=()):
    from forge_engine_b200.engine import StepEntry, build_batch

    cache.reserve(key, cache.request(key).length + len(tokens))
    return build_batch([StepEntry(key, tokens, list(want))], cache, DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_and_feed_forward_parts(fe, dtype) -> None:
    from forge_engine_b200.config import GatedMLPSpec, NormSpec
    from forge_engine_b200.parts import build_part

    ctx = build_ctx(dtype)
    g = torch.Generator().manual_seed(0)
    hidden, inter, n = 88, 136, 21
    w = {"gate_proj.weight": torch.randn((inter, hidden), generator=g) * 0.1,
         "up_proj.weight": torch.randn((inter, hidden), generator=g) * 0.1,
         "down_proj.weight": torch.randn((hidden, inter), generator=g) * 0.1}
    w = {k: v.bfloat16().float() for k, v in w.items()}
    ffn = build_part(GatedMLPSpec(hidden, inter), {k: v.to(dtype).to(DEV) for k, v in w.items()}, ctx)
    x = torch.randn((n, hidden), generator=g).bfloat16().float()
    ref = plain.feed_forward(x, {f"p.{k}": v for k, v in w.items()}, "p")
    out = ffn.forward(x.to(dtype).to(DEV)).float().cpu()
    torch.testing.assert_close(out, ref, **(F32 if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)))

    norm_w = 1 + 0.1 * torch.randn(hidden, generator=g)
    norm = build_part(NormSpec(hidden, 1e-5), {"weight": norm_w.to(DEV)}, ctx)
    res = torch.randn((n, hidden), generator=g)
    upd = torch.randn((n, hidden), generator=g).bfloat16().float()
    dev_res = res.clone().to(DEV)
    out = norm.add_forward(dev_res, upd.to(dtype).to(DEV)).float().cpu()
    torch.testing.assert_close(dev_res.cpu(), res + upd, atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(out, plain.rms_norm(res + upd, norm_w, 1e-5),
                               **(F32 if dtype == torch.float32 else dict(atol=2e-2, rtol=1e-2)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 9])
def test_attention_part_and_block_alone(fe, dtype, window) -> None:
    """One attention mixer and one whole block, fed in two portions, against the plain
    functions over the whole sequence."""
    from forge_engine_b200.cache import CacheManager
    from forge_engine_b200.config import AttentionSpec, GatedMLPSpec, LayerSpec, NormSpec, RotarySpec
    from forge_engine_b200.parts import arrangement_class, build_part

    raw = dict(plain.TINY_C, num_hidden_layers=1)
    if window:
        raw.update(use_sliding_window=True, sliding_window=window, max_window_layers=0)
    cfg = plain.PlainConfig.from_dict(raw)
    weights = plain.seeded_weights(cfg, 9)
    ctx = build_ctx(dtype)
    spec = AttentionSpec(cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                         True, cfg.rms_norm_eps, True, cfg.head_dim ** -0.5,
                         RotarySpec(cfg.head_dim, cfg.rope_theta, cfg.head_dim), window)
    prefix = "model.layers.0.self_attn"
    local = {k[len(prefix) + 1:]: v.to(dtype).to(DEV) for k, v in weights.items() if k.startswith(prefix)}
    mixer = build_part(spec, local, ctx)
    cache = CacheManager([mixer.cache_needs()], page_size=4, num_pages=16, max_requests=2, dtype=dtype, device=DEV)
    cache.begin_request("r")
    g = torch.Generator().manual_seed(2)
    n = 29
    x = torch.randn((n, cfg.hidden_size), generator=g).bfloat16().float()
    ref = plain.attention(x, weights, prefix, cfg, window)
    outs = []
    for lo, hi in ((0, 18), (18, 29)):
        batch = one_request_batch(cache, "r", [0] * (hi - lo))
        outs.append(mixer.forward(x[lo:hi].to(dtype).to(DEV), batch, cache.view(0)).float().cpu())
        cache.advance("r", hi)
    assert int(ctx.status.item()) == 0
    torch.testing.assert_close(torch.cat(outs), ref, **(F32 if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)))

    # the whole block: h += attn(norm(h)); returns ffn update
    layer = LayerSpec(NormSpec(cfg.hidden_size, cfg.rms_norm_eps), spec, NormSpec(cfg.hidden_size, cfg.rms_norm_eps),
                      GatedMLPSpec(cfg.hidden_size, cfg.intermediate_size))
    roles = {"input_norm": "model.layers.0.input_layernorm", "mixer": prefix,
             "post_norm": "model.layers.0.post_attention_layernorm", "ffn": "model.layers.0.mlp"}
    block_cls = arrangement_class("pre_norm")
    per_role = {role: {k[len(p) + 1:]: v.to(dtype).to(DEV) for k, v in weights.items() if k.startswith(p + ".")}
                for role, p in roles.items()}
    block = block_cls(layer, per_role, ctx)
    cache.end_request("r")
    cache.begin_request("r")
    batch = one_request_batch(cache, "r", [0] * n)
    h = x.clone().to(DEV)
    pending = block.forward(h, None, batch, cache.view(0))
    total = h.cpu() + pending.float().cpu()
    ref_h = plain.decoder_layer(x, weights, 0, cfg)
    torch.testing.assert_close(total, ref_h, **(F32 if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)))


def test_rotary_table_is_the_plain_formula(fe) -> None:
    from forge_engine_b200.config import RotarySpec
    from forge_engine_b200.parts import build_part

    part = build_part(RotarySpec(48, 5e6, 48), {}, build_ctx(torch.float32))
    inv_freq, rotary_dim = part.rotary()
    ref = 1.0 / (5e6 ** (torch.arange(0, 48, 2, dtype=torch.float32) / 48))
    assert rotary_dim == 48 and torch.equal(inv_freq.cpu(), ref)


# ---------------------------------------------------------------------------
# whole model
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(fe, dtype, tmp_path) -> None:
    """Sequences of 1, 2 and 3 tokens, and the first tokens of a longer one, alone and in
    one batch together."""
    from forge_engine_b200.engine import StepEntry

    cfg, weights, runner = runner_for(tmp_path, plain.TINY_B, 2, dtype, page=16)
    seqs = {f"s{n}": random_ids(cfg.vocab_size, n, 40 + n) for n in (1, 2, 3, 17)}
    for key, ids in seqs.items():
        runner.begin(key)
    logits = runner.step([StepEntry(k, ids, range(len(ids))) for k, ids in seqs.items()]).cpu()
    runner.check_status()
    row = 0
    for key, ids in seqs.items():
        ref = plain.forward_logits(ids, weights, cfg)
        torch.testing.assert_close(logits[row : row + len(ids)], ref, **bound(dtype, ref))
        row += len(ids)
        runner.end(key)
    # token by token from the very first one
    ids = seqs["s17"]
    ref = plain.forward_logits(ids, weights, cfg)
    runner.begin("t")
    for i, token in enumerate(ids):
        out = runner.step([StepEntry("t", [token], [0])]).cpu()
        torch.testing.assert_close(out[0], ref[i], **bound(dtype, ref))
    runner.end("t")
    runner.cache.check_consistency()
    assert runner.cache.leased_pages() == [0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(fe, dtype, tmp_path) -> None:
    """A short prompt followed by several hundred single-token steps, across many pages,
    with a windowed layer giving pages back on the way (config D)."""
    from forge_engine_b200.engine import StepEntry

    cfg, weights, runner = runner_for(tmp_path, plain.TINY_D, 6, dtype, page=4, pages=200)
    ids = random_ids(cfg.vocab_size, 420, 8)
    ref = plain.forward_logits(ids, weights, cfg)
    runner.begin("a")
    out = [runner.step([StepEntry("a", ids[:5], [4])]).cpu()[0]]
    for token in ids[5:]:
        out.append(runner.step([StepEntry("a", [token], [0])]).cpu()[0])
    runner.check_status()
    got = torch.stack(out)
    torch.testing.assert_close(got, ref[4:], **bound(dtype, ref))
    full, windowed = runner.cache.leased_pages()
    assert full == 105 and windowed <= 4       # window 11 over pages of 4
    runner.end("a")
    assert runner.cache.leased_pages() == [0, 0]


@pytest.mark.parametrize("graphs", [True, False])
def test_decoding_with_the_balanced_attention_kernel(fe, tmp_path, monkeypatch, graphs) -> None:
    """Requests of very different lengths decoded together with the kernel that spreads all
    key tiles evenly over the blocks (forced here: tiny models never reach the sizes at which
    it is chosen), one layer windowed, replayed from CUDA graphs and step by step."""
    from forge_engine_b200.engine import StepEntry

    from forge_engine_b200.engine import ModelRunner

    monkeypatch.setenv("FORGE_ENGINE_DECODE_BALANCED", "always")
    cfg, weights = make_model_folder(tmp_path / "model", plain.TINY_E, 7)
    runner = ModelRunner.from_folder(tmp_path / "model", dtype="bfloat16", page_size=16, num_pages=80,
                                     max_requests=4, use_graphs=graphs)
    lengths = {"a": 330, "b": 3, "c": 140}
    new = 72
    ids = {k: random_ids(cfg.vocab_size, n + new, 20 + i) for i, (k, n) in enumerate(lengths.items())}
    ref = {k: plain.forward_logits(v, weights, cfg) for k, v in ids.items()}
    for k, n in lengths.items():
        runner.begin(k)
        runner.step([StepEntry(k, ids[k][:n], [])])
    for i in range(new):
        keys = [k for k in lengths if not (k == "b" and i % 3 == 2)]      # b sits some steps out
        done = {k: lengths[k] + sum(1 for j in range(i) if not (k == "b" and j % 3 == 2)) for k in keys}
        out = runner.step([StepEntry(k, [ids[k][done[k]]], [0]) for k in keys]).float().cpu()
        for row, k in enumerate(keys):
            torch.testing.assert_close(out[row], ref[k][done[k]], **bound("bfloat16", ref[k]))
    runner.check_status()


def test_pages_run_out_without_side_effects(fe, tmp_path) -> None:
    from forge_engine_b200.engine import StepEntry
    from forge_engine_b200.errors import KVCacheCapacityError

    cfg, weights, runner = runner_for(tmp_path, plain.TINY_A, 0, "float32", page=4, pages=6)
    ids = random_ids(cfg.vocab_size, 30, 3)
    runner.begin("a"), runner.begin("b")
    runner.step([StepEntry("a", ids[:10], [])])
    with pytest.raises(KVCacheCapacityError):
        runner.step([StepEntry("a", ids[10:12], [1]), StepEntry("b", ids[:13], [12])])
    assert runner.cache.request("a").length == 10 and runner.cache.request("b").length == 0
    assert runner.cache.leased_pages() == [3]
    runner.cache.check_consistency()
    out = runner.step([StepEntry("a", ids[10:12], [1])]).cpu()
    torch.testing.assert_close(out[0], plain.forward_logits(ids[:12], weights, cfg)[11], **F32)
    with pytest.raises(ValueError, match="outside the vocabulary"):
        runner.step([StepEntry("a", [cfg.vocab_size], [0])])
    with pytest.raises(ValueError, match="only once"):
        runner.step([StepEntry("a", [1], [0]), StepEntry("a", [2], [0])])


def test_float32_checkpoint_in_bfloat16_engine_keeps_32_bit_tensors(fe, tmp_path) -> None:
    """A tensor stored in 32-bit stays 32-bit and its products run on the plain FFMA path."""
    from forge_engine_b200.engine import ModelRunner, StepEntry

    cfg, weights = make_model_folder(tmp_path / "m", plain.TINY_A, 0, store_dtype=torch.float32)
    runner = ModelRunner.from_folder(tmp_path / "m", dtype="bfloat16", page_size=8, num_pages=16, max_requests=2)
    assert runner.model.blocks[0].ffn.down.weight.dtype == torch.float32
    ids = random_ids(cfg.vocab_size, 20, 1)
    runner.begin("a")
    out = runner.step([StepEntry("a", ids, range(20))]).cpu()
    ref = plain.forward_logits(ids, weights, cfg)
    torch.testing.assert_close(out, ref, **bound("bfloat16", ref))


# ---------------------------------------------------------------------------
# generation through the entry point
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_matches_plain(fe, dtype, tmp_path) -> None:
    """Configuration A of the baseline: prompts of 5 / 9 / 13 tokens, 8 greedy tokens each,
    page size 4; in 32-bit the ids must equal the plain implementation's exactly."""
    from forge_engine_b200.config import EngineConfig, SchedulerConfig
    from forge_engine_b200.engine import Engine

    cfg, weights = make_model_folder(tmp_path / "m", dict(plain.TINY_A, eos_token_id=None), 0)
    engine = Engine.from_pretrained(
        tmp_path / "m",
        engine_config=EngineConfig(max_new_tokens=8, dtype=dtype),
        scheduler_config=SchedulerConfig(block_size=4, block_capacity=32, token_budget=16, chunk_size=6, max_batch_size=3),
    )
    prompts = [random_ids(cfg.vocab_size - 1, n, 1 + n) for n in (5, 9, 13)]
    outputs = engine.generate(prompts)
    for prompt, output in zip(prompts, outputs):
        assert len(output) == 8
        if dtype == "float32":
            assert output == plain.greedy_generate(prompt, 8, weights, cfg)
        else:
            # bfloat16: every chosen token is the plain argmax unless the top two are nearly tied
            ids = list(prompt)
            for token in output:
                ref = plain.forward_logits(ids, weights, cfg)[-1]
                top = torch.topk(ref, 2).values
                if float(top[0] - top[1]) > 6e-2:
                    assert token == int(ref.argmax())
                ids.append(token)
    snap = engine.scheduler.snapshot()
    assert snap.allocated_blocks == (0,) and snap.reserved_blocks == (0,)


def test_sampled_generation_is_reproducible_and_follows_the_plain_distribution(fe, tmp_path) -> None:
    """Configuration B of the baseline: prompts 1 / 7 / 33 / 40, portions of 8 mixed with
    decoding, temperature 0.8.  With the kernel's uniform restated on the host, every
    sampled id equals the draw from the plain implementation's filtered distribution."""
    from forge_engine_b200.config import EngineConfig, SchedulerConfig
    from forge_engine_b200.engine import Engine
    from forge_engine_b200.sampling import SamplingParams
    from test_gpu_kernels import twin_draw

    cfg, weights = make_model_folder(tmp_path / "m", dict(plain.TINY_B, eos_token_id=None), 2)
    sched = SchedulerConfig(block_size=16, block_capacity=32, token_budget=24, chunk_size=8, max_batch_size=4)
    prompts = [random_ids(cfg.vocab_size - 2, n, 3 + n) for n in (1, 7, 33, 40)]
    params = [SamplingParams(temperature=0.8, max_new_tokens=6, seed=4 + i, top_k=50 if i % 2 else None,
                             top_p=0.95 if i == 2 else 1.0) for i in range(4)]
    runs = []
    for _ in range(2):
        engine = Engine.from_pretrained(tmp_path / "m", engine_config=EngineConfig(dtype="float32"), scheduler_config=sched)
        runs.append(engine.generate(prompts, params))
    assert runs[0] == runs[1]
    for prompt, p, output in zip(prompts, params, runs[0]):
        ids = list(prompt)
        for counter, token in enumerate(output):
            ref = plain.forward_logits(ids, weights, cfg)[-1]
            want, running, target = twin_draw(ref, p.temperature, p.top_k, p.top_p, p.min_p, p.seed, counter)
            if token != want:
                assert float((running - target).abs().min()) < 1e-4 * float(running[-1])
            ids.append(token)


def test_stream_and_cli(fe, tmp_path, capsys) -> None:
    from forge_engine_b200.cli import main
    from forge_engine_b200.config import EngineConfig, SchedulerConfig
    from forge_engine_b200.engine import Engine
    from forge_engine_b200.sampling import SamplingParams

    cfg, weights = make_model_folder(tmp_path / "m", dict(plain.TINY_A, eos_token_id=None), 0)
    prompt = random_ids(cfg.vocab_size - 1, 6, 5)
    want = plain.greedy_generate(prompt, 5, weights, cfg)
    engine = Engine.from_pretrained(tmp_path / "m", engine_config=EngineConfig(dtype="float32"),
                                    scheduler_config=SchedulerConfig(block_size=4, block_capacity=16))
    assert list(engine.stream(prompt, SamplingParams(max_new_tokens=5))) == want
    stream = engine.stream(prompt, SamplingParams(max_new_tokens=5))
    assert next(stream) == want[0]
    stream.close()          # consumer stops early: pages still come back
    assert engine.scheduler.snapshot().allocated_blocks == (0,)
    code = main(["generate", "--model", str(tmp_path / "m"), "--prompt-ids", ",".join(map(str, prompt)),
                 "--max-new-tokens", "5", "--dtype", "float32", "--block-size", "4", "--block-capacity", "16"])
    assert code == 0
    assert capsys.readouterr().out.strip().splitlines()[-1] == ",".join(map(str, want))
    assert main(["generate", "--model", str(tmp_path / "nowhere"), "--prompt-ids", "1"]) == 1
    assert "forge-engine:" in capsys.readouterr().err
    assert main(["doctor"]) == 0
    assert "cuda_available=True" in capsys.readouterr().out


# ---------------------------------------------------------------------------
# a toy architecture defined here: a mixer with state of its own, a layer named twice,
# a run that reads another run's cache - without touching the package's files
# ---------------------------------------------------------------------------

@dataclass(frozen=True)
class ToyDecaySpec:
    hidden_size: int
    decay: float
    kind: str = "toy_decay_mixer"


def register_toy():
    from forge_engine_b200.cache import CacheNeeds, StateSpec
    from forge_engine_b200.config import (Architecture, AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec,
                                          NoPositionSpec, NormSpec, RunSpec, register_architecture)
    from forge_engine_b200.parts import Mixer, WeightInfo, register_part

    class ToyDecayMixer(Mixer):
        """s_t = decay * s_{t-1} + x_t W^T ; y_t = s_t.  The state s is per request and of
        fixed size; a portion continues from the state the last portion left."""

        def __init__(self, spec, weights, ctx):
            self.spec, self.w = spec, weights["w.weight"].float()
            self.dtype = ctx.dtype

        @classmethod
        def weight_shapes(cls, spec):
            return {"w.weight": WeightInfo((spec.hidden_size, spec.hidden_size))}

        def cache_needs(self):
            return CacheNeeds(state=StateSpec((self.spec.hidden_size,), "float32"))

        def forward(self, x, batch, cache):
            u = x.float() @ self.w.t()
            out = torch.empty_like(u)
            row = 0
            for slot, start, count in batch.entries:
                s = cache.state[slot]
                assert start > 0 or float(s.abs().sum()) == 0.0   # a fresh slot is zeroed
                for i in range(row, row + count):
                    s = self.spec.decay * s + u[i]
                    out[i] = s
                cache.state[slot] = s
                row += count
            return out.to(self.dtype)

    register_part("toy_decay_mixer", ToyDecayMixer, replace=True)

    def spec_of(raw: dict) -> ModelSpec:
        h = raw["hidden_size"]
        norm = NormSpec(h, raw["eps"])
        attn = AttentionSpec(h, 4, 2, 16, False, raw["eps"], False, 0.3, NoPositionSpec(), None)
        ffn = GatedMLPSpec(h, raw["inter"])

        def names(i):
            return {"input_norm": f"l{i}.n1", "mixer": f"l{i}.mix", "post_norm": f"l{i}.n2", "ffn": f"l{i}.ffn"}

        layers = (LayerSpec(norm, attn, norm, ffn, names(0)),
                  LayerSpec(norm, ToyDecaySpec(h, raw["decay"]), norm, ffn, names(1)))
        # layer 0, layer 1, layer 0 again with a cache of its own, layer 0 reading run 0's cache
        schedule = (RunSpec(0), RunSpec(1), RunSpec(0), RunSpec(1), RunSpec(0, cache_of=0))
        return ModelSpec(raw["vocab"], h, layers, schedule, norm, True, 4096, (), "emb.weight", "fnorm", "head.weight")

    register_architecture(Architecture("ToyForCausalLM", lambda raw: raw, spec_of), replace=True)


def toy_plain(ids, w, raw):
    """Whole-sequence restatement of the toy model with plain torch ops."""
    h = w["emb.weight"][torch.tensor(ids)]
    n, eps = len(ids), raw["eps"]

    def norm(x, name):
        return plain.rms_norm(x, w[name + ".weight"], eps)

    def ffn(x, p):
        return plain.feed_forward(x, w, p)

    def attn(x, p, kv_from=None):
        q = (x @ w[p + ".q_proj.weight"].t()).view(n, 4, 16)
        src = x if kv_from is None else kv_from
        k = (src @ w[p + ".k_proj.weight"].t()).view(n, 2, 16).repeat_interleave(2, 1)
        v = (src @ w[p + ".v_proj.weight"].t()).view(n, 2, 16).repeat_interleave(2, 1)
        s = torch.einsum("thd,shd->hts", q, k) * 0.3
        s = s + plain.causal_mask(n, s.dtype)
        o = torch.einsum("hts,shd->thd", torch.softmax(s, -1), v).reshape(n, 64)
        return o @ w[p + ".o_proj.weight"].t()

    def decay(x, p):
        u = x @ w[p + ".w.weight"].t()
        out, s = [], torch.zeros(x.shape[1])
        for i in range(n):
            s = raw["decay"] * s + u[i]
            out.append(s)
        return torch.stack(out)

    first_norm_input = None
    for run, layer in enumerate((0, 1, 0, 1, 0)):
        p = f"l{layer}"
        x = norm(h, p + ".n1")
        if run == 0:
            first_norm_input = x
        if layer == 1:
            h = h + decay(x, p + ".mix")
        elif run == 4:
            h = h + attn(x, p + ".mix", kv_from=first_norm_input)   # reads run 0's keys and values
        else:
            h = h + attn(x, p + ".mix")
        h = h + ffn(norm(h, p + ".n2"), p + ".ffn")
    return norm(h, "fnorm") @ w["emb.weight"].t()


def test_toy_architecture_registers_builds_and_steps(fe, tmp_path) -> None:
    from forge_engine_b200.engine import ModelRunner, StepEntry
    from forge_engine_b200.models import expected_tensors
    from forge_engine_b200.config import read_model_config
    from forge_engine_b200.weights import random_tensors, write_model_folder

    register_toy()
    raw = {"architectures": ["ToyForCausalLM"], "hidden_size": 64, "inter": 72, "vocab": 97, "eps": 1e-5, "decay": 0.8}
    _, _, spec = read_model_config(raw)
    tensors = random_tensors(expected_tensors(spec), seed=1, std=0.1)
    write_model_folder(tmp_path / "toy", raw, tensors)
    runner = ModelRunner.from_folder(tmp_path / "toy", dtype="float32", page_size=4, num_pages=64, max_requests=3)
    # two attention caches of their own (runs 0 and 2; run 4 shares run 0's), one state per decay run
    assert [g.units for g in runner.cache.groups] == [[0, 2]]
    assert runner.cache.state_of_run(1) is not runner.cache.state_of_run(3)
    w = {k: v.float() for k, v in tensors.items()}
    a, b = random_ids(97, 23, 1), random_ids(97, 14, 2)
    ref_a, ref_b = toy_plain(a, w, raw), toy_plain(b, w, raw)
    runner.begin("a")
    whole = runner.step([StepEntry("a", a, range(23))]).cpu()
    torch.testing.assert_close(whole, ref_a, atol=5e-5, rtol=1e-4)
    runner.end("a")
    # in portions, mixed with another request; slots are reused
    runner.begin("b"), runner.begin("a")
    rows_a, rows_b = [], []
    cuts_a, cuts_b = [9, 2, 1, 11], [3, 1, 10]
    sa = sb = 0
    for step in range(4):
        entries = [StepEntry("a", a[sa : sa + cuts_a[step]], range(cuts_a[step]))]
        if step < 3:
            entries.append(StepEntry("b", b[sb : sb + cuts_b[step]], range(cuts_b[step])))
        out = runner.step(entries).cpu()
        rows_a.append(out[: cuts_a[step]])
        if step < 3:
            rows_b.append(out[cuts_a[step] :])
            sb += cuts_b[step]
        sa += cuts_a[step]
    runner.check_status()
    torch.testing.assert_close(torch.cat(rows_a), ref_a, atol=5e-5, rtol=1e-4)
    torch.testing.assert_close(torch.cat(rows_b), ref_b, atol=5e-5, rtol=1e-4)
    runner.end("a"), runner.end("b")
    runner.cache.check_consistency()


# ---------------------------------------------------------------------------
# more toy parts defined here: a feed-forward with routing and another position encoding
# ---------------------------------------------------------------------------

@dataclass(frozen=True)
class ToyRoutedSpec:
    hidden_size: int
    inter: int
    experts: int
    kind: str = "toy_routed_ffn"


@dataclass(frozen=True)
class ToyScaleSpec:
    q_rate: float
    k_rate: float
    kind: str = "toy_scale_position"


def register_toy_routed():
    from forge_engine_b200.config import (Architecture, AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, NormSpec,
                                          RotarySpec, RunSpec, register_architecture)
    from forge_engine_b200.parts import FeedForward, PositionEncoding, WeightInfo, register_part

    class ToyRoutedFFN(FeedForward):
        """Router logits in 32-bit, the best expert per token, its output weighted by the
        expert's softmax probability: y = p_e * relu(x W1_e^T) W2_e^T."""

        def __init__(self, spec, weights, ctx):
            self.spec, self.dtype = spec, ctx.dtype
            self.router = weights["router.weight"].float()
            self.w1 = [weights[f"experts.{e}.w1.weight"].float() for e in range(spec.experts)]
            self.w2 = [weights[f"experts.{e}.w2.weight"].float() for e in range(spec.experts)]

        @classmethod
        def weight_shapes(cls, spec):
            shapes = {"router.weight": WeightInfo((spec.experts, spec.hidden_size))}
            for e in range(spec.experts):
                shapes[f"experts.{e}.w1.weight"] = WeightInfo((spec.inter, spec.hidden_size))
                shapes[f"experts.{e}.w2.weight"] = WeightInfo((spec.hidden_size, spec.inter))
            return shapes

        def forward(self, x):
            x = x.float()
            prob = torch.softmax(x @ self.router.t(), -1)
            best = prob.argmax(-1)
            out = torch.zeros_like(x)
            for e in range(self.spec.experts):
                rows = (best == e).nonzero().flatten()
                if rows.numel():
                    y = torch.relu(x[rows] @ self.w1[e].t()) @ self.w2[e].t()
                    out[rows] = prob[rows, e : e + 1] * y
            return out.to(self.dtype)

    class ToyScalePosition(PositionEncoding):
        """Queries grow and keys shrink with their position: q *= 1 + q_rate * pos,
        k /= 1 + k_rate * pos (no rotation)."""

        def __init__(self, spec, weights, ctx):
            self.spec = spec

        @classmethod
        def weight_shapes(cls, spec):
            return {}

        def apply(self, qkv, num_q_heads, num_kv_heads, head_dim, batch) -> None:
            pos = batch.positions.to(torch.float32).unsqueeze(1)
            q_end, k_end = num_q_heads * head_dim, (num_q_heads + num_kv_heads) * head_dim
            qkv[:, :q_end] = (qkv[:, :q_end].float() * (1 + self.spec.q_rate * pos)).to(qkv.dtype)
            qkv[:, q_end:k_end] = (qkv[:, q_end:k_end].float() / (1 + self.spec.k_rate * pos)).to(qkv.dtype)

    register_part("toy_routed_ffn", ToyRoutedFFN, replace=True)
    register_part("toy_scale_position", ToyScalePosition, replace=True)

    def spec_of(raw: dict) -> ModelSpec:
        h, eps = raw["hidden_size"], raw["eps"]
        norm = NormSpec(h, eps)
        scaled = AttentionSpec(h, 6, 3, 16, False, eps, False, 0.25, ToyScaleSpec(0.03, 0.05), None)
        rotary = AttentionSpec(h, 6, 3, 16, True, eps, False, 0.25, RotarySpec(16, 1e4, 16), None)

        def names(i):
            return {"input_norm": f"l{i}.n1", "mixer": f"l{i}.mix", "post_norm": f"l{i}.n2", "ffn": f"l{i}.ffn"}

        layers = (LayerSpec(norm, scaled, norm, ToyRoutedSpec(h, raw["inter"], raw["experts"]), names(0)),
                  LayerSpec(norm, rotary, norm, GatedMLPSpec(h, raw["inter"]), names(1)))
        schedule = (RunSpec(0), RunSpec(1))
        return ModelSpec(raw["vocab"], h, layers, schedule, norm, True, 4096, (), "emb.weight", "fnorm", "head.weight")

    register_architecture(Architecture("ToyRoutedForCausalLM", lambda raw: raw, spec_of), replace=True)


def toy_routed_plain(ids, w, raw):
    """Whole-sequence restatement with plain torch ops."""
    h = w["emb.weight"][torch.tensor(ids)]
    n, eps = len(ids), raw["eps"]
    pos = torch.arange(n, dtype=torch.float32)

    def norm(x, name):
        return plain.rms_norm(x, w[name + ".weight"], eps)

    def heads(x, p, which, count):
        return (x @ w[f"{p}.{which}_proj.weight"].t()).view(n, count, 16)

    def attend(q, k, v):
        k, v = k.repeat_interleave(2, 1), v.repeat_interleave(2, 1)
        s = torch.einsum("thd,shd->hts", q, k) * 0.25 + plain.causal_mask(n, q.dtype)
        return torch.einsum("hts,shd->thd", torch.softmax(s, -1), v).reshape(n, 96)

    # layer 0: scaled positions, routed feed-forward
    x = norm(h, "l0.n1")
    q, k, v = heads(x, "l0.mix", "q", 6), heads(x, "l0.mix", "k", 3), heads(x, "l0.mix", "v", 3)
    q = q * (1 + 0.03 * pos)[:, None, None]
    k = k / (1 + 0.05 * pos)[:, None, None]
    h = h + attend(q, k, v) @ w["l0.mix.o_proj.weight"].t()
    x = norm(h, "l0.n2")
    prob = torch.softmax(x @ w["l0.ffn.router.weight"].t(), -1)
    best = prob.argmax(-1)
    update = torch.zeros_like(x)
    for t in range(n):
        e = int(best[t])
        y = torch.relu(x[t] @ w[f"l0.ffn.experts.{e}.w1.weight"].t()) @ w[f"l0.ffn.experts.{e}.w2.weight"].t()
        update[t] = prob[t, e] * y
    h = h + update
    # layer 1: per-head norms, rotation, gated feed-forward
    x = norm(h, "l1.n1")
    q, k, v = heads(x, "l1.mix", "q", 6), heads(x, "l1.mix", "k", 3), heads(x, "l1.mix", "v", 3)
    q = plain.rms_norm(q, w["l1.mix.q_norm.weight"], eps)
    k = plain.rms_norm(k, w["l1.mix.k_norm.weight"], eps)
    cos, sin = plain.rotary_tables(torch.arange(n), 16, 1e4, torch.float32)
    q, k = plain.apply_rotary(q.transpose(0, 1), cos, sin).transpose(0, 1), plain.apply_rotary(k.transpose(0, 1), cos, sin).transpose(0, 1)
    h = h + attend(q, k, v) @ w["l1.mix.o_proj.weight"].t()
    h = h + plain.feed_forward(norm(h, "l1.n2"), w, "l1.ffn")
    return norm(h, "fnorm") @ w["emb.weight"].t()


def test_toy_routed_feed_forward_and_position_encoding(fe, tmp_path) -> None:
    """A feed-forward with routing and a position encoding of another kind, registered from
    here, built layer by layer next to the package's own parts, and stepped whole and in
    portions beside another request."""
    from forge_engine_b200.config import read_model_config
    from forge_engine_b200.engine import ModelRunner, StepEntry
    from forge_engine_b200.models import expected_tensors
    from forge_engine_b200.weights import random_tensors, write_model_folder

    register_toy_routed()
    raw = {"architectures": ["ToyRoutedForCausalLM"], "hidden_size": 80, "inter": 56, "experts": 3, "vocab": 101,
           "eps": 1e-5}
    _, _, spec = read_model_config(raw)
    tensors = random_tensors(expected_tensors(spec), seed=3, std=0.15)
    write_model_folder(tmp_path / "toy2", raw, tensors)
    runner = ModelRunner.from_folder(tmp_path / "toy2", dtype="float32", page_size=4, num_pages=48, max_requests=2)
    w = {k: v.float() for k, v in tensors.items()}
    a, b = random_ids(101, 21, 5), random_ids(101, 12, 6)
    ref_a, ref_b = toy_routed_plain(a, w, raw), toy_routed_plain(b, w, raw)
    runner.begin("a")
    whole = runner.step([StepEntry("a", a, range(21))]).cpu()
    torch.testing.assert_close(whole, ref_a, atol=5e-5, rtol=1e-4)
    runner.end("a")
    runner.begin("a"), runner.begin("b")
    rows_a, rows_b = [], []
    cuts_a, cuts_b = [7, 2, 12], [1, 9, 2]
    sa = sb = 0
    for step in range(3):
        out = runner.step([StepEntry("a", a[sa : sa + cuts_a[step]], range(cuts_a[step])),
                           StepEntry("b", b[sb : sb + cuts_b[step]], range(cuts_b[step]))]).cpu()
        rows_a.append(out[: cuts_a[step]])
        rows_b.append(out[cuts_a[step] :])
        sa += cuts_a[step]
        sb += cuts_b[step]
    runner.check_status()
    torch.testing.assert_close(torch.cat(rows_a), ref_a, atol=5e-5, rtol=1e-4)
    torch.testing.assert_close(torch.cat(rows_b), ref_b, atol=5e-5, rtol=1e-4)
    runner.end("a"), runner.end("b")
    runner.cache.check_consistency()


# ---------------------------------------------------------------------------
# a third toy: a model assembled by its architecture (scaled embedding), an arrangement
# that runs mixer and feed-forward side by side (no attribute named "mixer"), and a mixer
# with state of its own whose decode steps are replayed from CUDA graphs beside filler entries
# ---------------------------------------------------------------------------

@dataclass(frozen=True)
class ToyRunningSpec:
    hidden_size: int
    decay: float
    kind: str = "toy_running_mixer"


def register_toy_parallel():
    from forge_engine_b200.cache import CacheNeeds, StateSpec
    from forge_engine_b200.config import (Architecture, AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec,
                                          NoPositionSpec, NormSpec, RunSpec, register_architecture)
    from forge_engine_b200.models import DecoderModel
    from forge_engine_b200.ops import native
    from forge_engine_b200.parts import Mixer, WeightInfo, build_part, part_class, register_arrangement, register_part

    class ToyRunningMixer(Mixer):
        """s_t = decay * s_{t-1} + x_t W^T ; y_t = s_t, the state s per request.  A step of
        single tokens touches the state only through the device tensor ``batch.slots``, so it
        can be captured and replayed; filler entries of a replayed batch carry the null slot."""

        graph_safe = True

        def __init__(self, spec, weights, ctx):
            self.spec, self.w, self.dtype = spec, weights["w.weight"].float(), ctx.dtype

        @classmethod
        def weight_shapes(cls, spec):
            return {"w.weight": WeightInfo((spec.hidden_size, spec.hidden_size))}

        def cache_needs(self):
            return CacheNeeds(state=StateSpec((self.spec.hidden_size,), "float32"))

        def forward(self, x, batch, cache):
            u = x.float() @ self.w.t()
            if batch.max_new == 1:
                slots = batch.slots.long()
                s = self.spec.decay * cache.state.index_select(0, slots) + u
                cache.state.index_copy_(0, slots, s)
                return s.to(self.dtype)
            out = torch.empty_like(u)
            row = 0
            for slot, _, count in batch.entries:
                s = cache.state[slot]
                for i in range(row, row + count):
                    s = self.spec.decay * s + u[i]
                    out[i] = s
                cache.state[slot] = s
                row += count
            return out.to(self.dtype)

    class ParallelBlock:
        """h += token_mixer(norm(h)) + ffn(norm(h)): one norm, both parts read its output."""

        roles = ("input_norm", "mixer", "ffn")

        def __init__(self, spec, weights, ctx):
            self.norm = build_part(spec.input_norm, weights["input_norm"], ctx)
            self.token_mixer = build_part(spec.mixer, weights["mixer"], ctx)
            self.ffn = build_part(spec.ffn, weights["ffn"], ctx)

        @classmethod
        def weight_shapes(cls, spec):
            return {role: part_class(getattr(spec, role)).weight_shapes(getattr(spec, role)) for role in cls.roles}

        def cache_needs(self):
            return self.token_mixer.cache_needs()

        @property
        def graph_safe(self):
            return self.norm.graph_safe and self.token_mixer.graph_safe and self.ffn.graph_safe

        def forward(self, h, pending, batch, cache):
            normed = self.norm.add_forward(h, pending)
            return self.token_mixer.forward(normed, batch, cache) + self.ffn.forward(normed)

    class ScaledEmbeddingModel(DecoderModel):
        """The decoder with its embedding multiplied by a constant of the configuration."""

        def __init__(self, spec, weights, ctx, multiplier):
            super().__init__(spec, weights, ctx)
            self.multiplier = multiplier

        def forward(self, batch, cache):
            batch.shared.clear()
            h = torch.empty((batch.n_tokens, self.spec.hidden_size), dtype=torch.float32, device=self.ctx.device)
            native.embedding(batch.token_ids, self.embed, h, self.ctx.status)
            h.mul_(self.multiplier)
            pending = None
            for index, run in enumerate(self.spec.schedule):
                pending = self.blocks[run.layer].forward(h, pending, batch, cache.view(index))
            normed = self.final_norm.add_forward(h, pending, row_map=batch.want_rows)
            return self.head(normed, out_dtype=torch.float32)

    register_part("toy_running_mixer", ToyRunningMixer, replace=True)
    register_arrangement("toy_parallel", ParallelBlock, replace=True)
    multipliers = {}

    def spec_of(raw: dict) -> ModelSpec:
        h = raw["hidden_size"]
        norm = NormSpec(h, raw["eps"])
        ffn = GatedMLPSpec(h, raw["inter"])
        layers = [LayerSpec(norm, ToyRunningSpec(h, raw["decay"]), None, ffn,
                            {"input_norm": "l0.n", "mixer": "l0.mix", "ffn": "l0.ffn"}, "toy_parallel")]
        if raw["attention"]:
            attn = AttentionSpec(h, 4, 2, 16, False, raw["eps"], False, 0.3, NoPositionSpec(), None)
            layers.append(LayerSpec(norm, attn, norm, ffn,
                                    {"input_norm": "l1.n1", "mixer": "l1.mix", "post_norm": "l1.n2", "ffn": "l1.ffn"}))
        schedule = tuple(RunSpec(i) for i in range(len(layers))) + (RunSpec(0),)     # the stateful layer runs twice
        spec = ModelSpec(raw["vocab"], h, tuple(layers), schedule, norm, True, 4096, (), "emb.weight", "fnorm", "head.weight")
        multipliers[id(spec)] = raw["embedding_multiplier"]
        return spec

    def assemble(spec, weights, ctx):
        return ScaledEmbeddingModel(spec, weights, ctx, multipliers[id(spec)])

    register_architecture(Architecture("ToyParallelForCausalLM", lambda raw: raw, spec_of, assemble=assemble), replace=True)


def toy_parallel_plain(ids, w, raw):
    h = w["emb.weight"][torch.tensor(ids)] * raw["embedding_multiplier"]
    n, eps = len(ids), raw["eps"]

    def norm(x, name):
        return plain.rms_norm(x, w[name + ".weight"], eps)

    def running(x, p):
        u = x @ w[p + ".w.weight"].t()
        out, s = [], torch.zeros(x.shape[1])
        for i in range(n):
            s = raw["decay"] * s + u[i]
            out.append(s)
        return torch.stack(out)

    def parallel(h):
        x = norm(h, "l0.n")
        return h + running(x, "l0.mix") + plain.feed_forward(x, w, "l0.ffn")

    h = parallel(h)
    if raw["attention"]:
        x = norm(h, "l1.n1")
        q = (x @ w["l1.mix.q_proj.weight"].t()).view(n, 4, 16)
        k = (x @ w["l1.mix.k_proj.weight"].t()).view(n, 2, 16).repeat_interleave(2, 1)
        v = (x @ w["l1.mix.v_proj.weight"].t()).view(n, 2, 16).repeat_interleave(2, 1)
        s = torch.einsum("thd,shd->hts", q, k) * 0.3 + plain.causal_mask(n, q.dtype)
        h = h + torch.einsum("hts,shd->thd", torch.softmax(s, -1), v).reshape(n, 64) @ w["l1.mix.o_proj.weight"].t()
        h = h + plain.feed_forward(norm(h, "l1.n2"), w, "l1.ffn")
    h = parallel(h)          # the same layer again, with a state of its own for this run
    return norm(h, "fnorm") @ w["emb.weight"].t()


@pytest.mark.parametrize("attention", [True, False])
def test_toy_stateful_mixer_replayed_from_graphs_beside_fillers(fe, tmp_path, attention) -> None:
    """Registered from this file alone.  Three requests decode together: the batch is padded
    to four entries and replayed from a CUDA graph; the filler's state goes to the null slot,
    not to the slot of a live request.  Without the attention layer the model keeps no pages
    at all, only state."""
    from forge_engine_b200.config import read_model_config
    from forge_engine_b200.engine import ModelRunner, StepEntry
    from forge_engine_b200.weights import random_tensors, write_model_folder

    register_toy_parallel()
    raw = {"architectures": ["ToyParallelForCausalLM"], "hidden_size": 64, "inter": 80, "vocab": 89, "eps": 1e-5,
           "decay": 0.7, "embedding_multiplier": 3.0, "attention": attention}
    arch, _, spec = read_model_config(raw)
    tensors = random_tensors(arch.expected_tensors(spec), seed=4, std=0.1)
    write_model_folder(tmp_path / "toy3", raw, tensors)
    runner = ModelRunner.from_folder(tmp_path / "toy3", dtype="float32", page_size=4, num_pages=64, max_requests=3)
    assert type(runner.model).__name__ == "ScaledEmbeddingModel" and runner.use_graphs
    assert len(runner.cache.groups) == (1 if attention else 0)
    assert runner.cache.state_of_run(0).shape == (4, 64)            # three requests and the null slot
    w = {k: v.float() for k, v in tensors.items()}
    ids = {k: random_ids(89, n, 40 + n) for k, n in (("a", 30), ("b", 17), ("c", 22))}
    refs = {k: toy_parallel_plain(v, w, raw) for k, v in ids.items()}
    fed = {"a": 9, "b": 2, "c": 6}
    for k in ids:                                                    # a holds slot 0, the slot a filler must not touch
        runner.begin(k)
        out = runner.step([StepEntry(k, ids[k][: fed[k]], range(fed[k]))]).cpu()
        torch.testing.assert_close(out, refs[k][: fed[k]], atol=5e-5, rtol=1e-4)
    assert runner.cache.request("a").slot == 0
    live = ["a", "b", "c"]
    while live:
        out = runner.step([StepEntry(k, [ids[k][fed[k]]], [0]) for k in live]).cpu()
        for row, k in enumerate(live):
            torch.testing.assert_close(out[row], refs[k][fed[k]], atol=5e-5, rtol=1e-4)
            fed[k] += 1
        for k in [k for k in live if fed[k] == len(ids[k])]:
            runner.end(k)
            live.remove(k)
    runner.check_status()
    assert {key[0] for key in runner.graphs.captured} == {4, 2, 1}   # 3 live (one filler), then 2, then 1
    runner.cache.check_consistency()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_replay_equals_eager_steps(fe, dtype, tmp_path) -> None:
    """Decode steps replayed from CUDA graphs (padded to bucket sizes, fixed table widths)
    against the same steps launched eagerly, with requests joining and leaving."""
    from forge_engine_b200.engine import ModelRunner, StepEntry

    cfg, weights = make_model_folder(tmp_path / "m", plain.TINY_C, 5)
    ids = {k: random_ids(cfg.vocab_size, n, 30 + n) for k, n in (("a", 150), ("b", 40), ("c", 90))}
    results = {}
    for graphs in (False, True):
        runner = ModelRunner.from_folder(tmp_path / "m", dtype=dtype, page_size=8, num_pages=64, max_requests=4,
                                         use_graphs=graphs)
        assert runner.use_graphs == graphs
        rows = {k: [] for k in ids}
        fed = {"a": 100, "b": 3, "c": 60}
        for k in ids:
            runner.begin(k)
            runner.step([StepEntry(k, ids[k][: fed[k]], [])])
        live = ["a", "b", "c"]
        step = 0
        while live:
            entries = [StepEntry(k, [ids[k][fed[k]]], [0] if (step + i) % 3 else []) for i, k in enumerate(live)]
            out = runner.step(entries).cpu()
            row = 0
            for e in entries:
                if e.want:
                    rows[e.key].append((fed[e.key], out[row].clone()))
                    row += 1
                fed[e.key] += 1
            for k in [k for k in live if fed[k] == len(ids[k])]:
                runner.end(k)
                live.remove(k)
            step += 1
        runner.check_status()
        assert runner.cache.leased_pages() == [0]
        if graphs:
            assert len(runner.graphs.captured) >= 2      # batches of 3 (bucket 4), 2 and 1
        results[graphs] = rows
    for k in ids:
        ref = plain.forward_logits(ids[k], weights, cfg)
        assert len(results[True][k]) == len(results[False][k]) > 10
        for (pos_e, eager), (pos_g, replayed) in zip(results[False][k], results[True][k]):
            assert pos_e == pos_g
            torch.testing.assert_close(replayed, ref[pos_g], **bound(dtype, ref))
            if dtype == "float32":
                assert torch.equal(eager, replayed)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "E"])
def test_mixed_steps_replayed_from_graphs_equal_eager_steps(fe, dtype, name, tmp_path) -> None:
    """Steps that mix prompt portions with decoded tokens are replayed from CUDA graphs too
    (token and entry counts padded to a bucket with filler entries on the null page): the same
    schedule launched eagerly gives the same logits - the same bits in 32-bit - and both agree
    with the plain implementation.  Configuration E has a windowed layer group and head size 64."""
    from forge_engine_b200.engine import ModelRunner, StepEntry

    raw, seed = {"C": (plain.TINY_C, 5), "E": (plain.TINY_E, 7)}[name]
    cfg, weights = make_model_folder(tmp_path / "m", raw, seed)
    ids = {k: random_ids(cfg.vocab_size, n, 60 + n) for k, n in (("a", 140), ("b", 55), ("c", 97), ("d", 23))}
    prompt = {"a": 120, "b": 30, "c": 80, "d": 20}
    portion = (7, 33, 2, 18, 40, 5)
    results = {}
    for graphs in (False, True):
        runner = ModelRunner.from_folder(tmp_path / "m", dtype=dtype, page_size=8, num_pages=96, max_requests=4,
                                         use_graphs=graphs)
        runner.graphs.capture_after = 0          # capture a bucket at first sight (the default waits for the second)
        rows = {k: [] for k in ids}
        fed = {k: 0 for k in ids}
        live, waiting = [], ["a", "b", "c", "d"]
        step = 0
        while live or waiting:
            if waiting and step % 2 == 0:
                key = waiting.pop(0)
                runner.begin(key)
                live.append(key)
            entries = []
            for i, k in enumerate(live):
                if fed[k] < prompt[k]:
                    n = min(portion[(step + i) % len(portion)], prompt[k] - fed[k])
                    want = [n - 1] if fed[k] + n == prompt[k] else []
                else:
                    n, want = 1, [0]
                entries.append(StepEntry(k, ids[k][fed[k] : fed[k] + n], want))
            out = runner.step(entries).cpu()
            row = 0
            for e in entries:
                if e.want:
                    rows[e.key].append((fed[e.key] + len(e.tokens) - 1, out[row].clone()))
                    row += 1
                fed[e.key] += len(e.tokens)
            for k in [k for k in live if fed[k] == len(ids[k])]:
                runner.end(k)
                live.remove(k)
            step += 1
        runner.check_status()
        assert all(n == 0 for n in runner.cache.leased_pages())
        if graphs:
            mixed = [key for key in runner.graphs.captured if key[0] != key[1]]
            assert len(mixed) >= 3, list(runner.graphs.captured)      # several buckets of mixed steps were captured
        results[graphs] = rows
    for k in ids:
        ref = plain.forward_logits(ids[k], weights, cfg)
        assert len(results[True][k]) == len(results[False][k]) >= len(ids[k]) - prompt[k]
        for (pos_e, eager), (pos_g, replayed) in zip(results[False][k], results[True][k]):
            assert pos_e == pos_g
            torch.testing.assert_close(replayed, ref[pos_g], **bound(dtype, ref))
            if dtype == "float32":
                assert torch.equal(eager, replayed)


def test_mixed_step_captured_with_narrow_block_tables(fe, tmp_path) -> None:
    """A bucket's graph is captured with the token split of the step that asks for it: three
    portions of 30 tokens with pages of 4 have block tables of 8 pages, and a capture that put
    nearly all of the bucket's 96 tokens into one filler entry would need 24."""
    from forge_engine_b200.engine import ModelRunner, StepEntry

    cfg, weights = make_model_folder(tmp_path / "m", plain.TINY_B, 2)
    ids = {k: random_ids(cfg.vocab_size, 34, 300 + i) for i, k in enumerate("abc")}
    runner = ModelRunner.from_folder(tmp_path / "m", dtype="float32", page_size=4, num_pages=64, max_requests=3)
    runner.graphs.capture_after = 0
    for k in ids:
        runner.begin(k)
    first = runner.step([StepEntry(k, ids[k][:30], [29]) for k in ids]).cpu()
    assert any(key[:3] == (4, 96, 8) for key in runner.graphs.captured), list(runner.graphs.captured)
    second = runner.step([StepEntry(k, ids[k][30:], [3]) for k in ids]).cpu()
    runner.check_status()
    for row, k in enumerate(ids):
        ref = plain.forward_logits(ids[k], weights, cfg)
        torch.testing.assert_close(first[row], ref[29], **bound("float32", ref))
        torch.testing.assert_close(second[row], ref[33], **bound("float32", ref))


def test_scheduler_run_with_buckets_captured_midway_gives_the_eager_tokens(fe, tmp_path) -> None:
    """A long scheduler run under a small token budget with the default capture policy: the
    buckets of its mixed steps are seen 16 times, captured in the middle of the run and
    replayed from then on.  Configuration D has two windowed layers (pages are given back
    while requests live).  Every request's greedy tokens equal those of the same run launched
    eagerly, and the plain implementation's."""
    from forge_engine_b200.config import EngineConfig, SchedulerConfig
    from forge_engine_b200.engine import Engine, ModelRunner
    from forge_engine_b200.sampling import SamplingParams

    cfg, weights = make_model_folder(tmp_path / "m", dict(plain.TINY_D, eos_token_id=None), 6)
    prompts = [random_ids(cfg.vocab_size, 40, 800 + i) for i in range(40)]
    sched = SchedulerConfig(max_requests=40, max_batch_size=4, token_budget=12, chunk_size=8, block_size=4,
                            block_capacity=200, lookahead=False)
    outputs = {}
    for graphs in (False, True):
        runner = ModelRunner.from_folder(tmp_path / "m", dtype="float32", page_size=4, num_pages=200, max_requests=40,
                                         use_graphs=graphs)
        engine = Engine(runner, EngineConfig(max_new_tokens=5, dtype="float32"), sched)
        outputs[graphs] = engine.generate(prompts, SamplingParams(max_new_tokens=5))
        if graphs:
            assert runner.graphs.capture_after == 16
            mixed = [key for key in runner.graphs.captured if key[0] != key[1]]
            assert mixed, sorted(runner.graphs.seen.items(), key=lambda kv: -kv[1])[:5]
        assert all(n == 0 for n in runner.cache.leased_pages())
    assert outputs[True] == outputs[False]
    for prompt, output in list(zip(prompts, outputs[True]))[:6]:
        assert output == plain.greedy_generate(prompt, 5, weights, cfg)


def test_lookahead_gives_the_same_tokens_as_synchronous_steps(fe, tmp_path) -> None:
    """Decode steps launched one ahead (tokens fed on the device, events one step late)
    against fully synchronous scheduling: same outputs, greedy and sampled, with requests
    that stop on an end-of-sequence id in the middle and a late arrival."""
    from forge_engine_b200.config import EngineConfig, SchedulerConfig
    from forge_engine_b200.engine import Engine
    from forge_engine_b200.sampling import SamplingParams

    # many end-of-sequence ids, so that sampled requests do stop early
    raw = dict(plain.TINY_B, eos_token_id=list(range(300, 384)))
    cfg, weights = make_model_folder(tmp_path / "m", raw, 2)
    prompts = [random_ids(300, n, 70 + n) for n in (5, 12, 3, 20)]
    params = [SamplingParams(max_new_tokens=30), SamplingParams(temperature=1.0, seed=3, max_new_tokens=25),
              SamplingParams(temperature=0.9, top_k=40, seed=9, max_new_tokens=12),
              SamplingParams(temperature=1.2, seed=5, max_new_tokens=30)]
    late_prompt = random_ids(300, 7, 99)
    results = {}
    for lookahead in (False, True):
        engine = Engine.from_pretrained(
            tmp_path / "m", engine_config=EngineConfig(dtype="float32"),
            scheduler_config=SchedulerConfig(block_size=16, block_capacity=32, token_budget=64, max_batch_size=8,
                                             lookahead=lookahead))
        assert engine.scheduler.lookahead == lookahead
        ids = [engine.submit(p, sampling_params=sp) for p, sp in zip(prompts, params)]
        steps = 0
        late = None
        while not engine.scheduler.idle:
            engine.step()
            steps += 1
            if steps == 6:
                late = engine.submit(late_prompt, sampling_params=SamplingParams(max_new_tokens=9))
        views = [engine.scheduler.request(r) for r in ids + [late]]
        results[lookahead] = [(v.output_tokens, v.finish_reason) for v in views]
        snap = engine.scheduler.snapshot()
        assert snap.allocated_blocks == (0,) and snap.reserved_blocks == (0,)
        engine.runner.check_status()
    assert results[True] == results[False]
    reasons = [reason for _, reason in results[True]]
    assert "stop" in reasons and "length" in reasons      # both ways of finishing were exercised
    # the greedy request equals the plain implementation's greedy continuation up to its stop
    greedy_tokens = list(results[True][0][0])
    assert greedy_tokens == plain.greedy_generate(prompts[0], len(greedy_tokens), weights, plain.PlainConfig.from_dict(raw))


def test_arrivals_cancellations_and_few_pages_under_lookahead(fe, tmp_path) -> None:
    """Thirty greedy requests of random lengths arrive while others decode, some are
    cancelled half-way, and the pool is so small that admission has to wait for pages:
    every finished request equals the plain implementation's greedy continuation, and
    every page and slot is back at the end."""
    import random

    from forge_engine_b200.config import EngineConfig, SchedulerConfig
    from forge_engine_b200.engine import Engine
    from forge_engine_b200.sampling import SamplingParams

    cfg, weights = make_model_folder(tmp_path / "m", plain.TINY_A, 0)
    rng = random.Random(11)
    jobs = []
    for i in range(30):
        prompt = random_ids(cfg.vocab_size, rng.randint(1, 60), 500 + i)
        jobs.append((prompt, rng.randint(1, 24), rng.random() < 0.2))       # prompt, new tokens, cancel it?
    engine = Engine.from_pretrained(
        tmp_path / "m", engine_config=EngineConfig(dtype="float32"),
        scheduler_config=SchedulerConfig(max_requests=40, block_size=4, block_capacity=70, token_budget=48, max_batch_size=6,
                                         chunk_size=16, lookahead=True))
    submitted, cancelled = {}, set()
    waiting = list(enumerate(jobs))
    steps = 0
    while waiting or not engine.scheduler.idle:
        # two or three arrivals every few steps
        if waiting and steps % 3 == 0:
            for _ in range(min(len(waiting), rng.randint(1, 3))):
                index, (prompt, new, _) = waiting.pop(0)
                submitted[index] = engine.submit(prompt, sampling_params=SamplingParams(max_new_tokens=new))
        engine.step()
        steps += 1
        for index, rid in submitted.items():
            if jobs[index][2] and index not in cancelled:
                view = engine.scheduler.request(rid)
                if len(view.output_tokens) >= max(1, jobs[index][1] // 2) and not view.finish_reason:
                    engine.cancel(rid)
                    cancelled.add(index)
        assert steps < 3000
    engine.runner.check_status()
    finished = 0
    for index, rid in submitted.items():
        view = engine.scheduler.request(rid)
        prompt, new, _ = jobs[index]
        want = plain.greedy_generate(prompt, new, weights, cfg)
        got = list(view.output_tokens)
        if index in cancelled:
            assert got == want[: len(got)]
        else:
            # generation stops early only on an end-of-sequence id, which is not emitted
            assert got == want[: len(got)] and (len(got) == new or view.finish_reason == "stop")
            finished += 1
    assert finished >= 15 and len(cancelled) >= 3 and finished + len(cancelled) == 30
    snap = engine.scheduler.snapshot()
    assert snap.allocated_blocks == (0,) and snap.reserved_blocks == (0,) and snap.running == 0
    engine.runner.cache.check_consistency()


def test_benchmark_layer_shapes_in_32_bit_and_bfloat16(fe, tmp_path) -> None:
    """Two layers with the layer sizes of the 4B benchmark model (hidden 2560, 32/8 heads of
    128, intermediate 9728, theta 5e6) and a vocabulary that is no multiple of 128: the
    32-bit engine against the plain implementation, whole and cut, and the bfloat16 engine
    (tcgen05 products, tensor-core attention, replayed decode steps) against the same."""
    from forge_engine_b200.engine import ModelRunner, StepEntry

    raw = dict(plain.TINY_A, vocab_size=5003, hidden_size=2560, intermediate_size=9728, num_hidden_layers=2,
               num_attention_heads=32, num_key_value_heads=8, head_dim=128, rope_theta=5e6, rms_norm_eps=1e-6,
               tie_word_embeddings=True, eos_token_id=None)
    cfg, weights = make_model_folder(tmp_path / "m", raw, 11)
    ids = random_ids(cfg.vocab_size, 150, 4)
    ref = plain.forward_logits(ids, weights, cfg)
    for dtype in ("float32", "bfloat16"):
        runner = ModelRunner.from_folder(tmp_path / "m", dtype=dtype, page_size=16, num_pages=40, max_requests=4)
        runner.begin("whole")
        whole = runner.step([StepEntry("whole", ids, range(len(ids)))]).cpu()
        runner.end("whole")
        runner.begin("cut")
        rows = [runner.step([StepEntry("cut", ids[:97], range(97))]).cpu(),
                runner.step([StepEntry("cut", ids[97:118], range(21))]).cpu()]
        rows += [runner.step([StepEntry("cut", [t], [0])]).cpu() for t in ids[118:]]
        cut = torch.cat(rows)
        runner.end("cut")
        runner.check_status()
        if dtype == "float32":
            torch.testing.assert_close(whole, ref, atol=1e-4, rtol=1e-5)
            torch.testing.assert_close(cut, ref, atol=1e-4, rtol=1e-5)
        else:
            for got in (whole, cut):
                torch.testing.assert_close(got, ref, **bound(dtype, ref))
                tv = 0.5 * (torch.softmax(got.double(), -1) - torch.softmax(ref.double(), -1)).abs().sum(-1).max()
                assert float(tv) < 0.02
