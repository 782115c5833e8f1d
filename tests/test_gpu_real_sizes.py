"""The engine at the benchmark model's layer sizes (hidden 2560, 32 query and 8 key/value
heads of 128, intermediate 9728, theta 5e6), where the kernels run that the tiny
configurations never reach: the tcgen05 prefill attention beside the split decode kernel in
one batch, 64-token tiles of the tcgen05 product and the switch to the library product at
65 tokens, the decode kernel that spreads all requests' key tiles over the GPU chosen by
estimate at a replayed batch of 64, and once the full depth of 36 layers under the full
vocabulary of 151,936.

The plain implementation runs on the GPU here (plain torch operators in 32-bit, no TF32)
on the very tensors the engine was built from; on the CPU these checks would take minutes.
Weights are drawn on the device as bfloat16 values, so the 32-bit and the bfloat16 engine
and the plain implementation all hold the same model.
"""

from __future__ import annotations

from collections.abc import Mapping

import pytest
import torch

import plain_qwen3 as plain
import trace_modes
from helpers import random_ids

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

LAYER_SIZES = dict(plain.TINY_A, hidden_size=2560, intermediate_size=9728, num_attention_heads=32,
                   num_key_value_heads=8, head_dim=128, rope_theta=5e6, rms_norm_eps=1e-6,
                   tie_word_embeddings=True, eos_token_id=None, max_position_embeddings=8192)
TWO_LAYERS = dict(LAYER_SIZES, num_hidden_layers=2, vocab_size=5003)
FULL_MODEL = dict(LAYER_SIZES, num_hidden_layers=36, vocab_size=151936)

F32_ATOL = 1e-4          # 32-bit at this width (sums over 2,560 to 9,728 terms)
BF16_REL = 3e-2          # of the largest logit, as in the replay tests
BF16_TV = 2e-2


class Upcast(Mapping):
    """The same tensors raised to 32-bit when they are asked for (exact for bfloat16)."""

    def __init__(self, tensors) -> None:
        self.tensors = tensors

    def __getitem__(self, name):
        return self.tensors[name].float()

    def __iter__(self):
        return iter(self.tensors)

    def __len__(self):
        return len(self.tensors)


class Model:
    """A model drawn on the device, shared by the engines and the plain implementation."""

    def __init__(self, raw: dict, seed: int) -> None:
        from forge_engine_b200.config import read_model_config
        from forge_engine_b200.ops import native
        from forge_engine_b200.weights import RandomTensors

        native.require_cuda()
        native.lib()
        self.raw = raw
        self.cfg = plain.PlainConfig.from_dict(raw)
        self.arch, _, self.spec = read_model_config(raw)
        self.tensors = RandomTensors(self.arch.expected_tensors(self.spec), seed, dtype=torch.bfloat16, device=DEV)

    def runner(self, dtype: str, pages: int, requests: int, graphs: bool = True):
        from forge_engine_b200.engine import ModelRunner

        weights = self.tensors if dtype == "bfloat16" else Upcast(self.tensors)
        return ModelRunner.from_tensors(self.spec, weights, dtype=dtype, device=DEV, page_size=16, num_pages=pages,
                                        max_requests=requests, use_graphs=graphs, architecture=self.arch)

    def plain_logits(self, ids, dtype=torch.float32) -> torch.Tensor:
        """[tokens, vocab] on the CPU, worked out on the GPU by the plain implementation."""
        before = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            return plain.forward_logits(torch.tensor(ids, device=DEV), self.tensors, self.cfg, dtype).float().cpu()
        finally:
            torch.backends.cuda.matmul.allow_tf32 = before


@pytest.fixture(scope="module")
def two_layers():
    return Model(TWO_LAYERS, 11)


def total_variation(a: torch.Tensor, b: torch.Tensor) -> float:
    return float(0.5 * (torch.softmax(a.double(), -1) - torch.softmax(b.double(), -1)).abs().sum(-1).max())


def check_rows(dtype: str, got: torch.Tensor, ref: torch.Tensor, what: str) -> None:
    if dtype == "float32":
        torch.testing.assert_close(got, ref, atol=F32_ATOL, rtol=1e-5, msg=lambda m: f"{what}: {m}")
        return
    bound = BF16_REL * max(1.0, float(ref.abs().max()))
    assert float((got - ref).abs().max()) <= bound, what
    assert total_variation(got, ref) <= BF16_TV, what
    top = torch.topk(ref, 2, dim=-1).values
    clear = (top[:, 0] - top[:, 1]) > 2 * bound
    assert torch.equal(got.argmax(-1)[clear], ref.argmax(-1)[clear]), what


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_trace_with_few_pages(two_layers, dtype) -> None:
    """Up to four live requests, prompt portions of 5 to 70 tokens beside single decoded
    tokens of others in one batch, in a pool that holds just the trace's peak: in bfloat16
    the tcgen05 prefill kernel and the split decode kernel run for the same step."""
    from forge_engine_b200.engine import StepEntry
    from forge_engine_b200.ops import native

    lengths = (150, 97, 210, 64, 131, 180)
    sequences = {f"s{i}": random_ids(5003, n, 300 + i) for i, n in enumerate(lengths)}
    expected = {k: two_layers.plain_logits(v) for k, v in sequences.items()}
    trace = trace_modes.Trace()
    trace_modes.mixed(trace, sequences, chunk=(5, 2, 11, 40, 70))
    runner = two_layers.runner(dtype, pages=trace.peak_tokens // 16, requests=4)
    kinds = set()
    real = native.attention_mma

    def watch(*args, **kwargs):
        # positional: ..., status, run_prefill, run_decode, num_splits
        kinds.add((bool(args[14]), bool(args[15])))
        return real(*args, **kwargs)

    native.attention_mma = watch
    try:
        held: dict = {}
        results = {}
        for step in trace.steps:
            entries = []
            for item in step["entries"]:
                if not runner.cache.has_request(item["id"]):
                    runner.begin(item["id"])
                entries.append(StepEntry(item["id"], item["tokens"], item["want"]))
            results[step["step"]] = runner.step(entries).cpu()
            for key in step["end"]:
                for page in runner.cache.request(key).tables[0].pages:
                    held.setdefault(page, set()).add(key)
                runner.end(key)
        runner.check_status()
    finally:
        native.attention_mma = real
    assert runner.cache.leased_pages() == [0]
    assert max(len(keys) for keys in held.values()) >= 2, "no page was leased a second time"
    if dtype == "bfloat16":
        assert (True, True) in kinds, "no step ran the prefill and the decode kernel together"
    for step, row, key, position in trace.rows:
        check_rows(dtype, results[step][row : row + 1], expected[key][position : position + 1],
                   f"{key}[{position}] in step {step}")
    assert len(trace.rows) > 250


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_of_33_64_and_65_tokens(two_layers, dtype, monkeypatch) -> None:
    """33 and 64 tokens take the 64-token tile of the tcgen05 product; 65 tokens are the
    first that go to the library product.  One request fed 33 + 64 + 65 tokens, a second one beside it in the
    64-token step so that the step is exactly 64 tokens over two entries."""
    from forge_engine_b200.engine import StepEntry
    from forge_engine_b200.ops import native

    # the launch counts below are those of the default settings
    monkeypatch.delenv("FORGE_ENGINE_DECODE_CHAIN", raising=False)
    monkeypatch.delenv("FORGE_ENGINE_SUMMED_QKV", raising=False)
    a, b = random_ids(5003, 33 + 40 + 65, 21), random_ids(5003, 24 + 9, 22)
    ref_a, ref_b = two_layers.plain_logits(a), two_layers.plain_logits(b)
    runner = two_layers.runner(dtype, pages=24, requests=2)
    calls = []
    real = native.gemm_tc5
    monkeypatch.setattr(native, "gemm_tc5", lambda x, *args, **kw: (calls.append(x.shape[0]), real(x, *args, **kw))[1])
    runner.begin("a"), runner.begin("b")
    first = runner.step([StepEntry("a", a[:33], range(33))]).cpu()
    own_33 = list(calls)
    second = runner.step([StepEntry("a", a[33:73], range(40)), StepEntry("b", b[:24], range(24))]).cpu()
    own_64 = calls[len(own_33):]
    seen = len(calls)
    third = runner.step([StepEntry("a", a[73:], range(65))]).cpu()
    fourth = runner.step([StepEntry("b", b[24:], range(9))]).cpu()
    runner.check_status()
    if dtype == "bfloat16":
        # four projections per layer and the output head, all on the tcgen05 kernel ...
        assert own_33 == [33] * 9 and own_64 == [64] * 9
        # ... and none of the 65-token step's (the 9-token step after it is back on it)
        assert calls[seen:] == [9] * 9
    else:
        assert not calls
    check_rows(dtype, torch.cat([first, second[:40], third]), ref_a, "request a")
    check_rows(dtype, torch.cat([second[40:], fourth]), ref_b, "request b")


def test_decode_batch_of_48_uneven_requests_takes_the_balanced_kernel(two_layers, monkeypatch) -> None:
    """48 requests with 300 to 1,500 cached tokens (built by real prefill steps) decode
    together: the batch is padded to the bucket of 64 and replayed from a graph, and the
    estimate - not an override - sends its attention to the kernel that spreads the key
    tiles of all requests evenly over the GPU's blocks.  The same step launched eagerly
    takes that kernel for its real lengths.  Two tokens per request against the plain
    implementation."""
    import random

    from forge_engine_b200.engine import StepEntry

    monkeypatch.delenv("FORGE_ENGINE_DECODE_BALANCED", raising=False)
    rng = random.Random(5)
    lengths = [300, 1500] + [rng.randint(301, 1499) for _ in range(46)]
    sequences = [random_ids(5003, n + 2, 900 + i) for i, n in enumerate(lengths)]
    expected = [two_layers.plain_logits(s)[-2:] for s in sequences]
    for graphs in (True, False):
        runner = two_layers.runner("bfloat16", pages=sum(-(-(n + 2) // 16) for n in lengths), requests=48, graphs=graphs)
        assert runner.use_graphs == graphs
        batch, tokens = [], 0
        for i, (n, ids) in enumerate(zip(lengths, sequences)):
            runner.begin(i)
            batch.append(StepEntry(i, ids[:n], []))
            tokens += n
            if tokens > 6000 or i == len(lengths) - 1:
                runner.step(batch)
                batch, tokens = [], 0
        rows = []
        for t in (0, 1):
            rows.append(runner.step([StepEntry(i, [sequences[i][lengths[i] + t]], [0]) for i in range(48)]).cpu())
        runner.check_status()
        mixers = [block.mixer for block in runner.model.blocks]
        assert all(m.last_splits == 0 for m in mixers), [m.last_splits for m in mixers]
        if graphs:
            assert {key[0] for key in runner.graphs.captured} == {64}
        for i in range(48):
            got = torch.stack([rows[0][i], rows[1][i]])
            check_rows("bfloat16", got, expected[i], f"request {i} of {lengths[i]} tokens")


def test_bfloat16_engine_is_closer_to_32_bit_than_upstreams_bfloat16_flow(two_layers) -> None:
    """The engine keeps the residual stream, the norms' weight product and the rotation
    tables in 32-bit where upstream's bfloat16 model rounds them; so its logits lie nearer
    to the 32-bit model's than the plain implementation's bfloat16 data flow does."""
    from forge_engine_b200.engine import StepEntry

    ids = random_ids(5003, 120, 8)
    exact = two_layers.plain_logits(ids)
    upstream_flow = two_layers.plain_logits(ids, torch.bfloat16)
    runner = two_layers.runner("bfloat16", pages=8, requests=1)
    runner.begin("x")
    mine = runner.step([StepEntry("x", ids, range(len(ids)))]).cpu()
    runner.check_status()
    mine_error = float((mine - exact).abs().mean())
    flow_error = float((upstream_flow - exact).abs().mean())
    print(f"mean |error| against 32-bit: engine {mine_error:.3e}, plain bfloat16 flow {flow_error:.3e}")
    assert mine_error <= flow_error


def test_full_depth_and_vocabulary() -> None:
    """All 36 layers under the tied 151,936-row head, random weights: a 48-token prompt
    whole, and cut 16 + 24 + eight single tokens.  The 32-bit engine against the plain
    implementation in 32-bit (both against the plain implementation in 64-bit, which says how
    much 32-bit rounding alone moves these logits), and the bfloat16 engine against the
    32-bit logits by total variation and greedy agreement, as upstream's integrated check
    does (tools/validate_l4.py:27, 981-1045: prefill, then eight decode steps, each against
    uncached logits, total variation at most 0.05)."""
    from forge_engine_b200.engine import StepEntry

    model = Model(FULL_MODEL, 3)
    ids = random_ids(151936, 48, 5)
    exact = model.plain_logits(ids, torch.float64)
    ref = model.plain_logits(ids)
    plain_noise = float((ref - exact).abs().max())

    def both_ways(runner):
        runner.begin("whole")
        whole = runner.step([StepEntry("whole", ids, range(48))]).cpu()
        runner.end("whole")
        runner.begin("cut")
        rows = [runner.step([StepEntry("cut", ids[:16], range(16))]).cpu(),
                runner.step([StepEntry("cut", ids[16:40], range(24))]).cpu()]
        rows += [runner.step([StepEntry("cut", [t], [0])]).cpu() for t in ids[40:]]
        runner.end("cut")
        runner.check_status()
        return whole, torch.cat(rows)

    runner = model.runner("float32", pages=8, requests=2)
    assert len(runner.model.blocks) == 36 and runner.model.head.out_features == 151936
    whole, cut = both_ways(runner)
    del runner
    bound = max(F32_ATOL, 4.0 * plain_noise)
    for name, got in (("whole", whole), ("cut", cut)):
        error = float((got - exact).abs().max())
        print(f"32-bit {name}: max |error| against 64-bit {error:.3e} (plain 32-bit: {plain_noise:.3e})")
        assert error <= bound, name
        torch.testing.assert_close(got, ref, atol=bound, rtol=1e-5)
    torch.cuda.empty_cache()
    runner = model.runner("bfloat16", pages=8, requests=2)
    whole, cut = both_ways(runner)
    assert any(key[0] == 1 for key in runner.graphs.captured)      # the single tokens were replayed
    for name, got in (("whole", whole), ("cut", cut)):
        tv = total_variation(got, ref)
        print(f"bfloat16 {name}: total variation against 32-bit {tv:.3e}")
        assert tv <= 0.05, name
        top = torch.topk(ref, 2, dim=-1).values
        clear = (top[:, 0] - top[:, 1]) > 2 * BF16_REL * max(1.0, float(ref.abs().max()))
        assert torch.equal(got.argmax(-1)[clear], ref.argmax(-1)[clear]), name


def test_decode_steps_through_the_persistent_chain_kernel(two_layers, monkeypatch) -> None:
    """FORGE_ENGINE_DECODE_CHAIN=1: a layer's output projection, post-attention norm, gate/up
    with SiLU*mul and down projection run as one persistent kernel for steps of up to 16
    tokens (off by default: it measured slower than the separate kernels).  Three requests
    decode together after prompts of different lengths, replayed from a graph, against the
    plain implementation."""
    from forge_engine_b200.engine import StepEntry
    from forge_engine_b200.ops import native

    monkeypatch.setenv("FORGE_ENGINE_DECODE_CHAIN", "1")
    launches = []
    real = native.decode_chain
    monkeypatch.setattr(native, "decode_chain", lambda ops, n, status: (launches.append(n), real(ops, n, status))[1])
    lengths = (70, 9, 33)
    sequences = [random_ids(5003, n + 6, 700 + n) for n in lengths]
    expected = [two_layers.plain_logits(s)[-6:] for s in sequences]
    runner = two_layers.runner("bfloat16", pages=24, requests=3)
    for i, (n, ids) in enumerate(zip(lengths, sequences)):
        runner.begin(i)
        runner.step([StepEntry(i, ids[:n], [])])
    assert launches == [9, 9]                     # only the 9-token prompt is short enough; two layers
    rows = [runner.step([StepEntry(i, [sequences[i][lengths[i] + t]], [0]) for i in range(3)]).cpu() for t in range(6)]
    runner.check_status()
    assert launches[2:] == [4] * 4                # captured once: an eager pass and the capture, two layers, bucket of 4
    for i in range(3):
        check_rows("bfloat16", torch.stack([rows[t][i] for t in range(6)]), expected[i], f"request {i}")


@pytest.mark.parametrize("dtype,length", [("float32", 3000), ("bfloat16", 6000)])
def test_long_context_in_portions_then_decoding(two_layers, dtype, length) -> None:
    """A prompt of several thousand tokens fed in portions of 2,048 (block tables hundreds of
    pages wide, prefill portions that start thousands of tokens into the request), then
    decoded tokens whose attention is split 16 to 32 ways; beside it a short request, so that
    the decode steps hold very uneven contexts.  Logits at the ends of the portions and of
    every decoded token against the plain implementation."""
    from forge_engine_b200.engine import StepEntry

    long_ids = random_ids(5003, length + 5, 41)
    short_ids = random_ids(5003, 40 + 5, 42)
    ref_long, ref_short = two_layers.plain_logits(long_ids), two_layers.plain_logits(short_ids)
    runner = two_layers.runner(dtype, pages=-(-(length + 5) // 16) + 8, requests=2)
    runner.begin("long"), runner.begin("short")
    fed, rows, wanted = 0, [], []
    while fed < length:
        n = min(2048, length - fed)
        rows.append(runner.step([StepEntry("long", long_ids[fed : fed + n], [0, n - 1])]).cpu())
        wanted += [fed, fed + n - 1]
        fed += n
    check_rows(dtype, torch.cat(rows), ref_long[wanted], "ends of the long prompt's portions")
    out = runner.step([StepEntry("short", short_ids[:40], [39])]).cpu()
    check_rows(dtype, out, ref_short[39:40], "short prompt")
    for t in range(5):
        out = runner.step([StepEntry("long", [long_ids[length + t]], [0]),
                           StepEntry("short", [short_ids[40 + t]], [0])]).cpu()
        check_rows(dtype, out[0:1], ref_long[length + t : length + t + 1], f"long request, decoded token {t}")
        check_rows(dtype, out[1:2], ref_short[40 + t : 41 + t], f"short request, decoded token {t}")
    runner.check_status()
    if dtype == "bfloat16":
        assert any(key[2] >= 256 for key in runner.graphs.captured)       # block tables of 376 pages: bucket 512
