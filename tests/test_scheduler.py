"""The scheduler's decisions, with a fake step function on the CPU."""

from __future__ import annotations

import pytest
import torch

from forge_engine_b200.cache import CacheManager, CacheNeeds, PagedKVSpec
from forge_engine_b200.config import SchedulerConfig
from forge_engine_b200.engine.scheduler import RequestStatus, Scheduler
from forge_engine_b200.errors import KVCacheCapacityError, OverloadedError
from forge_engine_b200.sampling import SamplingParams

VOCAB = 32


class FakeRunner:
    """Keeps the real cache bookkeeping; logits make argmax = (last token + 1) % VOCAB."""

    def __init__(self, page_size=4, num_pages=16, max_requests=8, window=None, fail_on_step=None):
        needs = [CacheNeeds(kv=PagedKVSpec(1, 16, window))]
        self.cache = CacheManager(needs, page_size=page_size, num_pages=num_pages, max_requests=max_requests)
        self.batches = []
        self.fail_on_step = fail_on_step

    def step(self, entries):
        self.batches.append([(e.key, len(e.tokens), tuple(e.want)) for e in entries])
        if self.fail_on_step is not None and len(self.batches) == self.fail_on_step:
            raise KVCacheCapacityError("injected")
        rows = []
        for e in entries:
            request = self.cache.request(e.key)
            self.cache.reserve(e.key, request.length + len(e.tokens))
            self.cache.advance(e.key, request.length + len(e.tokens))
            for w in e.want:
                row = torch.zeros(VOCAB)
                row[(int(e.tokens[w]) + 1) % VOCAB] = 1.0
                rows.append(row)
        return torch.stack(rows) if rows else torch.zeros((0, VOCAB))


class ArgmaxSampler:
    def sample_to_host(self, logits, params, seeds, counters):
        self.last = (list(seeds), list(counters))
        return logits.argmax(-1).tolist()


def make(config=None, eos=(), **runner_args):
    runner = FakeRunner(**runner_args)
    scheduler = Scheduler(runner, ArgmaxSampler(), config or SchedulerConfig(block_size=4, block_capacity=16),
                          SamplingParams(max_new_tokens=4), eos_token_ids=eos, seed=0)
    return runner, scheduler


def test_generates_and_returns_everything() -> None:
    runner, s = make()
    rid = s.submit([3, 4, 5])
    events = s.run_until_idle()
    view = s.request(rid)
    assert view.status is RequestStatus.FINISHED and view.finish_reason == "length"
    assert view.output_tokens == (6, 7, 8, 9)
    assert [e.tokens for e in events] == [(6,), (7,), (8,), (9,)]
    # prompt in one step, then 3 decode steps: the last sampled token is never fed back
    assert [b[0][1] for b in runner.batches] == [3, 1, 1, 1]
    snap = s.snapshot()
    assert snap.reserved_blocks == (0,) and snap.allocated_blocks == (0,) and snap.terminal == 1
    runner.cache.check_consistency()
    assert view.reserved_blocks == (0,)


def test_prompts_are_cut_under_the_token_budget_and_decodes_go_first() -> None:
    config = SchedulerConfig(block_size=4, block_capacity=64, token_budget=8, max_batch_size=4, chunk_size=6)
    runner, s = make(config, num_pages=64)
    a = s.submit(list(range(1, 4)), request_id="a")            # 3 tokens
    s.step()
    assert runner.batches[-1] == [("a", 3, (2,))]
    b = s.submit(list(range(1, 18)), request_id="b")           # 17 tokens
    s.step()
    # a decodes (1 token) first; b gets min(17, chunk 6, budget 7) = 6, wants nothing yet
    assert runner.batches[-1] == [("a", 1, (0,)), ("b", 6, ())]
    s.step()
    assert runner.batches[-1] == [("a", 1, (0,)), ("b", 6, ())]
    s.step()
    # a samples its 4th and last token here; b feeds its last 5 and wants the final place
    assert s.request(a).status is RequestStatus.FINISHED
    assert runner.batches[-1] == [("a", 1, (0,)), ("b", 5, (4,))]
    assert s.request(b).status is RequestStatus.RUNNING and s.request(b).fed_tokens == 17
    assert all(sum(n for _, n, _ in batch) <= 8 for batch in runner.batches)
    snap = s.snapshot()
    assert (snap.last_prefill_tokens, snap.last_decode_tokens, snap.last_batch_tokens) == (5, 1, 6)
    assert (snap.model_steps, snap.prefill_tokens, snap.decode_tokens) == (4, 3 + 17, 3)
    assert snap.sampled_tokens == 5 and snap.last_step_ms > 0.0
    s.run_until_idle()
    snap = s.snapshot()
    assert snap.allocated_blocks == (0,)
    # every sampled token but the last of each request is fed back as one decoded token
    assert snap.sampled_tokens == 8 and snap.decode_tokens == 6 and snap.prefill_tokens == 20


def test_round_robin_and_max_batch_size() -> None:
    config = SchedulerConfig(block_size=4, block_capacity=64, token_budget=64, max_batch_size=2)
    runner, s = make(config, num_pages=64)
    for name in "abc":
        s.submit([1, 2], request_id=name, sampling_params=SamplingParams(max_new_tokens=3))
    s.step()
    assert [k for k, _, _ in runner.batches[-1]] == ["a", "b"]
    s.step()   # order is now c, a, b: c's prompt and a's decode; the decoded token stands first
    assert runner.batches[-1] == [("a", 1, (0,)), ("c", 2, (1,))]
    s.step()   # order b, c, a
    assert [k for k, _, _ in runner.batches[-1]] == ["b", "c"]
    s.run_until_idle()
    assert all(s.request(n).status is RequestStatus.FINISHED for n in "abc")


def test_fair_rotation_among_decoders() -> None:
    config = SchedulerConfig(block_size=4, block_capacity=64, token_budget=64, max_batch_size=2)
    runner, s = make(config, num_pages=64)
    for name in "abc":
        s.submit([1], request_id=name, sampling_params=SamplingParams(max_new_tokens=50))
    s.step()  # a, b prefill
    s.step()  # decoders a, b first -> c starves unless rotation works
    s.step()
    s.step()
    served = [k for batch in runner.batches for k, _, _ in batch]
    assert "c" in served
    counts = {n: served.count(n) for n in "abc"}
    assert max(counts.values()) - min(counts.values()) <= 2


def test_eos_stops_and_is_not_emitted() -> None:
    runner, s = make(eos=(7,))
    rid = s.submit([4])
    s.run_until_idle()
    view = s.request(rid)
    assert view.output_tokens == (5, 6) and view.finish_reason == "stop" and view.sampled_tokens == 3


def test_admission_queues_until_pages_return() -> None:
    # 8 pages of 4 tokens; each request reserves ceil((6 + 4) / 4) = 3 pages -> two fit, the third waits
    config = SchedulerConfig(block_size=4, block_capacity=8, token_budget=64, max_batch_size=8)
    runner, s = make(config, num_pages=8)
    ids = [s.submit([1, 2, 3, 4, 5, 6], request_id=n) for n in "abc"]
    s.step()
    snap = s.snapshot()
    assert snap.queued == 1 and snap.reserved_blocks == (6,)
    assert [k for k, _, _ in runner.batches[-1]] == ["a", "b"]
    first_pages = set(runner.cache.request("a").tables[0].pages)
    while not s.request("a").status.terminal:
        s.step()
    s.step()
    assert runner.cache.has_request("c")
    # c got pages that a or b held before: pages are used again
    s.run_until_idle()
    assert s.request("c").status is RequestStatus.FINISHED
    assert s.snapshot().reserved_blocks == (0,) and runner.cache.leased_pages() == [0]
    assert first_pages


def test_refuses_what_can_never_fit_and_the_request_bound() -> None:
    config = SchedulerConfig(block_size=4, block_capacity=4, max_requests=2)
    runner, s = make(config, num_pages=4)
    with pytest.raises(OverloadedError, match="needs 5 KV blocks"):
        s.submit(list(range(16)))
    with pytest.raises(ValueError, match="non-empty"):
        s.submit([])
    s.submit([1], request_id="x")
    with pytest.raises(ValueError, match="duplicate"):
        s.submit([1], request_id="x")
    s.submit([1], request_id="y")
    with pytest.raises(OverloadedError, match="request limit 2"):
        s.submit([1])


def test_cancel_and_forget() -> None:
    runner, s = make()
    a = s.submit([1, 2, 3], request_id="a")
    b = s.submit([1, 2, 3], request_id="b")
    s.step()
    assert s.cancel(a) and not s.cancel(a)
    assert s.request(a).status is RequestStatus.CANCELLED
    assert not runner.cache.has_request("a") and runner.cache.has_request("b")
    with pytest.raises(ValueError):
        s.forget(b)
    s.run_until_idle()
    s.forget(a), s.forget(b)
    with pytest.raises(KeyError):
        s.request(a)
    assert runner.cache.leased_pages() == [0]
    # cancelling a queued request that was never admitted
    c = s.submit([1], request_id="c")
    assert s.cancel(c)
    assert s.idle


def test_failed_step_fails_its_requests_and_frees_them() -> None:
    runner, s = make(fail_on_step=2)
    a = s.submit([1, 2, 3], request_id="a")
    s.step()
    b = s.submit([5], request_id="b")
    events = s.step()          # injected failure: both a (decode) and b (prompt) were in the batch
    assert {e.request_id for e in events} == {"a", "b"}
    for rid in (a, b):
        view = s.request(rid)
        assert view.status is RequestStatus.FAILED and "injected" in view.error
    assert runner.cache.leased_pages() == [0] and s.snapshot().reserved_blocks == (0,)
    c = s.submit([9], request_id="c")
    s.run_until_idle()
    assert s.request(c).status is RequestStatus.FINISHED


def test_seeds_and_counters_reach_the_sampler() -> None:
    runner, s = make()
    sampler = s.sampler
    s.submit([1], request_id="a", sampling_params=SamplingParams(max_new_tokens=3, seed=11, temperature=0.5))
    s.step()
    assert sampler.last == ([11], [0])
    s.step()
    assert sampler.last == ([11], [1])


def test_windowed_group_reserves_less() -> None:
    config = SchedulerConfig(block_size=4, block_capacity=8, token_budget=8, chunk_size=8)
    runner, s = make(config, num_pages=8, window=6)
    # full attention would need ceil(60/4) = 15 > 8 pages; a window of 6 needs ceil((5 + 8)/4) + 1 = 5
    rid = s.submit(list(range(1, 31)), sampling_params=SamplingParams(max_new_tokens=30))
    s.run_until_idle()
    assert s.request(rid).status is RequestStatus.FINISHED
    assert runner.cache.leased_pages() == [0]


def test_decode_split_choice() -> None:
    """The number of blocks per (request, kv head) in split decode attention: the measured
    rule for requests of even length, more splits when one request is much longer."""
    from forge_engine_b200.parts.attention import choose_splits

    assert choose_splits([33] * 8, 8) == 4          # 8 requests of 2,048 keys: 256 blocks fill the slots once
    assert choose_splits([33] * 64, 8) == 1         # the machine is full anyway
    assert choose_splits([128] * 64, 8) == 2        # ... but long contexts take two
    assert choose_splits([33], 8) == 8              # one request: a cluster of 8
    assert choose_splits([513], 8) == 32            # one long request: clusters of 8 through memory
    assert choose_splits([3] * 8, 8) == 1           # too short to split
    for counts in ([33] * 12, [33] * 3, [100] * 5, [513] + [33] * 7, [257] + [17] * 31, [129] + [33] * 63):
        splits = choose_splits(counts, 8)
        assert splits in (1, 2, 4, 8) or (splits % 8 == 0 and splits <= 64)
        assert max(counts) // splits >= 2 or splits == 1
    # one long request beside short ones gets more splits than the short ones alone would
    assert choose_splits([513] + [33] * 7, 8) > choose_splits([33] * 8, 8)
    assert choose_splits([257] + [17] * 31, 8) > choose_splits([17] * 32, 8)
    # the order of the requests does not matter
    assert choose_splits([33] * 7 + [513], 8) == choose_splits([513] + [33] * 7, 8)
    # where the kernel that spreads the tiles evenly over the blocks may run (answer 0): uneven
    # lengths and block counts that would need two uneven rounds go to it, what fills the
    # slots once and single requests (many pieces to combine) stay with the splits
    assert choose_splits([513] + [33] * 7, 8, balanced=True) == 0
    assert choose_splits([257] + [17] * 31, 8, balanced=True) == 0
    assert choose_splits([47] * 40, 8, balanced=True) == 0
    assert choose_splits([32] * 64, 8, balanced=True) == 0
    assert choose_splits([32] * 8, 8, balanced=True) == 4
    assert choose_splits([32] * 32, 8, balanced=True) == 1
    assert choose_splits([128], 8, balanced=True) == 32
    assert choose_splits([32], 8, balanced=True) == 8
    assert choose_splits([5] * 300, 8, balanced=True) == 1      # more entries than the kernel keeps on chip


class StrictRunner(FakeRunner):
    """Like the real step function it refuses a whole step for one bad token id or one
    request beyond the position limit; it can also take a decode step's tokens from a
    tensor, as a runner that replays captured steps does."""

    supports_device_tokens = True

    def __init__(self, max_positions=12, **kwargs):
        from types import SimpleNamespace

        super().__init__(**kwargs)
        self.model = SimpleNamespace(spec=SimpleNamespace(vocab_size=VOCAB, max_positions=max_positions))

    def step(self, entries, device_tokens=None):
        if device_tokens is not None:
            source, rows = device_tokens
            entries = [type(e)(e.key, [int(source[r])], e.want) for e, r in zip(entries, rows)]
        for e in entries:
            if any(not 0 <= int(t) < VOCAB for t in e.tokens):
                raise ValueError("token id outside the vocabulary")
            if self.cache.request(e.key).length + len(e.tokens) > self.model.spec.max_positions:
                raise RuntimeError("would exceed max_position_embeddings")
        return super().step(entries)


class AsyncArgmaxSampler(ArgmaxSampler):
    class _Done:
        def synchronize(self):
            pass

    def sample_async(self, logits, params, seeds, counters):
        ids = logits.argmax(-1).to(torch.int32)
        return ids, ids.clone(), self._Done()


@pytest.mark.parametrize("lookahead", [False, True])
def test_one_bad_request_is_refused_alone(lookahead) -> None:
    """A prompt with an id outside the vocabulary, or one that would pass the position
    limit while decoding, is refused at submit; the requests beside it finish."""
    config = SchedulerConfig(block_size=4, block_capacity=16, lookahead=lookahead)
    runner = StrictRunner(max_positions=12)
    s = Scheduler(runner, AsyncArgmaxSampler(), config, SamplingParams(max_new_tokens=4), seed=0)
    assert s.lookahead is lookahead
    good = [s.submit([1, 2, 3], request_id="a"), s.submit([9], request_id="b")]
    with pytest.raises(ValueError, match="outside the vocabulary"):
        s.submit([1, VOCAB, 2], request_id="bad-id")
    with pytest.raises(ValueError, match="outside the vocabulary"):
        s.submit([-1], request_id="negative")
    with pytest.raises(ValueError, match="max_position_embeddings"):
        s.submit(list(range(10)), request_id="too-long")          # 10 + 4 - 1 = 13 > 12
    s.step()
    # joins while the others decode; 9 + 4 - 1 = 12 positions is exactly the limit
    good.append(s.submit(list(range(9)), request_id="c"))
    with pytest.raises(ValueError, match="max_position_embeddings"):
        s.submit(list(range(9)), request_id="d", sampling_params=SamplingParams(max_new_tokens=5))
    s.run_until_idle()
    for rid in good:
        view = s.request(rid)
        assert view.status is RequestStatus.FINISHED and len(view.output_tokens) == 4, view
    assert s.request("a").output_tokens == (4, 5, 6, 7)
    with pytest.raises(KeyError):
        s.request("bad-id")
    assert runner.cache.leased_pages() == [0] and s.snapshot().reserved_blocks == (0,)
