"""Causal grouped-query attention over the paged cache.

Formulas: src/forge_engine/qwen3.py:108-207.  One fused projection gives q, k, v; one
kernel normalises q and k per head, rotates them and stores k, v into their pages; the
attention kernel then reads everything it needs from the pages, so a step's new tokens
and the earlier ones are treated alike.  The mixer keeps PagedKVSpec(kv heads,
head_dim, window) between steps.
"""

from __future__ import annotations

import functools
import os

import torch

from ..cache.manager import CacheNeeds, PagedKVSpec
from ..errors import UnsupportedShapeError
from ..ops import native
from .base import BuildContext, CacheView, Mixer, WeightInfo, build_part, register_part
from .linear import Linear, fused_rows


# Blocks of a decode kernel the GPU holds at once when nothing says otherwise (two per SM on
# the 148 SMs of a B200); a mixer asks the kernel library for the figure of its device.
DEFAULT_DECODE_SLOTS = 296
MAX_SPLITS = 64   # what the merge takes
# With more tokens a block of the projection finishes so many that the separate kernel is
# faster (measured: 2.35 -> 2.27 ms per step at 1 token, no change at 8, 6.2 -> 6.7 ms at 64).
FUSED_PROJECTION_ROWS = 16
CLUSTER_SPLITS = 8            # this many blocks combine their results inside a cluster
CLUSTER_WORTH_TILES = 96      # from here on (6,144 keys) more than one cluster per pair pays

# Costs in units of one 64-key tile of one block (about 1.4 us), from measurements of the
# split decode kernel on a B200: combining the splits inside a cluster, through global
# memory, and what every round of blocks over the machine's slots costs beside its tiles.
MERGE_IN_CLUSTER, MERGE_THROUGH_MEMORY, ROUND_OVERHEAD = 2, 9, 3
SPLIT_TILE_US = 1.45
BALANCED_BASE_US, BALANCED_TILE_US, BALANCED_PAIR_US, BALANCED_PIECE_US = 15.0, 0.0049, 0.003, 0.27
BALANCED_MAX_ENTRIES = 256    # what the balanced kernel keeps in shared memory


def choose_splits(tile_counts, kv_heads: int, balanced: bool = False, slots: int = DEFAULT_DECODE_SLOTS) -> int:
    """How many blocks share one (request, kv head)'s keys; ``tile_counts`` are the 64-key
    tiles of the step's requests.  Every request gets the same number of splits.  With
    ``balanced`` the answer may be 0: the kernel that spreads all tiles evenly over the
    machine's blocks is expected to be faster than any split.  ``slots``: blocks of the
    decode kernels the GPU holds at once."""
    return _choose_splits(tuple(sorted(max(1, int(t)) for t in tile_counts)), int(kv_heads), bool(balanced),
                          max(1, int(slots)))


def _even_splits(pairs: int, tiles: int, DECODE_SLOTS: int) -> int:
    """Requests of about the same length (measured on a B200, 8 kv heads, head size 128).
    Few pairs: fill the machine's slots once, every block getting at least four tiles; up to 8
    blocks combine inside a cluster, and going beyond (clusters of 8 whose results pass through
    memory) pays from about 6,000 keys on (one request: 8,192 keys 22.9 us with 8 splits,
    17.3 us with 32; 2,048 keys 7.7 against 10.8 us with 16).  With more pairs than half the
    slots the machine is full anyway: one split up to 4,096 keys (512 pairs of 2,048 keys:
    100 us against 116 us with two), two beyond.  Clusters of 3, 5, 6 or 7 blocks measured
    badly (12 requests: 38.8 us with 3 splits, 28.3 us with 2), so counts are powers of two."""
    most = max(1, min(MAX_SPLITS, tiles // 4))
    if pairs * 2 > DECODE_SLOTS:
        return 1 if tiles <= 64 else min(most, 2)
    splits = max(1, min(most, DECODE_SLOTS // pairs))
    if splits > CLUSTER_SPLITS:
        return CLUSTER_SPLITS if tiles < CLUSTER_WORTH_TILES else splits - splits % CLUSTER_SPLITS
    return 1 << (splits.bit_length() - 1)


def _split_cost(tile_counts: tuple, kv_heads: int, splits: int, DECODE_SLOTS: int) -> int:
    """Estimate for ``splits`` blocks per pair, in tiles of one block: the longest request
    decides how long its blocks run, while all blocks together pass through the machine's
    slots, in rounds if they are more: max(longest / s, all tiles / slots, rounds x the median
    block) + the cost of combining + an overhead per round."""
    pairs = len(tile_counts) * kv_heads
    longest, median = tile_counts[-1], tile_counts[len(tile_counts) // 2]
    total = sum(tile_counts) * kv_heads
    rounds = -(-pairs * splits // DECODE_SLOTS)
    merge = 0 if splits == 1 else (MERGE_IN_CLUSTER if splits <= CLUSTER_SPLITS else MERGE_THROUGH_MEMORY)
    tiles = max(-(-longest // splits), -(-total // DECODE_SLOTS), rounds * -(-median // splits))
    return tiles + merge + ROUND_OVERHEAD * rounds


@functools.lru_cache(maxsize=4096)
def _choose_splits(tile_counts: tuple, kv_heads: int, balanced: bool, DECODE_SLOTS: int) -> int:
    pairs = len(tile_counts) * kv_heads
    longest = tile_counts[-1]
    median = tile_counts[len(tile_counts) // 2]
    if longest < 2 * median:
        best = _even_splits(pairs, longest, DECODE_SLOTS)
    else:
        # One request much longer than most.  Measured: one request of 32,768 keys beside seven
        # of 2,048: 176 us with the 4 splits of even requests, 94-102 us with 16-32; one of
        # 16,384 beside 31 of 1,024: 329 us with 1, 108 us with 8; one of 8,192 beside 63 of
        # 2,048: 219 us with 1, 171 us with 2, 147 us with 4.
        best, best_cost = 1, None
        for splits in (1, 2, 4, 8, 16, 24, 32, 40, 48, 56, 64):
            if splits > 1 and (longest // splits < 2 or splits > MAX_SPLITS):
                break
            cost = _split_cost(tile_counts, kv_heads, splits, DECODE_SLOTS)
            if best_cost is None or cost < best_cost:
                best, best_cost = splits, cost
    if balanced and len(tile_counts) <= BALANCED_MAX_ENTRIES:
        # The balanced kernel (and the kernel that combines the pairs it cut) measured
        # 15 us + 4.9 ns per tile + 3 ns per pair, whatever the lengths are (8 requests of 2,048
        # keys 26 us, 64 of them 97 us, 200 of 300 keys 61 us); a tile of the split kernel's
        # estimate is 1.45 us (32 requests of 2,048 keys: 35 tiles, 50 us measured).  The
        # balanced kernel wins where blocks would run in two uneven rounds (40 requests of
        # 3,000 keys: 134 -> 90 us) and wherever lengths differ much (one request of 32,768
        # keys beside seven of 2,048: 96 -> 49 us; 64 requests of 16 to 4,096 keys: 140 -> 95 us).
        # Combining costs by the pieces of the longest pair (one request of 8,192 keys is cut
        # into 37 pieces per kv head: 31 us, against 17 us with 32 splits).
        total = sum(tile_counts) * kv_heads
        pieces = min(DECODE_SLOTS, longest * DECODE_SLOTS // total + 1)
        balanced_us = (BALANCED_BASE_US + BALANCED_TILE_US * total + BALANCED_PAIR_US * pairs
                       + BALANCED_PIECE_US * pieces)
        if balanced_us < SPLIT_TILE_US * _split_cost(tile_counts, kv_heads, best, DECODE_SLOTS):
            return 0
    return best


class GQAttention(Mixer):
    @property
    def graph_safe(self) -> bool:
        """The kernels here are; a position encoding that rewrites q and k itself decides."""
        return bool(getattr(self.position, "graph_safe", False))

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        if spec.head_dim % 16 or spec.head_dim > 256:
            raise UnsupportedShapeError(
                f"head_dim={spec.head_dim}: the attention kernels take multiples of 16 up to 256"
            )
        if spec.num_heads % spec.num_kv_heads:
            raise UnsupportedShapeError("num_heads must be a multiple of num_kv_heads")
        self.spec = spec
        self.ctx = ctx
        self.nq, self.nkv, self.d = spec.num_heads, spec.num_kv_heads, spec.head_dim
        bias = None
        rows = [self.nq * self.d, self.nkv * self.d, self.nkv * self.d]
        if spec.bias:
            bias = fused_rows(weights, ["q_proj.bias", "k_proj.bias", "v_proj.bias"], rows)
        # q, k and v are looked up one at a time and copied into the fused tensor
        self.qkv_proj = Linear(
            fused_rows(weights, ["q_proj.weight", "k_proj.weight", "v_proj.weight"], rows),
            bias,
            status=ctx.status,
        )
        self.o_proj = Linear(weights["o_proj.weight"], weights["o_proj.bias"] if spec.bias else None,
                             status=ctx.status)
        self.q_norm = self.k_norm = None
        if spec.qk_norm:
            self.q_norm = weights["q_norm.weight"].float().contiguous()
            self.k_norm = weights["k_norm.weight"].float().contiguous()
        self.position = build_part(spec.position, {}, ctx)
        self._slots = None
        self.plan_key = ("gqa_attention", self.nq, self.nkv, self.d, spec.window)
        self.last_splits = None   # what the last step's decode entries ran with (0: balanced kernel)

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        q, kv, h = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim, spec.hidden_size
        shapes = {
            "q_proj.weight": WeightInfo((q, h)),
            "k_proj.weight": WeightInfo((kv, h)),
            "v_proj.weight": WeightInfo((kv, h)),
            "o_proj.weight": WeightInfo((h, q)),
        }
        if spec.qk_norm:
            shapes["q_norm.weight"] = WeightInfo((spec.head_dim,), "norm")
            shapes["k_norm.weight"] = WeightInfo((spec.head_dim,), "norm")
        if spec.bias:
            shapes["q_proj.bias"] = WeightInfo((q,), "bias")
            shapes["k_proj.bias"] = WeightInfo((kv,), "bias")
            shapes["v_proj.bias"] = WeightInfo((kv,), "bias")
            shapes["o_proj.bias"] = WeightInfo((h,), "bias")
        return shapes

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(kv=PagedKVSpec(self.nkv, self.d, self.spec.window))

    def decode_slots(self) -> int:
        """Blocks of the decode kernels this device holds at once: what the balanced kernel
        of this head size is launched with (the library asks the occupancy of its own
        kernel), else two per SM."""
        if self._slots is None:
            blocks = native.attention_balanced_blocks(self.d) if self.d % 64 == 0 else 0
            if blocks <= 0:
                blocks = 2 * torch.cuda.get_device_properties(self.ctx.device).multi_processor_count
            self._slots = blocks
        return self._slots

    def forward(self, x, batch, cache: CacheView):
        out = self.attend(x, batch, cache)
        with self.ctx.section("mixer.o_proj"):
            return self.o_proj(out)

    def forward_add(self, x, batch, cache: CacheView, residual) -> bool:
        """``forward`` with the update added into the 32-bit ``residual`` by the output
        projection itself.  False (and nothing done) where that projection cannot."""
        if not self.o_proj.adds_into(x, residual) or self.ctx.timer is not None:
            return False
        return self.o_proj.add_into(self.attend(x, batch, cache), residual)

    def attend(self, x, batch, cache: CacheView):
        """Everything but the output projection: the heads' outputs [N, heads * head_dim]
        (a block that fuses ``o_proj`` with what follows takes them from here)."""
        with self.ctx.section("mixer.qkv_rope_cache"):
            qkv = self._project(x, batch, cache)
        k_cache, v_cache = cache.kv
        table = batch.group_tables[cache.group]
        out = torch.empty((x.shape[0], self.nq * self.d), dtype=qkv.dtype, device=x.device)
        groups = self.nq // self.nkv
        with self.ctx.section("mixer.attention"):
            if qkv.dtype == torch.bfloat16 and groups <= native.ATTN_DECODE_ROWS:
                self._tensor_core_attention(qkv, k_cache, v_cache, table, batch, out, groups)
            else:
                native.attention_simt(
                    qkv, qkv.shape[1], k_cache, v_cache, table, batch.positions, batch.token_entry,
                    self.spec.window, self.spec.scale, out, self.nq, self.ctx.status,
                )
        return out

    def _project(self, x, batch, cache: CacheView):
        """q, k, v of the step's tokens: projected, normalised per head, rotated; k and v
        stored in their pages.  Returns qkv with the finished queries."""
        k_cache, v_cache = cache.kv
        table = batch.group_tables[cache.group]
        rotary = self.position.rotary()
        if self._summed_projection(x, rotary, k_cache):
            # few tokens: the projection's k-splits add into a zeroed 32-bit buffer (no cluster,
            # more blocks), and the norm-and-rotate kernel reads the sums and leaves zeros behind
            width = self.qkv_proj.out_features
            # everything the second kernel needs is at hand before the first is launched: the
            # buffer is only zero again when both have run
            angles = self.position.table(batch) if hasattr(self.position, "table") else None
            qkv = torch.empty((x.shape[0], width), dtype=x.dtype, device=x.device)
            sums = native.projection_sums(x.device, x.shape[0] * width)[: x.shape[0] * width].view(x.shape[0], width)
            native.gemm_tc5(x, self.qkv_proj.weight, sums, native.TC5_ADD_F32, self.ctx.status, bias=self.qkv_proj.bias,
                            ksplit=native.tc5_ksplit_sums(width, self.qkv_proj.in_features, x.shape[0]))
            native.qk_rope_cache_sums(
                sums, qkv, self.q_norm, self.k_norm, self.spec.qk_norm_eps, rotary[0],
                batch.positions, batch.token_entry, k_cache, v_cache, table, self.nq, cache.owns, self.ctx.status,
                table=angles,
            )
        elif self._fused_projection(x, rotary, k_cache):
            # few tokens, heads of 128: norm, rotation and the page write happen in the
            # projection's own epilogue
            qkv = torch.empty((x.shape[0], self.qkv_proj.out_features), dtype=x.dtype, device=x.device)
            native.gemm_tc5_qkv_rope(
                x, self.qkv_proj.weight, self.qkv_proj.bias, qkv, self.q_norm, self.k_norm,
                self.spec.qk_norm_eps, self.position.table(batch), batch.positions, batch.token_entry, k_cache, v_cache, table,
                self.nq, cache.owns, self.ctx.status,
                ksplit=native.tc5_ksplit(self.qkv_proj.out_features, self.qkv_proj.in_features),
            )
        else:
            qkv = self.qkv_proj(x)
            angles = None
            if rotary is None:
                self.position.apply(qkv, self.nq, self.nkv, self.d, batch)
                inv_freq, rotary_dim = None, 0
            else:
                inv_freq, rotary_dim = rotary
                if hasattr(self.position, "table"):
                    angles = self.position.table(batch)
            native.qk_rope_cache(
                qkv, self.q_norm, self.k_norm, self.spec.qk_norm_eps, inv_freq, rotary_dim,
                batch.positions, batch.token_entry, k_cache, v_cache, table, self.nq,
                cache.owns, self.ctx.status, table=angles,
            )
        return qkv

    def _summed_projection(self, x, rotary, k_cache) -> bool:
        """Whether the q/k/v projection adds its k-splits into a 32-bit buffer that a separate
        norm-and-rotate kernel reads: few tokens, the tcgen05 kernel takes the call, and the
        position encoding rotates whole heads.  Up to FORGE_ENGINE_SUMMED_QKV tokens (64; 0 turns
        it off).  Measured at the 4B shape against the projection that sums its k-splits inside
        a cluster and norms and rotates in its own epilogue: 2.473 against 2.509 ms a decode
        step at batch 8, 2.940 against 3.017 at 16, 3.866 against 3.921 at 32, 5.82 against 5.85
        at 64, no difference at batch 1 and 2."""
        limit = int(os.environ.get("FORGE_ENGINE_SUMMED_QKV", "64"))
        return (x.shape[0] <= limit and self.d in (64, 128, 256) and rotary is not None and rotary[1] == self.d
                and k_cache.dtype == torch.bfloat16 and self.qkv_proj._tc5_ok(x))

    def _fused_projection(self, x, rotary, k_cache) -> bool:
        """Whether the q/k/v projection's epilogue can do the per-head norms, the rotation
        and the page write: the tcgen05 kernel takes the call, a head is one 128-feature
        tile, and the whole head is rotated."""
        return (self.d == 128 and rotary is not None and rotary[1] == 128 and hasattr(self.position, "table")
                and k_cache.dtype == torch.bfloat16
                and x.shape[0] <= FUSED_PROJECTION_ROWS and self.qkv_proj._tc5_ok(x)
                and os.environ.get("FORGE_ENGINE_FUSED_QKV", "1") != "0")

    def plan_step(self, entries: list, page_size: int, plans: dict) -> None:
        """The host's decision for a step of ``entries`` ((slot, cached, new) each): entries
        with few rows (new tokens x heads per kv head <= 16) take the split decode kernel, the
        rest the prefill kernel; both may run in one step.  (run prefill, run decode, splits
        of the decode kernel - 0: the kernel that spreads all tiles evenly) under this
        mixer's key; layers with the same geometry share it."""
        if self.ctx.dtype != torch.bfloat16 or self.plan_key in plans:
            return
        groups = self.nq // self.nkv
        limit = native.ATTN_DECODE_ROWS
        small = [(start, count) for _, start, count in entries if count * groups <= limit]
        run_decode = bool(small)
        run_prefill = len(small) < len(entries)
        splits = 1
        if run_decode:
            contexts = [start + count for start, count in small]
            if self.spec.window:
                contexts = [min(c, self.spec.window + limit) for c in contexts]
            # FORGE_ENGINE_DECODE_BALANCED: 0 never uses the balanced kernel, "always" uses it
            # wherever it can run, anything else lets the estimate decide
            wish = os.environ.get("FORGE_ENGINE_DECODE_BALANCED", "1")
            balanced = (self.d % 64 == 0 and page_size <= 64 and 64 % page_size == 0
                        and len(entries) <= BALANCED_MAX_ENTRIES and wish != "0")
            splits = 0 if balanced and wish == "always" else choose_splits(
                [-(-c // 64) for c in contexts], self.nkv, balanced, self.decode_slots())
        plans[self.plan_key] = (run_prefill, run_decode, splits)

    def _tensor_core_attention(self, qkv, k_cache, v_cache, table, batch, out, groups) -> None:
        if self.plan_key not in batch.plans:
            self.plan_step(batch.entries, k_cache.shape[2], batch.plans)
        run_prefill, run_decode, splits = batch.plans[self.plan_key]
        if run_decode:
            self.last_splits = splits
        native.attention_mma(
            qkv, qkv.shape[1], k_cache, v_cache, table, batch.cu_tokens, batch.starts,
            batch.n_entries, batch.max_new, self.spec.window, self.spec.scale, out, self.nq,
            self.ctx.status, run_prefill, run_decode, splits,
        )


register_part("gqa_attention", GQAttention, replace=True)
