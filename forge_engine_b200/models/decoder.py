"""A decoder-only language model assembled from a ModelSpec.

Data flow of one step (src/forge_engine/qwen3.py:297-342, restated for a flat batch):
embedding gather into the 32-bit residual stream, the runs of the schedule in order
(each a block with its cache view), final norm on the wanted rows only, and the output
projection to 32-bit logits.  Which blocks exist, which run uses which block and which
cache, is all data of the spec; this class has no sizes of its own.
"""

from __future__ import annotations

from collections.abc import Mapping

import torch

from ..config.specs import ModelSpec
from ..ops import native
from ..parts.base import BuildContext, WeightInfo, arrangement_class, build_part, part_class
from ..parts.linear import Linear


def expected_tensors(spec: ModelSpec) -> dict:
    """Checkpoint tensor name -> WeightInfo, in a fixed order (embedding, final norm,
    layers in order, output head), as upstream lists them (src/forge_engine/weights.py:253-282)."""
    out: dict[str, WeightInfo] = {
        spec.embed_name: WeightInfo((spec.vocab_size, spec.hidden_size)),
    }
    for local, info in part_class(spec.final_norm).weight_shapes(spec.final_norm).items():
        out[f"{spec.final_norm_name}.{local}"] = info
    for layer in spec.layers:
        block = arrangement_class(layer.arrangement)
        for role, shapes in block.weight_shapes(layer).items():
            prefix = layer.names[role]
            for local, info in shapes.items():
                out[f"{prefix}.{local}"] = info
    if not spec.tie_embeddings:
        out[spec.head_name] = WeightInfo((spec.vocab_size, spec.hidden_size))
    return out


class _Scoped(Mapping):
    """The tensors of one part by their local names: ``view[local]`` looks
    ``weights[prefix.local]`` up at that moment (a checkpoint that reads on access puts the
    tensor on the device then), so a part holds only what it keeps."""

    def __init__(self, weights, prefix: str, names) -> None:
        self._weights, self._prefix, self._names = weights, prefix, tuple(names)

    def __getitem__(self, local: str):
        if local not in self._names:
            raise KeyError(local)
        return self._weights[f"{self._prefix}.{local}"]

    def __iter__(self):
        return iter(self._names)

    def __len__(self) -> int:
        return len(self._names)


class DecoderModel:
    def __init__(self, spec: ModelSpec, weights: dict, ctx: BuildContext) -> None:
        self.spec = spec
        self.ctx = ctx
        self.embed = weights[spec.embed_name].contiguous()
        self.blocks = []
        for layer in spec.layers:
            block_cls = arrangement_class(layer.arrangement)
            per_role = {}
            for role, shapes in block_cls.weight_shapes(layer).items():
                prefix = layer.names[role]
                per_role[role] = _Scoped(weights, prefix, shapes)
            self.blocks.append(block_cls(layer, per_role, ctx))
        norm_shapes = part_class(spec.final_norm).weight_shapes(spec.final_norm)
        self.final_norm = build_part(spec.final_norm, _Scoped(weights, spec.final_norm_name, norm_shapes), ctx)
        self.head = Linear(self.embed if spec.tie_embeddings else weights[spec.head_name], status=ctx.status)
        for index, run in enumerate(spec.schedule):
            if not 0 <= run.layer < len(self.blocks):
                raise ValueError(f"run {index} names layer {run.layer}, which does not exist")
            if run.cache_of is not None and not 0 <= run.cache_of < index:
                raise ValueError(f"run {index} may only read the cache of an earlier run")

    @property
    def graph_safe(self) -> bool:
        """Whether a decode step of this model can be captured in a CUDA graph and replayed."""
        return (all(getattr(block, "graph_safe", False) for block in self.blocks)
                and getattr(self.final_norm, "graph_safe", False))

    def plan_step(self, entries: list, page_size: int) -> dict:
        """What the blocks' parts decide on the host for a step of these entries
        (``(slot, tokens cached, new tokens)`` each): {part's key: its decision}.  A step is
        captured in a CUDA graph once per distinct answer."""
        plans: dict = {}
        for block in self.blocks:
            planner = getattr(block, "plan_step", None)
            if planner is not None:
                planner(entries, page_size, plans)
        return plans

    # -- cache ---------------------------------------------------------------------
    def cache_needs(self) -> tuple:
        """(needs per run, {run: run whose cache it reads})."""
        needs = [self.blocks[run.layer].cache_needs() for run in self.spec.schedule]
        shares = {i: run.cache_of for i, run in enumerate(self.spec.schedule) if run.cache_of is not None}
        return needs, shares

    def weight_bytes(self) -> int:
        """Bytes of every distinct weight tensor a step reads once (tied tensors count once)."""
        seen: dict[int, int] = {}
        visited: set[int] = set()

        def visit(obj) -> None:
            if isinstance(obj, torch.Tensor):
                if obj.is_floating_point():
                    seen[obj.data_ptr()] = obj.numel() * obj.element_size()
                return
            if id(obj) in visited or isinstance(obj, (BuildContext, ModelSpec, str, int, float, type(None))):
                return
            visited.add(id(obj))
            if isinstance(obj, (list, tuple)):
                for item in obj:
                    visit(item)
            elif isinstance(obj, dict):
                for item in obj.values():
                    visit(item)
            elif hasattr(obj, "__dict__"):
                for item in vars(obj).values():
                    visit(item)

        visit(self.blocks)
        visit(self.final_norm)
        visit(self.head)
        return sum(seen.values())

    # -- one step ------------------------------------------------------------------
    def forward(self, batch, cache) -> torch.Tensor:
        """Run ``batch`` through all runs; returns logits [wanted rows, vocab] in 32-bit."""
        n = batch.n_tokens
        batch.shared.clear()      # what parts share lives for one pass only (a batch may be run again)
        h = torch.empty((n, self.spec.hidden_size), dtype=torch.float32, device=self.ctx.device)
        with self.ctx.section("embedding"):
            native.embedding(batch.token_ids, self.embed, h, self.ctx.status)
        pending = None
        for index, run in enumerate(self.spec.schedule):
            pending = self.blocks[run.layer].forward(h, pending, batch, cache.view(index))
        if batch.n_want == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.ctx.device)
        with self.ctx.section("final_norm"):
            normed = self.final_norm.add_forward(h, pending, row_map=batch.want_rows)
        with self.ctx.section("head"):
            return self.head(normed, out_dtype=torch.float32)
