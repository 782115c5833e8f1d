"""Arrangement of norm, mixer and feed-forward in one block.

"pre_norm" is upstream's decoder layer (src/forge_engine/qwen3.py:241-261):
h += mixer(norm1(h)); h += ffn(norm2(h)).  The residual stream ``h`` is a 32-bit
tensor updated in place; the block returns its last update *unadded* so that the next
block's first norm (or the final norm) adds it in the same kernel that normalises.
"""

from __future__ import annotations

from .base import BuildContext, CacheView, build_part, part_class, register_arrangement


class PreNormBlock:
    roles = ("input_norm", "mixer", "post_norm", "ffn")

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        """``weights[role]`` is the dict of that part's local tensors."""
        self.ctx = ctx
        self.input_norm = build_part(spec.input_norm, weights["input_norm"], ctx)
        self.mixer = build_part(spec.mixer, weights["mixer"], ctx)
        self.post_norm = build_part(spec.post_norm, weights["post_norm"], ctx)
        self.ffn = build_part(spec.ffn, weights["ffn"], ctx)

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        """role -> {local name -> WeightInfo}"""
        return {role: part_class(getattr(spec, role)).weight_shapes(getattr(spec, role)) for role in cls.roles}

    def cache_needs(self):
        return self.mixer.cache_needs()

    @property
    def graph_safe(self) -> bool:
        return all(getattr(part, "graph_safe", False)
                   for part in (self.input_norm, self.mixer, self.post_norm, self.ffn))

    def forward(self, h, pending, batch, cache: CacheView):
        """``h`` 32-bit [N, hidden] (in place); ``pending`` the previous block's update or
        None.  Returns this block's feed-forward update, still to be added."""
        if self.ctx.timer is None:
            normed = self.input_norm.add_forward(h, pending)
            update = self.mixer.forward(normed, batch, cache)
            normed = self.post_norm.add_forward(h, update)
            return self.ffn.forward(normed)
        with self.ctx.section("input_norm"):
            normed = self.input_norm.add_forward(h, pending)
        with self.ctx.section("mixer"):
            update = self.mixer.forward(normed, batch, cache)
        with self.ctx.section("post_norm"):
            normed = self.post_norm.add_forward(h, update)
        with self.ctx.section("ffn"):
            return self.ffn.forward(normed)


register_arrangement("pre_norm", PreNormBlock, replace=True)
