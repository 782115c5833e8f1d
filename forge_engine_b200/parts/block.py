"""Arrangement of norm, mixer and feed-forward in one block.

"pre_norm" is upstream's decoder layer (src/forge_engine/qwen3.py:241-261):
h += mixer(norm1(h)); h += ffn(norm2(h)).  The residual stream ``h`` is a 32-bit
tensor updated in place; the block returns its last update *unadded* so that the next
block's first norm (or the final norm) adds it in the same kernel that normalises.
"""

from __future__ import annotations

import os

import torch

from ..ops import native
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
        self._chain_parts = None

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        """role -> {local name -> WeightInfo}"""
        return {role: part_class(getattr(spec, role)).weight_shapes(getattr(spec, role)) for role in cls.roles}

    def cache_needs(self):
        return self.mixer.cache_needs()

    def plan_step(self, entries: list, page_size: int, plans: dict) -> None:
        planner = getattr(self.mixer, "plan_step", None)
        if planner is not None:
            planner(entries, page_size, plans)

    @property
    def graph_safe(self) -> bool:
        return all(getattr(part, "graph_safe", False)
                   for part in (self.input_norm, self.mixer, self.post_norm, self.ffn))

    def _chain(self):
        """What the one-kernel form of "output projection, norm, feed-forward" needs of this
        block's parts, or None: a mixer that can stop before its bias-free bfloat16 output
        projection, an RMS norm, and a gated feed-forward whose gate/up rows alternate in
        sixteens, all at sizes the kernel takes.  Worked out once."""
        if self._chain_parts is None:
            self._chain_parts = False
            o_proj = getattr(self.mixer, "o_proj", None)
            gate_up, down = getattr(self.ffn, "gate_up", None), getattr(self.ffn, "down", None)
            norm = self.post_norm
            usable = (self.ctx.dtype == torch.bfloat16 and hasattr(self.mixer, "attend")
                      and all(lin is not None and lin.bias is None and lin.weight.dtype == torch.bfloat16
                              for lin in (o_proj, gate_up, down))
                      and getattr(self.ffn, "block", 0) == 16
                      and hasattr(norm, "eps") and getattr(norm, "weight", None) is not None
                      and os.environ.get("FORGE_ENGINE_DECODE_CHAIN", "0") == "1")
            if usable:
                shapes = [(o_proj.out_features, o_proj.in_features, native.CHAIN_SRC_ACTIVATIONS, native.CHAIN_ADD),
                          (gate_up.out_features, gate_up.in_features, native.CHAIN_SRC_NORM, native.CHAIN_SILU_MUL),
                          (down.out_features, down.in_features, native.CHAIN_SRC_ACTIVATIONS, native.CHAIN_ADD)]
                if native.decode_chain_takes(shapes, 1):
                    self._chain_parts = (o_proj, norm, gate_up, down)
        return self._chain_parts or None

    def forward(self, h, pending, batch, cache: CacheView):
        """``h`` 32-bit [N, hidden] (in place); ``pending`` the previous block's update or
        None.  Returns this block's feed-forward update, still to be added (None when it
        has already been added)."""
        chain = self._chain() if batch.n_tokens <= native.CHAIN_MAX_TOKENS and self.ctx.timer is None else None
        if chain is not None:
            # few tokens: output projection (+= h), norm + gate/up with SiLU*mul and the down
            # projection (+= h) run as one persistent kernel whose weight stream never stops
            o_proj, norm, gate_up, down = chain
            normed = self.input_norm.add_forward(h, pending)
            heads = self.mixer.attend(normed, batch, cache)
            act = torch.empty((h.shape[0], gate_up.out_features // 2), dtype=torch.bfloat16, device=h.device)
            native.decode_chain(
                [dict(w=o_proj.weight, x=heads, out=h, src=native.CHAIN_SRC_ACTIVATIONS, epi=native.CHAIN_ADD),
                 dict(w=gate_up.weight, x=h, norm_w=norm.weight, eps=norm.eps, out=act,
                      src=native.CHAIN_SRC_NORM, epi=native.CHAIN_SILU_MUL),
                 dict(w=down.weight, x=act, out=h, src=native.CHAIN_SRC_ACTIVATIONS, epi=native.CHAIN_ADD)],
                h.shape[0], self.ctx.status)
            return None
        if self.ctx.timer is None:
            # a part that can add its update into the residual stream itself (in the epilogue of
            # its last projection) does so; the norm after it then only reads the stream
            normed = self.input_norm.add_forward(h, pending)
            adds = getattr(self.mixer, "forward_add", None)
            update = None if adds is not None and adds(normed, batch, cache, h) else self.mixer.forward(normed, batch, cache)
            normed = self.post_norm.add_forward(h, update)
            adds = getattr(self.ffn, "forward_add", None)
            return None if adds is not None and adds(normed, h) else self.ffn.forward(normed)
        with self.ctx.section("input_norm"):
            normed = self.input_norm.add_forward(h, pending)
        with self.ctx.section("mixer"):
            update = self.mixer.forward(normed, batch, cache)
        with self.ctx.section("post_norm"):
            normed = self.post_norm.add_forward(h, update)
        with self.ctx.section("ffn"):
            return self.ffn.forward(normed)


register_arrangement("pre_norm", PreNormBlock, replace=True)
