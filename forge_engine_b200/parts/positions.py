"""Position encodings for attention.

``RotaryEncoding`` restates src/forge_engine/qwen3.py:345-363: inv_freq_j =
1 / theta^(2j / rotary_dim) in 32-bit, angle = float(position) * inv_freq_j; the
rotation itself happens inside the fused q/k kernel.  Cosine and sine of a step's angles
are the same in every layer: ``table`` takes them once per step (in 32-bit, not rounded)."""

from __future__ import annotations

import torch

from ..ops import native
from .base import BuildContext, PositionEncoding, register_part


class RotaryEncoding(PositionEncoding):
    graph_safe = True

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        if spec.rotary_dim % 2 or spec.rotary_dim > spec.head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        self.rotary_dim = spec.rotary_dim
        self.theta = float(spec.theta)
        exponent = torch.arange(0, spec.rotary_dim, 2, dtype=torch.float32) / spec.rotary_dim
        self.inv_freq = (1.0 / (spec.theta**exponent)).to(ctx.device).contiguous()

    def rotary(self):
        return self.inv_freq, self.rotary_dim

    def table(self, batch) -> torch.Tensor:
        """[tokens, rotary_dim / 2, 2] (cos, sin) of this step's angles; worked out by the
        first layer that asks and shared through the batch."""
        key = ("rotary", self.theta, self.rotary_dim)
        table = batch.shared.get(key)
        if table is None:
            table = torch.empty((batch.n_tokens, self.rotary_dim // 2, 2), dtype=torch.float32, device=self.inv_freq.device)
            native.rope_table(batch.positions, self.inv_freq, table)
            batch.shared[key] = table
        return table


class NoPosition(PositionEncoding):
    graph_safe = True

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        pass


register_part("rope", RotaryEncoding, replace=True)
register_part("none", NoPosition, replace=True)
