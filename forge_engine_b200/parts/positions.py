"""Position encodings for attention.

``RotaryEncoding`` restates src/forge_engine/qwen3.py:345-363: inv_freq_j =
1 / theta^(2j / rotary_dim) in 32-bit, angle = float(position) * inv_freq_j; the
rotation itself happens inside the fused q/k kernel, which takes the table."""

from __future__ import annotations

import torch

from .base import BuildContext, PositionEncoding, register_part


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        if spec.rotary_dim % 2 or spec.rotary_dim > spec.head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        self.rotary_dim = spec.rotary_dim
        exponent = torch.arange(0, spec.rotary_dim, 2, dtype=torch.float32) / spec.rotary_dim
        self.inv_freq = (1.0 / (spec.theta**exponent)).to(ctx.device).contiguous()

    def rotary(self):
        return self.inv_freq, self.rotary_dim


class NoPosition(PositionEncoding):
    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        pass


register_part("rope", RotaryEncoding, replace=True)
register_part("none", NoPosition, replace=True)
