"""Gated feed-forward: down(silu(gate(x)) * up(x)) (src/forge_engine/qwen3.py:210-227).
gate and up are one fused projection; the activation product is one kernel."""

from __future__ import annotations

import torch

from ..errors import ConfigError
from ..ops import native
from .base import BuildContext, FeedForward, WeightInfo, register_part
from .linear import Linear, fused_rows, interleaved_rows

GATE_UP_BLOCK = 16


class GatedMLP(FeedForward):
    graph_safe = True

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        if spec.activation != "silu":
            raise ConfigError(f"activation {spec.activation!r} is not implemented (silu only)")
        self.inter = spec.intermediate_size
        # Rows of the fused weight alternate 16 gate and 16 up features where the size allows:
        # the tensor-core kernel then finishes silu(gate) * up in its epilogue.
        self.block = GATE_UP_BLOCK if self.inter % GATE_UP_BLOCK == 0 else 0
        # the sources are looked up one at a time and copied into the fused tensor
        if self.block:
            fused = interleaved_rows(weights, "gate_proj.weight", "up_proj.weight", self.inter, self.block)
        else:
            fused = fused_rows(weights, ["gate_proj.weight", "up_proj.weight"], [self.inter, self.inter])
        self.gate_up = Linear(fused, status=ctx.status)
        self.down = Linear(weights["down_proj.weight"], status=ctx.status)

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        h, i = spec.hidden_size, spec.intermediate_size
        return {
            "gate_proj.weight": WeightInfo((i, h)),
            "up_proj.weight": WeightInfo((i, h)),
            "down_proj.weight": WeightInfo((h, i)),
        }

    def forward_add(self, x, residual) -> bool:
        """``forward`` with the update added into the 32-bit ``residual`` by the down projection
        itself.  False (and nothing done) where that projection cannot."""
        if not (self.block == 16 and self.down.adds_into(x, residual) and self.gate_up._tc5_ok(x)
                and self.gate_up.out_features % 32 == 0 and self.gate_up.bias is None):
            return False
        return self.down.add_into(self.gate_up.silu_mul(x, self.block), residual)

    def forward(self, x):
        act = self.gate_up.silu_mul(x, self.block) if self.block else None
        if act is None:
            gate_up = self.gate_up(x)
            act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
            native.silu_mul(gate_up, act, self.block)
        return self.down(act)


register_part("gated_mlp", GatedMLP, replace=True)
