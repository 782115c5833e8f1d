"""Gated feed-forward: down(silu(gate(x)) * up(x)) (src/forge_engine/qwen3.py:210-227).
gate and up are one fused projection; the activation product is one kernel."""

from __future__ import annotations

import torch

from ..errors import ConfigError
from ..ops import native
from .base import BuildContext, FeedForward, WeightInfo, register_part
from .linear import Linear, fuse_rows


class GatedMLP(FeedForward):
    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        if spec.activation != "silu":
            raise ConfigError(f"activation {spec.activation!r} is not implemented (silu only)")
        self.inter = spec.intermediate_size
        self.gate_up = Linear(fuse_rows([weights["gate_proj.weight"], weights["up_proj.weight"]]))
        self.down = Linear(weights["down_proj.weight"])

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        h, i = spec.hidden_size, spec.intermediate_size
        return {
            "gate_proj.weight": WeightInfo((i, h)),
            "up_proj.weight": WeightInfo((i, h)),
            "down_proj.weight": WeightInfo((h, i)),
        }

    def forward(self, x):
        gate_up = self.gate_up(x)
        act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
        native.silu_mul(gate_up, act)
        return self.down(act)


register_part("gated_mlp", GatedMLP, replace=True)
