"""RMS normalisation (src/forge_engine/qwen3.py:91-105), fused with the residual sum
(src/forge_engine/_triton_kernels.py:32-58).  Sum, variance, scaling and the weight
product are all taken in 32-bit; the result is rounded once, on store."""

from __future__ import annotations

import torch

from ..ops import native
from .base import BuildContext, Norm, WeightInfo, register_part


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        self.size = spec.size
        self.eps = float(spec.eps)
        self.weight = weights["weight"].to(device=ctx.device, dtype=torch.float32).contiguous()
        self.dtype = ctx.dtype

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        return {"weight": WeightInfo((spec.size,), "norm")}

    def add_forward(self, residual, update, row_map=None):
        """residual (32-bit [N, size]) += update; returns the normalised rows in the
        activation dtype.  With ``row_map`` only those rows are produced and the
        residual is left untouched."""
        rows = residual.shape[0] if row_map is None else row_map.numel()
        out = torch.empty((rows, self.size), dtype=self.dtype, device=residual.device)
        native.add_rmsnorm(residual, update, self.weight, out, self.eps, row_map,
                           write_residual=row_map is None)
        return out

    def forward(self, x):
        """Norm of a 32-bit tensor without a residual update."""
        return self.add_forward(x, None)


register_part("rmsnorm", RMSNorm, replace=True)
