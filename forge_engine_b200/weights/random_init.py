"""Seeded random weights: in memory, or written out as a model folder.

Upstream has no such mode (its tests rely on torch's default initialisers,
tests/test_qwen3.py:48-49).  Here matrices and biases are N(0, std), norm weights are
1 + N(0, 0.1).  Every tensor is drawn from a generator of its own, seeded with the model's
seed and the tensor's place in ``expected_tensors``, so a tensor's values do not depend on
which others were drawn before it: ``RandomTensors`` draws a tensor when the model asks
for it (benchmark-sized models are assembled layer by layer and never exist twice).
"""

from __future__ import annotations

import json
from collections.abc import Mapping
from pathlib import Path

import torch
from safetensors.torch import save_file

from .loader import SINGLE_NAME


class RandomTensors(Mapping):
    """name -> freshly drawn tensor (not kept); iteration follows ``expected``.

    On the CPU the values are the same on every machine; on a CUDA device they are
    reproducible for that device type only (used for benchmark-sized models)."""

    PIECE = 1 << 20

    def __init__(self, expected: dict, seed: int, *, std: float = 0.02, dtype=torch.bfloat16, device="cpu") -> None:
        self._expected = expected
        self._index = {name: i for i, name in enumerate(expected)}
        self.seed, self.std, self.dtype, self.device = int(seed), float(std), dtype, device

    def __len__(self) -> int:
        return len(self._expected)

    def __iter__(self):
        return iter(self._expected)

    def __getitem__(self, name: str) -> torch.Tensor:
        info = self._expected[name]
        generator = torch.Generator(device=self.device).manual_seed(self.seed * 1_000_003 + self._index[name])
        out = torch.empty(info.shape, dtype=self.dtype, device=self.device)
        flat = out.view(-1)
        # drawn in 32-bit in pieces of at most 2^20 values, so that a large table (an embedding)
        # does not exist a second time in 32-bit while it is drawn
        for begin in range(0, max(1, flat.numel()), self.PIECE):
            count = min(self.PIECE, flat.numel() - begin)
            noise = torch.randn(count, generator=generator, dtype=torch.float32, device=self.device)
            flat[begin : begin + count] = noise.mul_(0.1).add_(1.0) if info.role == "norm" else noise.mul_(self.std)
            del noise
        return out

    def close(self) -> None:
        pass


def random_tensors(expected: dict, seed: int, *, std: float = 0.02, dtype=torch.bfloat16,
                   device="cpu") -> dict:
    """Every tensor of ``expected`` at once, as ``RandomTensors`` draws them."""
    lazy = RandomTensors(expected, seed, std=std, dtype=dtype, device=device)
    return {name: lazy[name] for name in expected}


def write_model_folder(folder: str | Path, config: dict, tensors: dict) -> Path:
    """Write ``config.json`` and ``model.safetensors``; returns the folder."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config, indent=2) + "\n")
    save_file({k: v.detach().cpu().contiguous() for k, v in tensors.items()}, str(folder / SINGLE_NAME))
    return folder
