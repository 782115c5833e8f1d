"""Seeded random weights: in memory, or written out as a model folder.

Upstream has no such mode (its tests rely on torch's default initialisers,
tests/test_qwen3.py:48-49).  Here matrices and biases are N(0, std), norm weights are
1 + N(0, 0.1); tensors are drawn in the fixed order of ``expected_tensors``.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors.torch import save_file

from .loader import SINGLE_NAME


def random_tensors(expected: dict, seed: int, *, std: float = 0.02, dtype=torch.bfloat16,
                   device="cpu") -> dict:
    """Draw every tensor of ``expected`` from one generator seeded with ``seed``.

    On the CPU the values are the same on every machine; on a CUDA device they are
    reproducible for that device type only (used for benchmark-sized models)."""
    generator = torch.Generator(device=device).manual_seed(seed)
    out = {}
    for name, info in expected.items():
        noise = torch.randn(info.shape, generator=generator, dtype=torch.float32, device=device)
        value = noise.mul_(0.1).add_(1.0) if info.role == "norm" else noise.mul_(std)
        out[name] = value.to(dtype)
    return out


def write_model_folder(folder: str | Path, config: dict, tensors: dict) -> Path:
    """Write ``config.json`` and ``model.safetensors``; returns the folder."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config, indent=2) + "\n")
    save_file({k: v.detach().cpu().contiguous() for k, v in tensors.items()}, str(folder / SINGLE_NAME))
    return folder
