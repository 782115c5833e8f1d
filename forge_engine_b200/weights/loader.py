"""Read a checkpoint's tensors by name from safetensors files.

Upstream copies one tensor at a time by name from the shards listed in
``model.safetensors.index.json`` and refuses name-set, shape and dtype mismatches
(src/forge_engine/weights.py:202-243).  Here a single ``model.safetensors`` without an
index is accepted as well, and *all* problems are reported in one error.

Dtype rule: in the bfloat16 engine a tensor stays in the dtype it is stored in
(bfloat16 stays bfloat16, a tensor stored in 32-bit stays 32-bit, float16 is rounded
to bfloat16, integer tables become int32); in the float32 engine every floating
tensor is raised to 32-bit, which is exact.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors import safe_open

from ..errors import WeightsError

INDEX_NAME = "model.safetensors.index.json"
SINGLE_NAME = "model.safetensors"


def _files_by_tensor(folder: Path) -> dict:
    index = folder / INDEX_NAME
    if index.is_file():
        weight_map = json.loads(index.read_text()).get("weight_map")
        if not isinstance(weight_map, dict):
            raise WeightsError(f"{index} has no 'weight_map'")
        return {name: folder / shard for name, shard in weight_map.items()}
    files = [folder / SINGLE_NAME] if (folder / SINGLE_NAME).is_file() else sorted(folder.glob("*.safetensors"))
    if not files:
        raise WeightsError(f"no safetensors file in {folder}")
    out: dict[str, Path] = {}
    for path in files:
        with safe_open(str(path), framework="pt", device="cpu") as handle:
            for name in handle.keys():
                out[name] = path
    return out


def _keep_dtype(tensor: torch.Tensor, engine_dtype: torch.dtype) -> torch.Tensor:
    if not tensor.is_floating_point():
        return tensor.to(torch.int32)
    if engine_dtype == torch.float32:
        return tensor.float()
    if tensor.dtype in (torch.float32, torch.bfloat16):
        return tensor
    if tensor.dtype == torch.float64:
        return tensor.float()
    return tensor.to(torch.bfloat16)


def load_checkpoint(
    folder: str | Path,
    expected: dict,
    engine_dtype: torch.dtype,
    device,
    optional: tuple = (),
) -> dict:
    """Return name -> tensor on ``device`` for exactly the names of ``expected``.

    ``optional`` names may be present in the files without being expected (a tied
    model that also stores its output head); they are not loaded."""
    folder = Path(folder)
    located = _files_by_tensor(folder)
    missing = [name for name in expected if name not in located]
    unexpected = sorted(name for name in located if name not in expected and name not in optional)
    by_file: dict[Path, list] = {}
    for name in expected:
        if name in located:
            by_file.setdefault(located[name], []).append(name)
    wrong = []
    absent_files = [str(p) for p in by_file if not p.is_file()]
    if absent_files:
        raise WeightsError("checkpoint shards are missing: " + ", ".join(absent_files))
    for path, names in by_file.items():
        with safe_open(str(path), framework="pt", device="cpu") as handle:
            present = set(handle.keys())
            for name in names:
                if name not in present:
                    missing.append(name)
                    continue
                shape = tuple(handle.get_slice(name).get_shape())
                if shape != tuple(expected[name].shape):
                    wrong.append(f"{name}: stored {shape}, model needs {tuple(expected[name].shape)}")
    if missing or unexpected or wrong:
        lines = [f"checkpoint in {folder} does not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(wrong))
        raise WeightsError("\n".join(lines))
    out: dict[str, torch.Tensor] = {}
    for path in sorted(by_file):
        with safe_open(str(path), framework="pt", device="cpu") as handle:
            for name in by_file[path]:
                out[name] = _keep_dtype(handle.get_tensor(name), engine_dtype).to(device)
    return {name: out[name] for name in expected}
