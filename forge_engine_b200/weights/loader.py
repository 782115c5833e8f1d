"""Read a checkpoint's tensors by name from safetensors files.

Upstream copies one tensor at a time by name from the shards listed in
``model.safetensors.index.json`` and refuses name-set, shape and dtype mismatches
(src/forge_engine/weights.py:202-243).  Here a single ``model.safetensors`` without an
index is accepted as well, and *all* problems are reported in one error.

Tensors are read when the model asks for them, one at a time, as upstream copies one
tensor at a time into a model built without storage (src/forge_engine/weights.py:193-196,
210-243): ``open_checkpoint`` checks names, shapes and stored dtypes from the files'
headers and returns a mapping that reads a tensor from its shard and puts it on the device
on access.  The model is assembled layer by layer, each part fusing what it needs
(q/k/v rows, gate/up rows) and dropping the sources, so that at no time more than one
layer's tensors exist twice.  Every tensor is also checked for NaN and infinities
(src/forge_engine/weights.py:240-241); the flags are read once, in ``close()``.

Dtype rule: in the bfloat16 engine a tensor stays in the dtype it is stored in
(bfloat16 stays bfloat16, a tensor stored in 32-bit stays 32-bit, float16 is rounded
to bfloat16, integer tables become int32); in the float32 engine every floating
tensor is raised to 32-bit, which is exact.
"""

from __future__ import annotations

import json
from collections.abc import Mapping
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


_FLOAT_NAMES = {"F64", "F32", "F16", "BF16"}


def _stored_dtype(handle, name: str) -> str:
    """The dtype string of the file's header ("BF16", "F32", "I64", ...)."""
    try:
        return str(handle.get_slice(name).get_dtype())
    except Exception:  # older bindings: read the tensor
        return {torch.float64: "F64", torch.float32: "F32", torch.float16: "F16",
                torch.bfloat16: "BF16"}.get(handle.get_tensor(name).dtype, "other")


def _all_finite(tensor: torch.Tensor) -> torch.Tensor:
    """0-d bool tensor on the tensor's device; large tensors are tested in pieces, so that the
    test's temporaries (an absolute value and masks, several bytes per element) stay small
    beside the tensor."""
    flat = tensor.reshape(-1)
    piece = 1 << 20
    if flat.numel() <= piece:
        return torch.isfinite(flat).all()
    ok = torch.ones((), dtype=torch.bool, device=tensor.device)
    for begin in range(0, flat.numel(), piece):
        ok = ok & torch.isfinite(flat[begin : begin + piece]).all()
    return ok


class CheckpointTensors(Mapping):
    """name -> tensor on the device, read from the shard when asked for (and not kept).

    Iteration follows ``expected``.  ``close()`` closes the shards and raises one
    ``WeightsError`` naming every tensor read so far that holds NaN or an infinity."""

    def __init__(self, folder: Path, expected: dict, by_name: dict, engine_dtype: torch.dtype, device) -> None:
        self.folder = folder
        self._expected = expected
        self._by_name = by_name          # name -> shard path
        self._dtype = engine_dtype
        self._device = device
        self._handles: dict = {}
        self._finite: list = []          # (name, 0-d bool tensor on the device)

    def __len__(self) -> int:
        return len(self._expected)

    def __iter__(self):
        return iter(self._expected)

    def __getitem__(self, name: str) -> torch.Tensor:
        if name not in self._expected:
            raise KeyError(name)
        path = self._by_name[name]
        handle = self._handles.get(path)
        if handle is None:
            handle = self._handles[path] = safe_open(str(path), framework="pt", device="cpu").__enter__()
        tensor = _keep_dtype(handle.get_tensor(name), self._dtype).to(self._device)
        if tensor.is_floating_point():
            self._finite.append((name, _all_finite(tensor)))
        return tensor

    def close(self) -> None:
        for handle in self._handles.values():
            handle.__exit__(None, None, None)
        self._handles.clear()
        flags, self._finite = self._finite, []
        if flags:
            finite = torch.stack([flag for _, flag in flags]).cpu().tolist()   # one read-back
            bad = [name for (name, _), ok in zip(flags, finite) if not ok]
            if bad:
                raise WeightsError(
                    f"checkpoint in {self.folder} holds values that are not finite:\n"
                    f"  NaN or infinity ({len(bad)}): " + ", ".join(bad)
                )

    def __enter__(self) -> "CheckpointTensors":
        return self

    def __exit__(self, exc_type, exc, tb) -> None:
        if exc_type is None:
            self.close()
        else:
            for handle in self._handles.values():
                handle.__exit__(None, None, None)
            self._handles.clear()


def open_checkpoint(
    folder: str | Path,
    expected: dict,
    engine_dtype: torch.dtype,
    device,
    optional: tuple = (),
) -> CheckpointTensors:
    """Check the files' headers against ``expected`` (name -> WeightInfo) and return the
    lazy mapping.  All problems - missing and unexpected names, wrong shapes, a matrix, norm
    or bias that is not stored as floating point - are listed in one error.

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
    wrong, wrong_dtype = [], []
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
                stored = _stored_dtype(handle, name)
                if getattr(expected[name], "role", "matrix") in ("matrix", "norm", "bias") and stored not in _FLOAT_NAMES:
                    wrong_dtype.append(f"{name}: stored as {stored}, a floating-point tensor is needed")
    if missing or unexpected or wrong or wrong_dtype:
        lines = [f"checkpoint in {folder} does not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(wrong))
        if wrong_dtype:
            lines.append(f"  wrong dtypes ({len(wrong_dtype)}): " + "; ".join(wrong_dtype))
        raise WeightsError("\n".join(lines))
    by_name = {name: path for path, names in by_file.items() for name in names}
    return CheckpointTensors(folder, expected, by_name, engine_dtype, device)


def load_checkpoint(
    folder: str | Path,
    expected: dict,
    engine_dtype: torch.dtype,
    device,
    optional: tuple = (),
) -> dict:
    """All tensors of ``expected`` at once: name -> tensor on ``device`` (what
    ``open_checkpoint`` gives, read eagerly and checked)."""
    with open_checkpoint(folder, expected, engine_dtype, device, optional) as tensors:
        return {name: tensors[name] for name in expected}
