"""Helpers shared by the GPU tests: model folders from plain weights, trace replay."""

from __future__ import annotations

import json
import struct
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch
from safetensors.torch import save_file

import plain_qwen3 as plain

ROOT = Path(__file__).resolve().parent.parent


def make_model_folder(folder: Path, raw: dict, seed: int, store_dtype=torch.bfloat16):
    """Write config.json + model.safetensors with the plain implementation's seeded
    weights (values are bfloat16-representable, so both store dtypes hold the same model).
    Returns (PlainConfig, weights as float32)."""
    cfg = plain.PlainConfig.from_dict(raw)
    weights = plain.seeded_weights(cfg, seed)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(raw))
    save_file({k: v.to(store_dtype).contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    return cfg, weights


def random_ids(vocab: int, length: int, seed: int) -> list:
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=generator).tolist()


def run_trace(model_dir: Path, out_dir: Path, dtype: str, max_tokens: int, steps: list,
              extra_args: tuple = ()) -> dict:
    """Run bin/trace_run on ``steps`` (list of dicts) and return {step: float32 array [wanted, vocab]}."""
    vocab = json.loads((model_dir / "config.json").read_text())["vocab_size"]
    payload = "".join(json.dumps(s) + "\n" for s in steps)
    done = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
         "--out", str(out_dir), "--max-tokens", str(max_tokens), *extra_args],
        input=payload, capture_output=True, text=True, timeout=900,
    )
    if done.returncode != 0:
        raise RuntimeError(f"trace_run failed ({done.returncode}):\n{done.stdout[-2000:]}\n{done.stderr[-4000:]}")
    lines = [l for l in done.stdout.splitlines() if l.startswith("done ")]
    assert [l.split()[1] for l in lines] == [str(s["step"]) for s in steps], done.stdout[-2000:]
    out = {}
    for s in steps:
        path = out_dir / f"{s['step']}.f32"
        wanted = sum(len(e.get("want", [])) for e in s["entries"])
        if wanted:
            out[s["step"]] = np.fromfile(str(path), dtype="<f4").reshape(wanted, vocab)
        else:
            assert not path.exists()
    return out
