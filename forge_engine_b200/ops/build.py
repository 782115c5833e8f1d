"""Build the CUDA sources of ``csrc/`` into one shared library, in-tree.

nvcc is called directly (no framework headers are needed: the kernels take raw
pointers), one process per source file, then one link.  The library is rebuilt only
when a source, a header or a flag changed.  While compiling, a line is printed to
stderr for every file so that a first call in a fresh checkout shows it is alive.
If the package folder cannot be written, a per-user temporary folder is used.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

from ..errors import CUDAUnavailableError

CSRC = Path(__file__).resolve().parent.parent / "csrc"
LIB_NAME = "libforge_engine_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def find_nvcc() -> str:
    for candidate in (
        os.environ.get("FORGE_ENGINE_NVCC"),
        shutil.which("nvcc"),
        "/usr/local/cuda/bin/nvcc",
        os.path.join(os.environ.get("CUDA_HOME", "/nonexistent"), "bin", "nvcc"),
    ):
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise CUDAUnavailableError("nvcc was not found; the CUDA kernels cannot be built")


# Sources compiled once per head size (-DFE_HEAD_DIM=...), each into a library of its own.
PER_HEAD_DIM = ("attention_mma.cu",)


def _sources() -> list[Path]:
    return sorted(p for p in CSRC.glob("*.cu") if p.name not in PER_HEAD_DIM)


def _fingerprint(nvcc: str, sources: list, defines: list) -> str:
    digest = hashlib.sha256()
    for path in sorted(list(sources) + list(CSRC.glob("*.cuh"))):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + defines).encode())
    digest.update(nvcc.encode())
    return digest.hexdigest()


def _writable_dir() -> Path:
    target = CSRC / "_build"
    try:
        target.mkdir(exist_ok=True)
        probe = target / f".probe{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return target
    except OSError:
        fallback = Path(tempfile.gettempdir()) / f"forge_engine_b200_build_{os.getuid()}"
        fallback.mkdir(parents=True, exist_ok=True)
        return fallback


def _say(message: str) -> None:
    print(f"[forge-engine build] {message}", file=sys.stderr, flush=True)


def _build(lib_name: str, sources: list, defines: list, verbose: bool) -> Path:
    """Compile ``sources`` with ``defines`` into ``lib_name`` unless an up-to-date copy exists."""
    nvcc = find_nvcc()
    out_dir = _writable_dir()
    lib = out_dir / lib_name
    stamp = out_dir / (lib_name + ".fingerprint")
    fingerprint = _fingerprint(nvcc, sources, defines)
    if lib.is_file() and stamp.is_file() and stamp.read_text() == fingerprint:
        return lib
    started = time.time()
    if verbose:
        _say(f"compiling {len(sources)} CUDA file(s) for sm_100a into {out_dir / lib_name} (first call only)")
    tag = hashlib.sha256((lib_name + " ".join(defines)).encode()).hexdigest()[:8]

    def compile_one(src: Path) -> Path:
        obj = out_dir / f"{src.stem}.{tag}.{os.getpid()}.o"
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *defines, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        t0 = time.time()
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            raise CUDAUnavailableError(f"nvcc failed on {src.name}:\n{done.stdout}\n{done.stderr}")
        if verbose:
            _say(f"  {src.name} {' '.join(defines)} done in {time.time() - t0:.1f}s")
        return obj

    workers = max(1, min(len(sources), os.cpu_count() or 1))
    with ThreadPoolExecutor(max_workers=workers) as pool:
        objects = list(pool.map(compile_one, sources))
    tmp_lib = out_dir / f".{lib_name}.{os.getpid()}"
    link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp_lib), *map(str, objects)]
    done = subprocess.run(link, capture_output=True, text=True)
    for obj in objects:
        try:
            obj.unlink()
        except OSError:
            pass
    if done.returncode != 0:
        raise CUDAUnavailableError(f"linking {lib_name} failed:\n{done.stdout}\n{done.stderr}")
    os.replace(tmp_lib, lib)
    stamp.write_text(fingerprint)
    if verbose:
        _say(f"built {lib.name} in {time.time() - started:.1f}s")
    return lib


def library_path(verbose: bool = True) -> Path:
    """The library of kernels that take every size at run time."""
    return _build(LIB_NAME, _sources(), [], verbose)


def attention_library_path(head_dim: int, verbose: bool = True) -> Path:
    """The tensor-core attention kernels specialised for one head size."""
    if head_dim % 16 or not 16 <= head_dim <= 256:
        raise CUDAUnavailableError(f"no tensor-core attention for head_dim={head_dim}")
    name = f"libforge_engine_b200_attn_d{head_dim}.so"
    return _build(name, [CSRC / n for n in PER_HEAD_DIM], [f"-DFE_HEAD_DIM={head_dim}"], verbose)
