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


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _fingerprint(nvcc: str) -> str:
    digest = hashlib.sha256()
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh"))):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
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


def library_path(build_if_needed: bool = True, verbose: bool = True) -> Path:
    """Return the path of an up-to-date library, compiling it first if necessary."""
    nvcc = find_nvcc()
    out_dir = _writable_dir()
    lib = out_dir / LIB_NAME
    stamp = out_dir / "fingerprint.txt"
    fingerprint = _fingerprint(nvcc)
    if lib.is_file() and stamp.is_file() and stamp.read_text() == fingerprint:
        return lib
    if not build_if_needed:
        raise CUDAUnavailableError(f"{lib} is missing or stale")
    sources = _sources()
    started = time.time()
    if verbose:
        _say(f"compiling {len(sources)} CUDA files for sm_100a into {out_dir} (first call only)")

    def compile_one(src: Path) -> Path:
        obj = out_dir / (src.stem + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        t0 = time.time()
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            raise CUDAUnavailableError(f"nvcc failed on {src.name}:\n{done.stdout}\n{done.stderr}")
        if verbose:
            _say(f"  {src.name} done in {time.time() - t0:.1f}s")
        return obj

    workers = max(1, min(len(sources), os.cpu_count() or 1))
    with ThreadPoolExecutor(max_workers=workers) as pool:
        objects = list(pool.map(compile_one, sources))
    tmp_lib = out_dir / f".{LIB_NAME}.{os.getpid()}"
    link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp_lib), *map(str, objects)]
    done = subprocess.run(link, capture_output=True, text=True)
    if done.returncode != 0:
        raise CUDAUnavailableError(f"linking {LIB_NAME} failed:\n{done.stdout}\n{done.stderr}")
    os.replace(tmp_lib, lib)
    stamp.write_text(fingerprint)
    if verbose:
        _say(f"built {lib.name} in {time.time() - started:.1f}s")
    return lib
