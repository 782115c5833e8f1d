"""ctypes binding of the kernel library and thin tensor-level wrappers.

Every wrapper checks dtype, device and contiguity, passes raw pointers and the
current CUDA stream, and raises on a non-zero return.  There is no fallback: without
a CUDA device or without the library these functions raise ``CUDAUnavailableError``.
"""

from __future__ import annotations

import ctypes
import os as _os
from ctypes import c_float, c_int, c_ulonglong, c_void_p

import torch

from ..errors import CUDAUnavailableError, ForgeEngineError, UnsupportedShapeError
from .build import attention_library_path, library_path

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

STATUS_BITS = {
    1: "a token id lies outside the vocabulary",
    2: "a block-table entry is negative or outside the page pool",
    4: "a position lies outside its request's block table",
    8: "a bounded wait inside a kernel ran out",
    16: "logits contain NaN or +inf",
}

_ERRORS = {
    10001: "unsupported dtype combination",
    10002: "unsupported shape",
    10003: "pointer or stride not aligned as the kernel needs",
    10004: "size beyond what the kernel can launch",
}

_lib = None

# Kernel launches issued through this module since import (a claim for benchmarks).
LAUNCHES = 0


def lib() -> ctypes.CDLL:
    """Load (building first if needed) the kernel library exactly once."""
    global _lib
    if _lib is None:
        path = library_path()
        try:
            _lib = ctypes.CDLL(str(path))
        except OSError as error:
            raise CUDAUnavailableError(f"cannot load {path}: {error}") from error
        _declare(_lib)
    return _lib


def _declare(handle: ctypes.CDLL) -> None:
    p, i, f = c_void_p, c_int, c_float
    signatures = {
        "fe_embedding": [p, p, i, p, i, i, i, p, p],
        "fe_add_rmsnorm": [p, p, i, p, p, i, p, i, i, f, i, p],
        "fe_silu_mul": [p, p, i, i, i, i, p],
        "fe_qk_rope_cache": [p, i, p, p, f, p, p, i, p, p, p, p, p, i, i, i, i, i, i, i, i, p, p],
        "fe_qk_rope_cache_sums": [p, p, p, p, f, p, p, p, p, p, p, p, i, i, i, i, i, i, i, i, p, p],
        "fe_rope_table": [p, p, i, i, p, p],
        "fe_attention_simt": [p, i, i, p, p, p, i, i, i, p, p, i, f, p, i, i, i, i, p, p],
        "fe_gemm_simt": [p, i, p, i, p, p, i, i, i, i, i, p],
        "fe_sample": [p, i, i, p, p, p, p, p, p, p, p, p],
        "fe_gemm_tc5": [p, p, p, p, i, i, i, i, i, p, p, p, p],
        "fe_gemm_tc5_qkv_rope": [p, p, p, p, i, i, i, p, p, f, p, p, p, p, p, p, i, i, i, i, i, i, p, p],
    }
    for name, argtypes in signatures.items():
        fn = getattr(handle, name)
        fn.argtypes = argtypes
        fn.restype = c_int
    handle.fe_uniform_host.argtypes = [c_ulonglong, c_ulonglong]
    handle.fe_uniform_host.restype = c_float


_attention_libs: dict = {}
_attention_handles: dict = {}


def attention_lib(head_dim: int):
    """The tensor-core attention entry point compiled for ``head_dim`` (built on first use)."""
    fn = _attention_libs.get(head_dim)
    if fn is None:
        path = attention_library_path(head_dim)
        try:
            handle = ctypes.CDLL(str(path))
        except OSError as error:
            raise CUDAUnavailableError(f"cannot load {path}: {error}") from error
        fn = getattr(handle, f"fe_attention_mma_d{head_dim}")
        p, i, f = c_void_p, c_int, c_float
        fn.argtypes = [p, i, p, p, p, p, i, i, i, i, i, p, p, i, i, i, i, f, i, i, p, p, p, p]
        fn.restype = c_int
        _attention_libs[head_dim] = fn
        _attention_handles[head_dim] = handle
    return fn


def has_symbol(name: str) -> bool:
    return hasattr(lib(), name)


def check(code: int, what: str) -> None:
    global LAUNCHES
    if code == 0:
        LAUNCHES += 1
        return
    if code in _ERRORS:
        raise UnsupportedShapeError(f"{what}: {_ERRORS[code]}")
    raise ForgeEngineError(f"{what}: CUDA error {code}")


# ---------------------------------------------------------------------------
# scratch memory with canary words
# ---------------------------------------------------------------------------

CANARY = 0x5AFEC0DE
GUARD_BYTES = 256


class GuardedBuffer:
    """A device buffer with ``GUARD_BYTES`` of a fixed bit pattern before and after it.

    Stands in for a memory checker: a kernel that writes one element before or past its
    scratch (or its cache pool) changes a canary word, which ``damaged()`` reports."""

    def __init__(self, name: str, numel: int, dtype: torch.dtype, device, zero: bool = False) -> None:
        self.name = name
        item = torch.empty((), dtype=dtype).element_size()
        guard = GUARD_BYTES // item
        body = -(-max(1, numel) // guard) * guard          # the rear guard starts 256-byte aligned
        flat = (torch.zeros if zero else torch.empty)(guard + body + guard, dtype=dtype, device=device)
        self._flat = flat
        self.data = flat[guard : guard + numel]
        self._guards = (flat[:guard].view(torch.int32), flat[guard + body :].view(torch.int32))
        for words in self._guards:
            words.fill_(CANARY)

    def numel(self) -> int:
        return self.data.numel()

    def damaged(self) -> torch.Tensor:
        """0-d bool tensor on the device: a canary word was overwritten."""
        return (self._guards[0] != CANARY).any() | (self._guards[1] != CANARY).any()


class _Scratch:
    """Scratch buffers of this module, per (kind, device).  A buffer that turns out too
    small is replaced by a larger one; the old one stays referenced, because a captured CUDA
    graph may still hold its address."""

    def __init__(self) -> None:
        self.current: dict = {}
        self.all: list = []

    def get(self, kind: str, device, numel: int, dtype: torch.dtype, floor: int, zero: bool = False) -> torch.Tensor:
        key = (kind, torch.device(device))
        buffer = self.current.get(key)
        if buffer is None or buffer.numel() < numel:
            buffer = GuardedBuffer(f"{kind} scratch", max(numel, floor), dtype, device, zero)
            self.current[key] = buffer
            self.all.append(buffer)
        return buffer.data


_scratch = _Scratch()


def damaged_canaries(extra=()) -> list:
    """Names of the scratch buffers of this module (and of ``extra`` GuardedBuffers, such as
    the cache pools) whose canary words no longer hold their pattern; synchronises."""
    buffers = list(_scratch.all) + list(extra)
    if not buffers:
        return []
    by_device: dict = {}
    for buffer in buffers:
        by_device.setdefault(buffer.data.device, []).append(buffer)
    bad = []
    for group in by_device.values():
        flags = torch.stack([b.damaged() for b in group]).cpu().tolist()
        bad.extend(b.name for b, flag in zip(group, flags) if flag)
    return bad


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise CUDAUnavailableError("no CUDA device: this engine runs on the GPU only")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream() -> int:
    """Handle of the current CUDA stream of the current device (asked for at every launch: a
    graph capture runs on a stream of its own)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise UnsupportedShapeError(f"dtype {t.dtype} is neither float32 nor bfloat16") from None


def _dense(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise CUDAUnavailableError(f"{name} must live on the CUDA device")
    if not t.is_contiguous():
        raise UnsupportedShapeError(f"{name} must be contiguous")
    return t


# ---------------------------------------------------------------------------
# wrappers
# ---------------------------------------------------------------------------


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> None:
    """out[n] = float(table[ids[n]]); out is the 32-bit residual stream [N, H]."""
    _dense(ids, "ids"), _dense(table, "table"), _dense(out, "out")
    assert ids.dtype == torch.int32 and out.dtype == torch.float32
    n, hidden = out.shape
    check(
        lib().fe_embedding(ptr(ids), ptr(table), code(table), ptr(out), n, hidden, table.shape[0],
                           ptr(status), stream()),
        "embedding",
    )


def add_rmsnorm(
    residual: torch.Tensor,
    update: torch.Tensor | None,
    weight: torch.Tensor,
    out: torch.Tensor,
    eps: float,
    row_map: torch.Tensor | None = None,
    write_residual: bool = True,
) -> None:
    """residual += update (32-bit, in place unless ``write_residual`` is false);
    out = rmsnorm(residual) * weight.  With ``row_map`` row r of ``out`` comes from
    row ``row_map[r]`` of ``residual`` and ``update``."""
    _dense(residual, "residual"), _dense(weight, "weight"), _dense(out, "out")
    assert residual.dtype == torch.float32 and weight.dtype == torch.float32
    rows, size = out.shape
    assert residual.shape[1] == size and weight.numel() == size
    if update is not None:
        _dense(update, "update")
        assert update.shape == residual.shape
    if row_map is not None:
        assert row_map.dtype == torch.int32 and row_map.numel() == rows
    else:
        assert residual.shape[0] == rows
    check(
        lib().fe_add_rmsnorm(
            ptr(residual), ptr(update), code(update) if update is not None else code(out),
            ptr(weight), ptr(out), code(out), ptr(row_map), rows, size, float(eps),
            1 if write_residual else 0, stream(),
        ),
        "add_rmsnorm",
    )


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0) -> None:
    """out[n, i] = silu(gate[n, i]) * up[n, i].  ``block`` 0: a row of ``gate_up`` is all gate
    features then all up features; ``block`` B: it alternates B gate, B up features."""
    _dense(gate_up, "gate_up"), _dense(out, "out")
    rows, inter = out.shape
    assert gate_up.shape == (rows, 2 * inter) and gate_up.dtype == out.dtype
    check(lib().fe_silu_mul(ptr(gate_up), ptr(out), code(out), rows, inter, int(block), stream()), "silu_mul")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, table: torch.Tensor) -> None:
    """table[t, j] = (cos, sin) of float(positions[t]) * inv_freq[j], in 32-bit."""
    _dense(positions, "positions"), _dense(inv_freq, "inv_freq"), _dense(table, "table")
    n, half = positions.numel(), inv_freq.numel()
    assert positions.dtype == torch.int32 and inv_freq.dtype == torch.float32
    assert table.dtype == torch.float32 and table.shape == (n, half, 2)
    check(lib().fe_rope_table(ptr(positions), ptr(inv_freq), half, n, ptr(table), stream()), "rope_table")


def qk_rope_cache(
    qkv: torch.Tensor,
    q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None,
    eps: float,
    inv_freq: torch.Tensor | None,
    rotary_dim: int,
    positions: torch.Tensor,
    token_entry: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    num_q_heads: int,
    write_kv: bool,
    status: torch.Tensor,
    table: torch.Tensor | None = None,
) -> None:
    """Normalise and rotate q (in place) and k, and store k, v into their pages.

    qkv is [N, (nq + 2 nkv) * D]; the caches are [pages, nkv, page_size, D].  ``table``:
    ``rope_table`` of these tokens (then the kernel does not take cosine and sine itself)."""
    _dense(qkv, "qkv"), _dense(k_cache, "k_cache"), _dense(v_cache, "v_cache")
    _dense(block_table, "block_table")
    num_pages, nkv, page_size, head_dim = k_cache.shape
    n = qkv.shape[0]
    assert qkv.shape[1] == (num_q_heads + 2 * nkv) * head_dim
    assert k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
    assert block_table.dtype == torch.int32 and block_table.dim() == 2
    assert positions.dtype == torch.int32 and token_entry.dtype == torch.int32
    for w in (q_weight, k_weight, inv_freq, table):
        assert w is None or (w.dtype == torch.float32 and w.is_cuda and w.is_contiguous())
    assert table is None or (inv_freq is not None and table.shape == (n, rotary_dim // 2, 2))
    check(
        lib().fe_qk_rope_cache(
            ptr(qkv), code(qkv), ptr(q_weight), ptr(k_weight), float(eps), ptr(inv_freq), ptr(table),
            int(rotary_dim), ptr(positions), ptr(token_entry), ptr(k_cache), ptr(v_cache),
            ptr(block_table), block_table.shape[1], page_size, num_pages, num_q_heads, nkv,
            head_dim, n, 1 if write_kv else 0, ptr(status), stream(),
        ),
        "qk_rope_cache",
    )


def qk_rope_cache_sums(
    sums: torch.Tensor,
    q_out: torch.Tensor,
    q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None,
    eps: float,
    inv_freq: torch.Tensor | None,
    positions: torch.Tensor,
    token_entry: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    num_q_heads: int,
    write_kv: bool,
    status: torch.Tensor,
    table: torch.Tensor | None = None,
) -> None:
    """``qk_rope_cache`` for a projection whose k-splits were added into the 32-bit ``sums``
    [N, (nq + 2 nkv) * D]: reads the sums and leaves zeros behind, stores the finished
    queries as bfloat16 into the q columns of ``q_out`` (same shape) and k, v into their
    bfloat16 pages.  The whole head is rotated (or none of it: inv_freq and table None)."""
    _dense(sums, "sums"), _dense(q_out, "q_out"), _dense(k_cache, "k_cache"), _dense(v_cache, "v_cache")
    _dense(block_table, "block_table")
    num_pages, nkv, page_size, head_dim = k_cache.shape
    n = q_out.shape[0]
    width = (num_q_heads + 2 * nkv) * head_dim
    assert sums.dtype == torch.float32 and sums.numel() >= n * width and q_out.shape == (n, width)
    assert q_out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16
    assert block_table.dtype == torch.int32 and block_table.dim() == 2
    assert positions.dtype == torch.int32 and token_entry.dtype == torch.int32
    for w in (q_weight, k_weight, inv_freq, table):
        assert w is None or (w.dtype == torch.float32 and w.is_cuda and w.is_contiguous())
    assert table is None or table.shape == (n, head_dim // 2, 2)
    check(
        lib().fe_qk_rope_cache_sums(
            ptr(sums), ptr(q_out), ptr(q_weight), ptr(k_weight), float(eps), ptr(inv_freq), ptr(table),
            ptr(positions), ptr(token_entry), ptr(k_cache), ptr(v_cache), ptr(block_table),
            block_table.shape[1], page_size, num_pages, num_q_heads, nkv, head_dim, n,
            1 if write_kv else 0, ptr(status), stream(),
        ),
        "qk_rope_cache_sums",
    )


def projection_sums(device: torch.device, count: int) -> torch.Tensor:
    """A 32-bit buffer of at least ``count`` zeros that lives as long as the process, for
    projections that add their k-splits into it; whoever reads the sums puts zeros back."""
    return _scratch.get("projection sums", device, count, torch.float32, 1 << 20, zero=True)


def attention_simt(
    q: torch.Tensor,
    q_stride: int,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    positions: torch.Tensor,
    token_entry: torch.Tensor,
    window: int | None,
    scale: float,
    out: torch.Tensor,
    num_q_heads: int,
    status: torch.Tensor,
) -> None:
    """General paged causal attention; q row n starts at q + n * q_stride elements."""
    num_pages, nkv, page_size, head_dim = k_cache.shape
    n = out.shape[0]
    assert out.shape[1] == num_q_heads * head_dim and out.dtype == q.dtype == k_cache.dtype
    check(
        lib().fe_attention_simt(
            ptr(q), int(q_stride), code(q), ptr(k_cache), ptr(v_cache), ptr(block_table),
            block_table.shape[1], page_size, num_pages, ptr(positions), ptr(token_entry),
            int(window or 0), float(scale), ptr(out), num_q_heads, nkv, head_dim, n, ptr(status),
            stream(),
        ),
        "attention_simt",
    )


_balanced_blocks: dict = {}


def attention_balanced_blocks(head_dim: int) -> int:
    """Blocks the balanced decode kernel of this head size runs with (0: it cannot run)."""
    blocks = _balanced_blocks.get(head_dim)
    if blocks is None:
        attention_lib(head_dim)
        fn = getattr(_attention_handles[head_dim], f"fe_attn_balanced_blocks_d{head_dim}")
        fn.restype = c_int
        fn.argtypes = []
        blocks = _balanced_blocks[head_dim] = int(fn())
    return blocks


def _attention_counters(device, pairs: int) -> torch.Tensor:
    """Zeroed arrival counters, one per (entry, kv head); launches leave them zeroed."""
    return _scratch.get("attention counters", device, pairs, torch.int32, 8192, zero=True)


def _attention_workspace(device, floats: int) -> torch.Tensor:
    """Partial results of split decode attention.  One buffer per device serves every layer:
    a layer's attention has combined its parts before the next layer's begins."""
    return _scratch.get("attention workspace", device, floats, torch.float32, 1 << 22)


ATTN_DECODE_ROWS = 16  # rows (new tokens x heads per kv head) the split decode kernel takes


def attention_mma(
    q: torch.Tensor,
    q_stride: int,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    cu_tokens: torch.Tensor,
    starts: torch.Tensor,
    entries: int,
    max_new: int,
    window: int | None,
    scale: float,
    out: torch.Tensor,
    num_q_heads: int,
    status: torch.Tensor,
    run_prefill: bool,
    run_decode: bool,
    num_splits: int = 1,
    merge_in_kernel: bool = True,
) -> None:
    """Tensor-core paged attention (bfloat16).  Entries with more than 16 rows (new
    tokens x heads per kv head) go to the prefill kernel, the others to the split
    decode kernel; ``run_prefill`` / ``run_decode`` say which kinds the batch holds.
    ``num_splits`` blocks share a request's keys; 0 spreads the key tiles of all decode
    entries evenly over as many blocks as the GPU holds at once."""
    num_pages, nkv, page_size, head_dim = k_cache.shape
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    groups = num_q_heads // nkv
    mode = (1 if run_prefill else 0) | (2 if run_decode else 0)
    workspace = counters = None
    if run_decode and num_splits == 0:
        blocks = attention_balanced_blocks(head_dim)
        if blocks <= 0:
            raise UnsupportedShapeError(f"attention_mma: no balanced decode kernel for head size {head_dim}")
        workspace = _attention_workspace(q.device, 2 * blocks * ATTN_DECODE_ROWS * (head_dim + 2))
    elif run_decode and num_splits > 1:
        floats = entries * nkv * num_splits * ATTN_DECODE_ROWS * (head_dim + 2)
        workspace = _attention_workspace(q.device, floats)
        if merge_in_kernel:
            counters = _attention_counters(q.device, entries * nkv)
    check(
        attention_lib(head_dim)(
            ptr(q), int(q_stride), ptr(out), ptr(k_cache), ptr(v_cache), ptr(block_table),
            block_table.shape[1], page_size, num_pages, nkv, groups, ptr(cu_tokens), ptr(starts),
            entries, int(max_new), int(q.shape[0]), int(window or 0), float(scale), mode, int(num_splits),
            ptr(workspace), ptr(counters), ptr(status), stream(),
        ),
        "attention_mma",
    )


def gemm_simt(
    x: torch.Tensor,
    w: torch.Tensor,
    out: torch.Tensor,
    bias: torch.Tensor | None = None,
    accumulate: bool = False,
) -> None:
    """out = x @ w.T (+ bias) (+ out) with plain 32-bit FMAs; w is [out, in]."""
    _dense(x, "x"), _dense(w, "w"), _dense(out, "out")
    n, k = x.shape
    o = w.shape[0]
    assert w.shape[1] == k and out.shape == (n, o)
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == o)
    check(
        lib().fe_gemm_simt(ptr(x), code(x), ptr(w), code(w), ptr(bias), ptr(out), code(out), n, o, k,
                           1 if accumulate else 0, stream()),
        "gemm_simt",
    )


TC5_STORE_BF16, TC5_STORE_F32, TC5_ADD_F32, TC5_SILU_MUL = 0, 1, 2, 3


def tc5_tile(n: int) -> int:
    return 16 if n <= 16 else 32 if n <= 32 else 64 if n <= 64 else 128 if n <= 128 else 256


def _tc5_workspace(device, tiles: int, ksplit: int, tile_n: int):
    """(partial tiles, arrival counters) for k-splits that do not add up inside a cluster."""
    part = _scratch.get("gemm partial tiles", device, tiles * ksplit * tile_n * 128, torch.float32, 1 << 22)
    count = _scratch.get("gemm tile counters", device, tiles, torch.int32, 16384, zero=True)
    return part, count


def gemm_tc5_set_test_fault(wait_limit: int = 0, skip_kblock: int = -1) -> None:
    """For tests of the bounded waits: later ``gemm_tc5`` launches poll at most ``wait_limit``
    times per wait and leave out the load of k-block ``skip_kblock``, so that a block gives
    up, sets status bit 8 and returns.  ``(0, -1)`` restores the usual behaviour."""
    fn = lib().fe_gemm_tc5_set_test_fault
    fn.argtypes = [ctypes.c_uint, c_int]
    fn.restype = None
    fn(int(wait_limit), int(skip_kblock))


TC5_MAX_ROWS = int(_os.environ.get("FORGE_ENGINE_TC5_MAX_ROWS", "64"))   # up to this many rows the tcgen05 kernel is used instead of the library GEMM


_ADD_TARGET = int(_os.environ.get("FORGE_ENGINE_ADD_BLOCKS", "288"))
_ADD_LIMIT = int(_os.environ.get("FORGE_ENGINE_ADD_SPLITS", "16"))


def tc5_ksplit_add(o: int, k: int) -> int:
    """Blocks per 128-feature tile of a product that adds into the residual stream.  Its
    partial sums meet in memory through atomic adds, so the k-splits need not form a cluster
    and there may be more of them: about 288 blocks, just under the 296 a B200 holds at once
    (measured at the 4B shape, batch 8, per decode step: 2.60 ms with 8 splits, 2.53 with 12,
    2.51 with 14 or 15, 2.72 with 16 - 320 blocks no longer run in one round).  So whatever the
    number of tiles, the splits never make more blocks than are resident at once (two per SM;
    FORGE_ENGINE_RESIDENT_BLOCKS overrides the count).  A block keeps at least four 64-wide
    k-blocks."""
    tiles = -(-o // 128)
    fits = max(1, _resident_blocks() // tiles)          # never more blocks than run at once
    return max(1, min(_ADD_LIMIT, round(_ADD_TARGET / tiles), fits, (k // 64) // 4))


_SUMS_TARGET = int(_os.environ.get("FORGE_ENGINE_SUMS_BLOCKS", "0"))


def tc5_ksplit_sums(o: int, k: int, n: int) -> int:
    """Blocks per 128-feature tile of the q/k/v projection that adds its k-splits into 32-bit
    sums for ``n`` tokens.  Up to 16 tokens it aims at 240 blocks instead of 288: the attention
    kernel that follows finds room on more SMs while the projection still runs and has keys in
    flight earlier (4B shape, 48 tiles, per decode step at batch 1 / 8 / 16: 2.098 / 2.445 /
    2.915 ms with 5 splits against 2.105 / 2.460 / 2.929 with 6; at batch 32 and 64 six are
    better, 3.819 / 5.775 against 3.840 / 5.796 ms).  FORGE_ENGINE_SUMS_BLOCKS names another
    number of blocks to aim at."""
    target = _SUMS_TARGET or (240 if n <= 16 else _ADD_TARGET)
    tiles = -(-o // 128)
    return max(1, min(_ADD_LIMIT, round(target / tiles), max(1, _resident_blocks() // tiles), (k // 64) // 4))


_RESIDENT_BLOCKS = 0


def _resident_blocks() -> int:
    """Blocks of the tcgen05 product for few tokens that the GPU holds at once: two per SM."""
    global _RESIDENT_BLOCKS
    if not _RESIDENT_BLOCKS:
        _RESIDENT_BLOCKS = int(_os.environ.get("FORGE_ENGINE_RESIDENT_BLOCKS", "0")) or \
            2 * torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _RESIDENT_BLOCKS


def tc5_ksplit(o: int, k: int) -> int:
    """Blocks per 128-feature tile for few tokens.  A weight with few tiles is cut along k
    so that about 190 blocks stream it (measured best on a B200: 4 for 48 tiles, 8 for 20);
    up to 8 such blocks form a cluster and add their partial tiles through shared memory.
    A block keeps at least four 64-wide k-blocks."""
    tiles = -(-o // 128)
    return max(1, min(8, round(int(_os.environ.get("FORGE_ENGINE_TC5_BLOCKS", "192")) / tiles), (k // 64) // 4))


def gemm_tc5(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, status: torch.Tensor,
             bias: torch.Tensor | None = None, ksplit: int = 1) -> None:
    """out = x @ w.T on tcgen05 tensor cores (bfloat16 operands, TMA-fed).

    epilogue 0: out bf16 [n, o]; 1: out f32 [n, o]; 2: out f32 [n, o] += product;
    3: out bf16 [n, o/2] = silu(gate) * up for w whose rows alternate 16 gate, 16 up features.
    ``ksplit`` blocks share an output tile (deterministic reduction through a workspace)."""
    _dense(x, "x"), _dense(w, "w"), _dense(out, "out")
    n, k = x.shape
    o = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == k
    if epilogue == TC5_SILU_MUL:
        assert out.shape == (n, o // 2) and out.dtype == torch.bfloat16
    else:
        assert out.shape == (n, o)
        assert out.dtype == (torch.bfloat16 if epilogue == TC5_STORE_BF16 else torch.float32)
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == o)
    part = count = None
    ksplit = max(1, min(int(ksplit), -(-k // 64)))
    if ksplit > 1:
        tile_n = tc5_tile(n)
        tiles = -(-o // 128) * -(-n // tile_n)
        part, count = _tc5_workspace(x.device, tiles, ksplit, tile_n)
    check(lib().fe_gemm_tc5(ptr(x), ptr(w), ptr(bias), ptr(out), n, o, k, int(epilogue), ksplit, ptr(part),
                            ptr(count), ptr(status), stream()),
          "gemm_tc5")


def gemm_tc5_qkv_rope(
    x: torch.Tensor,
    w: torch.Tensor,
    bias: torch.Tensor | None,
    qkv: torch.Tensor,
    q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None,
    eps: float,
    table: torch.Tensor | None,
    positions: torch.Tensor,
    token_entry: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    num_q_heads: int,
    write_kv: bool,
    status: torch.Tensor,
    ksplit: int = 1,
) -> None:
    """The fused q/k/v projection of up to 64 tokens for heads of 128: x @ w.T on tcgen05,
    then per head the q/k RMS norm, the rotation and - for keys and values - the write into
    the cache pages, all in the product's epilogue.  ``qkv`` [n, (nq + 2 nkv) * 128] receives
    the finished queries (its key and value columns are not written).  ``table`` is the
    ``rope_table`` of these tokens [n, 64, 2], or None for no rotation."""
    _dense(x, "x"), _dense(w, "w"), _dense(qkv, "qkv"), _dense(k_cache, "k_cache"), _dense(v_cache, "v_cache")
    _dense(block_table, "block_table")
    n, k = x.shape
    num_pages, nkv, page_size, head_dim = k_cache.shape
    assert head_dim == 128 and n <= TC5_MAX_ROWS
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and qkv.dtype == torch.bfloat16
    assert k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16
    assert w.shape == ((num_q_heads + 2 * nkv) * 128, k) and qkv.shape == (n, w.shape[0])
    assert block_table.dtype == torch.int32 and block_table.dim() == 2
    assert positions.dtype == torch.int32 and token_entry.dtype == torch.int32
    for name, t in (("q_weight", q_weight), ("k_weight", k_weight), ("table", table), ("bias", bias)):
        assert t is None or (t.dtype == torch.float32 and t.is_cuda and t.is_contiguous()), \
            f"{name}: a contiguous 32-bit tensor on the GPU is needed, got {t.dtype} on {t.device}"
    assert table is None or table.shape == (n, 64, 2)
    check(
        lib().fe_gemm_tc5_qkv_rope(
            ptr(x), ptr(w), ptr(bias), ptr(qkv), n, k, max(1, min(8, int(ksplit))), ptr(q_weight), ptr(k_weight),
            float(eps), ptr(table), ptr(positions), ptr(token_entry), ptr(k_cache), ptr(v_cache), ptr(block_table),
            block_table.shape[1], page_size, num_pages, num_q_heads, nkv, 1 if write_kv else 0, ptr(status), stream(),
        ),
        "gemm_tc5_qkv_rope",
    )


# ---------------------------------------------------------------------------
# several dependent projections of a decode step in one persistent kernel
# ---------------------------------------------------------------------------

CHAIN_SRC_ACTIVATIONS, CHAIN_SRC_NORM = 0, 1
CHAIN_ADD, CHAIN_SILU_MUL = 0, 1
CHAIN_MAX_TOKENS = 16


class _ChainOp(ctypes.Structure):
    _fields_ = [("w", c_void_p), ("x", c_void_p), ("norm_w", c_void_p), ("out", c_void_p),
                ("m", c_int), ("k", c_int), ("src", c_int), ("epi", c_int), ("eps", c_float)]


def _chain_ops(ops: list):
    array = (_ChainOp * len(ops))()
    for slot, op in zip(array, ops):
        w = op["w"]
        slot.w, slot.x, slot.out = ptr(w), ptr(op["x"]), ptr(op["out"])
        slot.norm_w = ptr(op.get("norm_w"))
        slot.m, slot.k = int(w.shape[0]), int(w.shape[1])
        slot.src, slot.epi, slot.eps = int(op["src"]), int(op["epi"]), float(op.get("eps", 0.0))
    return array


def decode_chain_takes(shapes: list, n: int) -> bool:
    """Whether ``decode_chain`` takes projections of these ``(m, k, src, epi)`` for ``n`` tokens."""
    array = (_ChainOp * len(shapes))()
    for slot, (m, k, src, epi) in zip(array, shapes):
        slot.m, slot.k, slot.src, slot.epi = int(m), int(k), int(src), int(epi)
    fn = lib().fe_decode_chain_check
    fn.argtypes = [ctypes.POINTER(_ChainOp), c_int, c_int]
    fn.restype = c_int
    return fn(array, len(shapes), int(n)) == 0


def decode_chain(ops: list, n: int, status: torch.Tensor) -> None:
    """Up to three projections, each reading what the one before wrote, in one launch.

    Every op is a dict: ``w`` bfloat16 [m, k]; ``src`` CHAIN_SRC_ACTIVATIONS with ``x`` bfloat16
    [n, k], or CHAIN_SRC_NORM with ``x`` the 32-bit residual stream [n, k], ``norm_w`` [k] and
    ``eps`` (the operand is then rmsnorm(x) * norm_w); ``epi`` CHAIN_ADD with ``out`` 32-bit
    [n, m] that the product is added to, or CHAIN_SILU_MUL with ``out`` bfloat16 [n, m / 2] for
    a weight whose rows alternate 16 gate and 16 up features.  ``n`` <= 16 tokens."""
    for op in ops:
        w, x, out = _dense(op["w"], "w"), _dense(op["x"], "x"), _dense(op["out"], "out")
        m, k = w.shape
        assert w.dtype == torch.bfloat16 and x.shape == (n, k)
        if op["src"] == CHAIN_SRC_NORM:
            norm_w = _dense(op["norm_w"], "norm_w")
            assert x.dtype == torch.float32 and norm_w.dtype == torch.float32 and norm_w.numel() == k
        else:
            assert x.dtype == torch.bfloat16
        if op["epi"] == CHAIN_ADD:
            assert out.dtype == torch.float32 and out.shape == (n, m)
        else:
            assert out.dtype == torch.bfloat16 and out.shape == (n, m // 2)
    handle = lib()
    handle.fe_decode_chain_counters.restype = c_int
    handle.fe_decode_chain_staging.restype = c_int
    device = ops[0]["w"].device
    counters = _scratch.get("chain counters", device, handle.fe_decode_chain_counters(), torch.int32, 0, zero=True)
    staging = _scratch.get("chain staging", device, handle.fe_decode_chain_staging(), torch.float32, 0, zero=True)
    fn = handle.fe_decode_chain
    fn.argtypes = [ctypes.POINTER(_ChainOp), c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
    fn.restype = c_int
    check(fn(_chain_ops(ops), len(ops), int(n), ptr(counters), ptr(staging), ptr(status), stream()), "decode_chain")


def sample(
    logits: torch.Tensor,
    out: torch.Tensor,
    status: torch.Tensor,
    temperature: torch.Tensor | None = None,
    top_k: torch.Tensor | None = None,
    top_p: torch.Tensor | None = None,
    min_p: torch.Tensor | None = None,
    seeds: torch.Tensor | None = None,
    counters: torch.Tensor | None = None,
) -> None:
    """One token per row of 32-bit logits; all parameter tensors are per row."""
    _dense(logits, "logits")
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and out.numel() >= rows
    for t, dt in ((temperature, torch.float32), (top_k, torch.int32), (top_p, torch.float32),
                  (min_p, torch.float32), (seeds, torch.int64), (counters, torch.int64)):
        assert t is None or (t.dtype == dt and t.is_cuda and t.numel() >= rows)
    check(
        lib().fe_sample(ptr(logits), rows, vocab, ptr(temperature), ptr(top_k), ptr(top_p), ptr(min_p),
                        ptr(seeds), ptr(counters), ptr(out), ptr(status), stream()),
        "sample",
    )
