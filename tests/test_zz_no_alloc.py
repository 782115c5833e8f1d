"""The allocation-free decode attention entry point, called through its exported C symbol.

Programs that embed the kernel library without torch (or that have given all device
memory to an allocator of their own, or cannot afford cudaMalloc's device-wide stall in a
serving loop) call ``fe_attention_decode_noalloc_d<HEAD>``: its scratch is an array inside
the library.  Here it is loaded with ctypes exactly as such a program would, and its output
is compared with the usual entry point's (which gets a workspace from the caller) on two
calls in a row with different inputs, so that whatever the first call left in the shared
scratch is shown not to matter.  This file sorts last on purpose: a run that stops at the
first failure has then already run every other test.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

from test_gpu_kernels import DEV, dense_attention, paged_layout, plant_keys, status_word

pytestmark = pytest.mark.gpu

HEAD = 128


def load_symbol():
    from forge_engine_b200.ops import native
    from forge_engine_b200.ops.build import attention_library_path

    native.require_cuda()
    handle = ctypes.CDLL(str(attention_library_path(HEAD)))
    fn = getattr(handle, f"fe_attention_decode_noalloc_d{HEAD}")
    p, i = c_void_p, c_int
    fn.argtypes = [p, i, p, p, p, p, i, i, i, i, i, p, p, i, i, i, c_float, i, p, p]
    fn.restype = c_int
    return fn


def call_both(fn, seed: int, lengths: list, splits: int, window: int, new: int = 1, nq: int = 32, nkv: int = 8):
    """One step of ``new`` tokens per entry through both entry points.  The last query of
    every entry is aimed at single keys on the edges of its window and of its key tiles, so
    that a key missed at a split's border or admitted from outside the window would show."""
    from forge_engine_b200.ops import native

    page = 16
    k_cache, v_cache, table, keys, values = paged_layout(lengths, page, nkv, HEAD, torch.bfloat16, seed=seed)
    g = torch.Generator().manual_seed(seed + 1)
    entries = len(lengths)
    q = torch.randn((entries * new, nq * HEAD), generator=g).to(torch.bfloat16)
    for r, n in enumerate(lengths):
        if n >= 2:
            plant_keys(k_cache, v_cache, table, keys, values, r, window, q[(r + 1) * new - 1])
    q = q.to(DEV)
    cu = torch.arange(0, entries * new + 1, new, dtype=torch.int32, device=DEV)
    starts = torch.tensor([n - new for n in lengths], dtype=torch.int32, device=DEV)
    scale = HEAD ** -0.5
    usual = torch.empty((entries * new, nq * HEAD), dtype=torch.bfloat16, device=DEV)
    status = status_word()
    native.attention_mma(q, nq * HEAD, k_cache, v_cache, table, cu, starts, entries, new, window, scale, usual,
                         nq, status, run_prefill=False, run_decode=True, num_splits=splits)
    mine = torch.full_like(usual, float("nan"))
    torch.cuda.synchronize()
    # what the call itself does to the allocator: nothing (its scratch is inside the library)
    held, reserved = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    code = fn(q.data_ptr(), nq * HEAD, mine.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), table.data_ptr(),
              table.shape[1], page, k_cache.shape[0], nkv, nq // nkv, cu.data_ptr(), starts.data_ptr(), entries, new,
              window, scale, splits, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == (held, reserved)
    assert code == 0 and int(status.item()) == 0
    # against the usual entry point: the same kernels on the same inputs, so the same numbers
    torch.testing.assert_close(mine.float(), usual.float(), atol=2e-2, rtol=2e-2)
    # and against the dense 64-bit reference, with the tolerance of the other attention tests
    for r, n in enumerate(lengths):
        rows = q[r * new : (r + 1) * new].cpu().view(new, nq, HEAD)
        ref = dense_attention(rows, keys[r], values[r], torch.arange(n - new, n), scale, window)
        torch.testing.assert_close(mine[r * new : (r + 1) * new].double().cpu().view(new, nq, HEAD), ref,
                                   atol=2e-2, rtol=2e-2)
    return mine


def test_no_alloc_entry_matches_the_usual_one_twice_in_a_row() -> None:
    fn = load_symbol()
    first = call_both(fn, 11, [700, 64, 1, 2048], splits=6, window=0)
    second = call_both(fn, 23, [1500, 333, 65], splits=9, window=400)   # other sizes over the leftovers
    assert first.shape != second.shape
    call_both(fn, 31, [900, 70, 2100], splits=4, window=70)
    # one split: results go straight to the output, the array is not used, so entry counts
    # far beyond what the array could hold for more splits are taken
    call_both(fn, 37, [130] * 150 + [1, 600], splits=1, window=0)
    # a few new tokens per entry (4 tokens x 4 heads per kv head = the kernel's 16 rows)
    call_both(fn, 41, [500, 68, 4], splits=3, window=0, new=4)
    call_both(fn, 43, [300, 77], splits=2, window=100, new=2, nq=16, nkv=2)


def test_no_alloc_entry_refuses_what_does_not_fit() -> None:
    fn = load_symbol()
    dummy = torch.zeros(64, dtype=torch.int32, device=DEV)
    aligned = torch.zeros(4096, dtype=torch.bfloat16, device=DEV)
    args = lambda entries, splits, max_new=1: (  # noqa: E731
        aligned.data_ptr(), 4096, aligned.data_ptr(), aligned.data_ptr(), aligned.data_ptr(), dummy.data_ptr(), 1, 16,
        1, 8, 4, dummy.data_ptr(), dummy.data_ptr(), entries, max_new, 0, 0.1, splits, dummy.data_ptr(), 0)
    assert fn(*args(64, 8)) == 10005       # 64 * 8 * 8 * 16 * 130 floats > 1,048,576
    assert fn(*args(1, 1, max_new=5)) == 10002   # 5 tokens x 4 heads = 20 rows: not a decode shape
    torch.cuda.synchronize()
