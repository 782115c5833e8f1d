"""Kernels at sizes drawn from a seed, where the other kernel tests name theirs: the tcgen05
product with its epilogues and k-splits, and the tensor-core attention kernels (prefill,
split decode, the decode form that spreads key tiles evenly), each against a 64-bit
reference of the same rounded inputs."""

from __future__ import annotations

import random

import pytest
import torch

import test_gpu_attention_mma as attention_cases
from test_gpu_kernels import DEV, status_word

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def native():
    from forge_engine_b200.ops import native as module

    module.require_cuda()
    module.lib()
    return module


def test_tcgen05_product_at_random_sizes(native) -> None:
    """1 to 64 tokens, 8 to 4,104 output features (no multiple of the 128-feature tile
    needed), inner sizes from 8 to 4,104 in steps of 8, 1 to 16 k-splits (more than 8 do not
    form a cluster; more than the inner size has 64-wide blocks are cut down), with and
    without bias: 32-bit store, bfloat16 store, add into a 32-bit tensor twice in a row, and
    SiLU(gate) * up over interleaved rows."""
    from forge_engine_b200.parts.linear import interleave_rows

    rng = random.Random(41)
    status = status_word()
    for trial in range(120):
        n = rng.choice([1, 2, 3, 7, 8, 9, 15, 16, 17, 31, 32, 33, 47, 63, 64])
        o = rng.choice([8, 16, 24, 100, 128, 136, 256, 520, 1000, 2560, 4104])
        k = 8 * rng.choice([1, 2, 3, 7, 8, 9, 16, 31, 32, 33, 100, 320, 513])
        ksplit = rng.choice([1, 1, 2, 3, 4, 5, 8, 11, 14, 16])
        g = torch.Generator().manual_seed(trial)
        x = torch.randn((n, k), generator=g).bfloat16().to(DEV)
        w = (torch.randn((o, k), generator=g) * k ** -0.5).bfloat16().to(DEV)
        bias = torch.randn(o, generator=g).to(DEV) if rng.random() < 0.5 else None
        ref = x.double() @ w.double().t() + (bias.double() if bias is not None else 0)
        mode = rng.choice(["f32", "bf16", "add", "add", "silu"])
        what = f"trial {trial}: {n} tokens, {o} features, inner size {k}, {ksplit} splits, bias {bias is not None}, {mode}"
        if mode == "f32":
            out = torch.full((n, o), float("nan"), dtype=torch.float32, device=DEV)
            native.gemm_tc5(x, w, out, native.TC5_STORE_F32, status, bias=bias, ksplit=ksplit)
            torch.testing.assert_close(out.double(), ref, atol=3e-4, rtol=1e-5, msg=lambda m: f"{what}: {m}")
        elif mode == "bf16":
            out = torch.full((n, o), float("nan"), dtype=torch.bfloat16, device=DEV)
            native.gemm_tc5(x, w, out, native.TC5_STORE_BF16, status, bias=bias, ksplit=ksplit)
            torch.testing.assert_close(out.double(), ref, atol=1e-2, rtol=1e-2, msg=lambda m: f"{what}: {m}")
        elif mode == "add":
            base = torch.randn((n, o), generator=g).to(DEV)
            acc = base.clone()
            for _ in range(2):
                native.gemm_tc5(x, w, acc, native.TC5_ADD_F32, status, bias=bias, ksplit=ksplit)
            torch.testing.assert_close(acc.double(), base.double() + 2 * ref, atol=6e-4, rtol=1e-5, msg=lambda m: f"{what}: {m}")
        else:
            inter = -(-o // 32) * 16
            gate = (torch.randn((inter, k), generator=g) * k ** -0.5).bfloat16().to(DEV)
            up = (torch.randn((inter, k), generator=g) * k ** -0.5).bfloat16().to(DEV)
            expected = torch.nn.functional.silu(x.double() @ gate.double().t()) * (x.double() @ up.double().t())
            out = torch.full((n, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
            native.gemm_tc5(x, interleave_rows(gate, up, 16), out, native.TC5_SILU_MUL, status, ksplit=min(ksplit, 8))
            torch.testing.assert_close(out.double(), expected, atol=1e-2, rtol=1e-2, msg=lambda m: f"{what}: {m}")
        assert int(status.item()) == 0, what


@pytest.mark.parametrize("seed,head_sizes", [(7, (16, 32, 48, 64, 128)), (8, (80, 96, 112, 192, 256))])
def test_attention_kernels_at_random_sizes(native, seed, head_sizes) -> None:
    """1 to 9 requests of 1 to 3,000 keys, the last 1 to all of them new (whole prompts,
    portions, a few tokens, single tokens side by side), 1 to 16 query heads per key/value
    head, pages of 4 to 128, windows from 1 key upwards, 1 to 32 splits of the decode kernel
    or its evenly spread form, splits combined in the kernel or by a second one."""
    rng = random.Random(seed)
    for trial in range(30):
        d = rng.choice(head_sizes)
        groups = rng.choice([1, 2, 3, 4, 5, 8, 16])
        nkv = rng.choice([1, 2, 3, 8])
        page = rng.choice([4, 8, 16, 32, 64, 128])
        window = rng.choice([None, None, 1, 17, 70, 200, 1000])
        lengths, new = [], []
        for _ in range(rng.randint(1, 9)):
            n = rng.choice([1, 2, rng.randint(1, 70), rng.randint(1, 700), rng.randint(1, 3000)])
            kind = rng.random()
            new.append(1 if kind < 0.4 else (min(n, rng.randint(1, 5)) if kind < 0.6 else (n if kind < 0.8 else rng.randint(1, n))))
            lengths.append(n)
        splits = rng.choice([0, 1, 2, 3, 5, 8, 13, 16, 32])
        if splits == 0 and not (d % 64 == 0 and page <= 64 and 64 % page == 0):
            splits = 1                       # the evenly spread form takes heads of 64 and 128 and pages up to 64
        try:
            attention_cases.run_case(native, nkv * groups, nkv, d, page, window, lengths, new, splits,
                                     sharp=rng.random() < 0.5 and lengths[0] > 4, merge_in_kernel=rng.random() < 0.8)
        except AssertionError as error:
            raise AssertionError(f"trial {trial}: {nkv * groups} heads over {nkv}, head size {d}, pages of {page}, window "
                                 f"{window}, keys {lengths}, new {new}, {splits} splits: {error}") from error
