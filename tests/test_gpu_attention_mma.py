"""The tensor-core attention kernels alone (bfloat16): prefill tiles, split decode and the
merge, against a 64-bit dense reference on the same rounded inputs."""

from __future__ import annotations

import pytest
import torch

from test_gpu_kernels import DEV, dense_attention, paged_layout, plant_keys, status_word

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def native():
    from forge_engine_b200.ops import native as module

    module.require_cuda()
    module.lib()
    return module


def run_case(native, nq, nkv, d, page, window, lengths, new_counts, splits, sharp=False, merge_in_kernel=True,
             plant=True):
    """Request r holds lengths[r] keys after the step, the last new_counts[r] of them new.
    ``plant``: the last query of every entry that takes the decode kernel is aimed at single
    keys on the edges of its window and of its tiles (see ``plant_keys``)."""
    dtype = torch.bfloat16
    k_cache, v_cache, table, keys, values = paged_layout(lengths, page, nkv, d, dtype, seed=d + nq + page)
    g = torch.Generator().manual_seed(2)
    cu, starts = [0], []
    for n, c in zip(lengths, new_counts):
        cu.append(cu[-1] + c)
        starts.append(n - c)
    total = cu[-1]
    stride = (nq + 2 * nkv) * d          # q sits at the front of a fused qkv row, like in the engine
    qkv = torch.randn((total, stride), generator=g).to(dtype)
    if sharp:                            # one far key dominates one query row
        qkv[0, :d] = (keys[0][3, 0].float() * 4).to(dtype)
    groups = nq // nkv
    rows = [c * groups for c in new_counts]
    if plant:
        for r, (n, c) in enumerate(zip(lengths, new_counts)):
            if c * groups <= 16 and n >= 2:
                plant_keys(k_cache, v_cache, table, keys, values, r, window, qkv[cu[r + 1] - 1, : nq * d])
    out = torch.full((total, nq * d), float("nan"), dtype=dtype, device=DEV)
    status = status_word()
    native.attention_mma(
        qkv.to(DEV), stride, k_cache, v_cache, table,
        torch.tensor(cu, dtype=torch.int32, device=DEV), torch.tensor(starts, dtype=torch.int32, device=DEV),
        len(lengths), max(new_counts), window, d ** -0.5, out, nq, status,
        run_prefill=any(r > 16 for r in rows), run_decode=any(r <= 16 for r in rows), num_splits=splits,
        merge_in_kernel=merge_in_kernel,
    )
    assert int(status.item()) == 0
    for r, (n, c) in enumerate(zip(lengths, new_counts)):
        q = qkv[cu[r] : cu[r + 1], : nq * d].view(c, nq, d)
        positions = torch.arange(n - c, n)
        ref = dense_attention(q, keys[r], values[r], positions, d ** -0.5, window)
        mine = out[cu[r] : cu[r + 1]].view(c, nq, d).double().cpu()
        assert torch.isfinite(mine).all()
        torch.testing.assert_close(mine, ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("nq,nkv,d,page", [(32, 8, 128, 16), (8, 2, 64, 16), (6, 3, 48, 8), (4, 2, 16, 4),
                                           (5, 1, 32, 16), (16, 1, 256, 32), (12, 4, 80, 16), (4, 2, 192, 16)])
@pytest.mark.parametrize("window", [None, 70])
def test_prefill_and_decode_mixed(native, nq, nkv, d, page, window) -> None:
    # whole prompts, a portion that starts mid-page, single decoded tokens, a 2-token portion
    lengths = [300, 200, 129, 1, 64, 450, 33]
    new_counts = [300, 73, 1, 1, 2, 1, 33]
    run_case(native, nq, nkv, d, page, window, lengths, new_counts, splits=3, sharp=True)


@pytest.mark.parametrize("nq,nkv,d,page", [(8, 8, 64, 8), (16, 8, 128, 32), (16, 2, 128, 64), (16, 1, 64, 128),
                                           (8, 2, 128, 4), (6, 3, 128, 16)])
@pytest.mark.parametrize("window", [None, 200])
def test_prefill_tensor_memory_kernel_shapes(native, nq, nkv, d, page, window) -> None:
    """The tcgen05 prefill kernel at 1, 2, 4, 8 and 16 heads per kv head, page sizes from 4
    to 128, prompts that end inside a query tile, inside a key tile and on their edges, a
    portion that starts in the middle of a page, and a window that ends inside a tile."""
    lengths = [700, 513, 384, 128, 257, 31]
    new_counts = [700, 130, 384, 128, 64, 31]
    run_case(native, nq, nkv, d, page, window, lengths, new_counts, splits=2, sharp=True)


def test_prefill_portion_deep_in_a_long_context(native) -> None:
    """A 1,000-token portion that starts 5,000 tokens into its request (47 key tiles, the
    rings of key and value stages wrap many times), beside a whole 3,000-token prompt."""
    run_case(native, 8, 2, 128, 16, None, [6000, 3000], [1000, 3000], splits=1, sharp=True)
    run_case(native, 8, 2, 128, 16, 1500, [6000, 3000], [1000, 3000], splits=1)


@pytest.mark.parametrize("splits", [1, 2, 5, 8, 16, 32])
def test_split_decode_long_contexts(native, splits) -> None:
    lengths = [2048, 1, 777, 64, 65, 4000]
    run_case(native, 32, 8, 128, 16, None, lengths, [1] * 6, splits)
    run_case(native, 32, 8, 128, 16, 500, lengths, [1] * 6, splits)
    run_case(native, 32, 8, 128, 16, 70, lengths, [1] * 6, splits)
    # the splits combined by a second kernel instead of by the block that arrives last
    run_case(native, 32, 8, 128, 16, None, lengths, [1] * 6, splits, merge_in_kernel=False)


@pytest.mark.parametrize("nq,nkv,d,page", [(32, 8, 128, 16), (8, 2, 64, 64), (16, 1, 128, 4), (6, 3, 64, 8), (16, 1, 256, 32),
                                           (4, 2, 192, 16)])
@pytest.mark.parametrize("window", [None, 500])
def test_balanced_decode(native, nq, nkv, d, page, window) -> None:
    """splits = 0: the key tiles of all decode entries spread evenly over the GPU's blocks.
    Requests far longer than a block's share (cut into many pieces), shorter than it (several
    pairs in one block), of one key, of a tile's exact length; prompt portions beside them."""
    run_case(native, nq, nkv, d, page, window, [20000, 1, 777, 64, 65, 4000, 128, 9000], [1] * 8, 0)
    run_case(native, nq, nkv, d, page, window, [3], [1], 0)
    run_case(native, nq, nkv, d, page, window, [300, 5000, 200, 64, 2], [300, 1, 40, 1, 2], 0)
    run_case(native, nq, nkv, d, page, window, [700] * 40 + [701, 1, 12000], [1] * 43, 0, sharp=True)


def test_rows_do_not_depend_on_the_batch(native) -> None:
    """The prefill kernel gives the same bits for a request alone and beside others."""
    dtype = torch.bfloat16
    nq, nkv, d, page = 8, 2, 64, 16
    lengths, news = [200, 150, 90], [200, 150, 90]
    k_cache, v_cache, table, keys, values = paged_layout(lengths, page, nkv, d, dtype, seed=3)
    g = torch.Generator().manual_seed(4)
    q = torch.randn((sum(news), nq * d), generator=g).to(dtype).to(DEV)

    def run(which):
        cu = [0]
        for r in which:
            cu.append(cu[-1] + news[r])
        rows = torch.cat([q[sum(news[:r]) : sum(news[: r + 1])] for r in which]).contiguous()
        out = torch.empty_like(rows)
        native.attention_mma(rows, nq * d, k_cache, v_cache, table[list(which)].contiguous(),
                             torch.tensor(cu, dtype=torch.int32, device=DEV),
                             torch.zeros(len(which), dtype=torch.int32, device=DEV), len(which),
                             max(news[r] for r in which), None, d ** -0.5, out, nq, status_word(), True, False, 1)
        return out

    together = run((0, 1, 2))
    alone = run((1,))
    assert torch.equal(together[200:350], alone)
