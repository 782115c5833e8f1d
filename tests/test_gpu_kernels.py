"""Each CUDA kernel alone against a plain PyTorch 32/64-bit reference of the same
operation, at sizes other than the tiny models' (odd widths, many heads, long contexts)."""

from __future__ import annotations

import math

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def native():
    from forge_engine_b200.ops import native as module

    module.require_cuda()
    module.lib()
    return module


def status_word():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def tol(dtype):
    return dict(atol=2e-6, rtol=2e-6) if dtype == torch.float32 else dict(atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding(native, dtype) -> None:
    g = torch.Generator().manual_seed(0)
    table = torch.randn((331, 203), generator=g).to(dtype).to(DEV)
    ids = torch.randint(0, 331, (57,), generator=g).to(torch.int32).to(DEV)
    out = torch.empty((57, 203), dtype=torch.float32, device=DEV)
    status = status_word()
    native.embedding(ids, table, out, status)
    assert torch.equal(out, table[ids.long()].float())
    assert int(status.item()) == 0
    ids[5] = 331
    native.embedding(ids, table, out, status)
    assert int(status.item()) == 1 and float(out[5].abs().sum()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [37, 300])
@pytest.mark.parametrize("size", [72, 203, 2560, 5000, 12292, 16384, 16388])
def test_add_rmsnorm(native, dtype, size, rows) -> None:
    g = torch.Generator().manual_seed(size)
    residual = torch.randn((rows, size), generator=g).to(DEV)
    update = torch.randn((rows, size), generator=g).to(dtype).to(DEV)
    weight = (1 + 0.1 * torch.randn(size, generator=g)).to(DEV)
    eps = 3e-6
    summed = residual.double() + update.double()
    ref = summed * torch.rsqrt(summed.square().mean(-1, keepdim=True) + eps) * weight.double()
    out = torch.empty((rows, size), dtype=dtype, device=DEV)
    res = residual.clone()
    native.add_rmsnorm(res, update, weight, out, eps)
    torch.testing.assert_close(res.double(), summed, atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(out.double(), ref, **tol(dtype))
    # no update: the plain RMSNorm (compare with the plain implementation's function)
    out2 = torch.empty_like(out)
    res2 = residual.clone()
    native.add_rmsnorm(res2, None, weight, out2, eps)
    assert torch.equal(res2, residual)
    torch.testing.assert_close(out2.float().cpu(), plain.rms_norm(residual.cpu(), weight.cpu(), eps), **tol(dtype))
    # row map: only some rows, residual untouched
    rows_wanted = torch.tensor([36, 0, 17], dtype=torch.int32, device=DEV)
    out3 = torch.empty((3, size), dtype=dtype, device=DEV)
    res3 = residual.clone()
    native.add_rmsnorm(res3, update, weight, out3, eps, rows_wanted, write_residual=False)
    assert torch.equal(res3, residual)
    torch.testing.assert_close(out3.double(), ref[rows_wanted.long()], **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inter", [200, 203, 9728])
def test_silu_mul(native, dtype, inter) -> None:
    g = torch.Generator().manual_seed(inter)
    x = torch.randn((19, 2 * inter), generator=g).mul(3).to(dtype).to(DEV)
    out = torch.empty((19, inter), dtype=dtype, device=DEV)
    native.silu_mul(x, out)
    xd = x.double()
    ref = torch.nn.functional.silu(xd[:, :inter]) * xd[:, inter:]
    torch.testing.assert_close(out.double(), ref, **tol(dtype))
    for block in (8, 16) if inter % 16 == 0 else ():
        # rows that alternate `block` gate and `block` up features
        blocks = xd.view(19, inter // block, 2, block)
        ref = (torch.nn.functional.silu(blocks[:, :, 0]) * blocks[:, :, 1]).reshape(19, inter)
        native.silu_mul(x, out, block)
        torch.testing.assert_close(out.double(), ref, **tol(dtype))


@pytest.mark.parametrize("xd,wd,yd", [
    (torch.float32, torch.float32, torch.float32),
    (torch.bfloat16, torch.float32, torch.bfloat16),
    (torch.bfloat16, torch.bfloat16, torch.float32),
    (torch.bfloat16, torch.bfloat16, torch.bfloat16),
])
@pytest.mark.parametrize("n,o,k", [(1, 331, 80), (7, 203, 131), (130, 65, 1000), (64, 64, 16)])
def test_gemm_simt(native, xd, wd, yd, n, o, k) -> None:
    g = torch.Generator().manual_seed(n * 1000 + o)
    x = torch.randn((n, k), generator=g).to(xd).to(DEV)
    w = torch.randn((o, k), generator=g).mul(0.1).to(wd).to(DEV)
    bias = torch.randn(o, generator=g).to(DEV)
    ref = x.double() @ w.double().t()
    y = torch.empty((n, o), dtype=yd, device=DEV)
    native.gemm_simt(x, w, y)
    bound = dict(atol=2e-5, rtol=1e-5) if yd == torch.float32 else dict(atol=3e-2, rtol=1e-2)
    torch.testing.assert_close(y.double(), ref, **bound)
    native.gemm_simt(x, w, y, bias)
    torch.testing.assert_close(y.double(), ref + bias.double(), **bound)
    if yd == torch.float32:
        base = torch.randn((n, o), generator=g).to(DEV)
        acc = base.clone()
        native.gemm_simt(x, w, acc, None, accumulate=True)
        torch.testing.assert_close(acc.double(), ref + base.double(), **bound)
    # a row's result does not depend on the other rows of the call
    if n > 1:
        alone = torch.empty((1, o), dtype=yd, device=DEV)
        native.gemm_simt(x[n - 1 : n].contiguous(), w, alone, bias)
        assert torch.equal(alone[0], y[n - 1])


def paged_layout(lengths, page_size, nkv, d, dtype, seed, spare_pages=5):
    """Random keys/values for several requests scattered over shuffled pages."""
    g = torch.Generator().manual_seed(seed)
    pages_per = [-(-n // page_size) for n in lengths]
    total = sum(pages_per) + spare_pages
    order = torch.randperm(total, generator=g).tolist()
    width = max(pages_per) + 1
    table = torch.full((len(lengths), width), -1, dtype=torch.int32)
    k_cache = torch.randn((total, nkv, page_size, d), generator=g).to(dtype)   # garbage everywhere
    v_cache = torch.randn((total, nkv, page_size, d), generator=g).to(dtype)
    keys, values = [], []
    cursor = 0
    for r, n in enumerate(lengths):
        k = torch.randn((n, nkv, d), generator=g).to(dtype)
        v = torch.randn((n, nkv, d), generator=g).to(dtype)
        keys.append(k), values.append(v)
        for p in range(pages_per[r]):
            page = order[cursor]
            cursor += 1
            table[r, p] = page
            lo, hi = p * page_size, min(n, (p + 1) * page_size)
            k_cache[page, :, : hi - lo] = k[lo:hi].transpose(0, 1)
            v_cache[page, :, : hi - lo] = v[lo:hi].transpose(0, 1)
    return k_cache.to(DEV), v_cache.to(DEV), table.to(DEV), keys, values


def plant_keys(k_cache, v_cache, table, keys, values, r, window, q_row):
    """Make request ``r``'s last query depend on single keys at the places where a kernel
    can go wrong: the oldest key it may see (the first of its window, or key 0), the key
    just before it (which a window must hide: it gets the largest score of all and a huge
    value), both sides of the edges of the first and the last 64-key tile, the middle, and
    its own key.  ``q_row`` ([nq * d] or longer, the query heads first) is overwritten with
    the direction all planted keys share, so each of them outweighs all random keys
    together and a missed, doubled or wrongly admitted key moves the result by far more
    than the tolerance.  Changes ``keys[r]``, ``values[r]`` and the cache pages alike."""
    n, nkv, d = keys[r].shape
    page = k_cache.shape[2]
    lo = max(0, n - window) if window else 0
    u = torch.ones(d)
    u[1::2] = -1.0
    places = {lo, n - 1, (lo + n) // 2}
    for edge in (lo + 63, lo + 64, n - 65, n - 64):
        if lo <= edge < n:
            places.add(edge)
    planted = [(pos, 2.0, None) for pos in sorted(places)]
    if lo > 0:
        planted.append((lo - 1, 3.0, 50.0))
    for pos, gain, value in planted:
        keys[r][pos] = (gain * u).to(keys[r].dtype)
        if value is not None:
            values[r][pos] = value
        at = int(table[r, pos // page])
        k_cache[at, :, pos % page] = keys[r][pos].to(k_cache.device)
        v_cache[at, :, pos % page] = values[r][pos].to(v_cache.device)
    heads = q_row.numel() // d
    q_row.view(heads, d)[:] = (1.5 * u).to(q_row.dtype)
    return len(planted)


def dense_attention(q, k, v, positions, scale, window):
    """q [T, nq, d] at ``positions``; k, v [S, nkv, d]; 64-bit softmax attention."""
    nq, nkv = q.shape[1], k.shape[1]
    k = k.double().repeat_interleave(nq // nkv, dim=1)
    v = v.double().repeat_interleave(nq // nkv, dim=1)
    scores = torch.einsum("thd,shd->hts", q.double(), k) * scale
    key_pos = torch.arange(k.shape[0])
    allowed = key_pos[None, :] <= positions[:, None]
    if window:
        allowed = allowed & (positions[:, None] - key_pos[None, :] < window)
    scores = scores.masked_fill(~allowed[None], float("-inf"))
    return torch.einsum("hts,shd->thd", torch.softmax(scores, -1), v)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d,page,window", [
    (8, 2, 64, 16, None), (6, 3, 48, 8, None), (32, 8, 128, 16, None), (5, 1, 16, 4, 37), (4, 4, 256, 32, 100),
])
def test_attention_simt(native, dtype, nq, nkv, d, page, window) -> None:
    lengths = [300, 1, 129, 64]
    k_cache, v_cache, table, keys, values = paged_layout(lengths, page, nkv, d, dtype, seed=d + nq)
    g = torch.Generator().manual_seed(1)
    # queries: the last few positions of request 0, the only one of 1, a middle run of 2, all of 3's tail
    plan = [(0, list(range(290, 300))), (1, [0]), (2, [15, 16, 17, 128]), (3, [31, 32, 63])]
    token_entry, positions = [], []
    for entry, pos in plan:
        token_entry += [entry] * len(pos)
        positions += pos
    n = len(positions)
    q = torch.randn((n, nq, d), generator=g).to(dtype)
    # one far key that matters: align a query of request 0 with key 3 so that its score stands out
    q[0, 0] = (keys[0][3, 0].float() * 4).to(dtype)
    scale = d ** -0.5
    out = torch.empty((n, nq * d), dtype=dtype, device=DEV)
    status = status_word()
    native.attention_simt(
        q.reshape(n, nq * d).to(DEV), nq * d, k_cache, v_cache, table,
        torch.tensor(positions, dtype=torch.int32, device=DEV),
        torch.tensor(token_entry, dtype=torch.int32, device=DEV), window, scale, out, nq, status,
    )
    assert int(status.item()) == 0
    row = 0
    for entry, pos in plan:
        ref = dense_attention(q[row : row + len(pos)], keys[entry], values[entry], torch.tensor(pos), scale, window)
        mine = out[row : row + len(pos)].view(len(pos), nq, d).double().cpu()
        torch.testing.assert_close(mine, ref, **(dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)))
        row += len(pos)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d,rot,norm", [(8, 2, 32, 32, True), (6, 3, 48, 48, True), (32, 8, 128, 128, True),
                                                (4, 1, 64, 32, True), (4, 2, 16, 16, False), (6, 2, 64, 64, True),
                                                (3, 1, 256, 256, True), (5, 1, 128, 128, False)])
def test_qk_rope_cache(native, dtype, nq, nkv, d, rot, norm) -> None:
    g = torch.Generator().manual_seed(d)
    page, theta, eps = 8, 12345.0, 2e-6
    lengths = [21, 9]
    starts = [13, 0]    # request 0 already holds 13 tokens
    table = torch.tensor([[4, 1, 6, -1], [0, 5, -1, -1]], dtype=torch.int32, device=DEV)
    positions = list(range(13, 21)) + list(range(0, 9))
    entry = [0] * 8 + [1] * 9
    n = len(positions)
    qkv = torch.randn((n, (nq + 2 * nkv) * d), generator=g).to(dtype)
    qw = (1 + 0.1 * torch.randn(d, generator=g))
    kw = (1 + 0.1 * torch.randn(d, generator=g))
    k_cache = torch.zeros((7, nkv, page, d), dtype=dtype, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    inv_freq = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    dev_qkv = qkv.clone().to(DEV)
    status = status_word()
    native.qk_rope_cache(
        dev_qkv, qw.to(DEV) if norm else None, kw.to(DEV) if norm else None, eps, inv_freq.to(DEV), rot,
        torch.tensor(positions, dtype=torch.int32, device=DEV), torch.tensor(entry, dtype=torch.int32, device=DEV),
        k_cache, v_cache, table, nq, True, status,
    )
    assert int(status.item()) == 0
    x = qkv.float()
    q = x[:, : nq * d].view(n, nq, d)
    k = x[:, nq * d : (nq + nkv) * d].view(n, nkv, d)
    v = x[:, (nq + nkv) * d :].view(n, nkv, d)
    if norm:
        q, k = plain.rms_norm(q, qw, eps), plain.rms_norm(k, kw, eps)
    pos = torch.tensor(positions)
    cosine, sine = plain.rotary_tables(pos, rot, theta, torch.float32)

    def rotate(t):   # [n, heads, d], the first ``rot`` elements of each head
        head = t[..., :rot].transpose(0, 1)
        turned = plain.apply_rotary(head, cosine, sine).transpose(0, 1)
        return torch.cat((turned, t[..., rot:]), dim=-1)

    q_ref, k_ref = rotate(q), rotate(k)
    bound = dict(atol=3e-6, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=1e-2)
    torch.testing.assert_close(dev_qkv[:, : nq * d].float().cpu().view(n, nq, d), q_ref, **bound)
    for i, (e, p) in enumerate(zip(entry, positions)):
        page_id = int(table[e, p // page])
        torch.testing.assert_close(k_cache[page_id, :, p % page].float().cpu(), k_ref[i], **bound)
        assert torch.equal(v_cache[page_id, :, p % page].cpu(), v[i].to(dtype))
    # with the angles' cosines and sines taken beforehand: the same bits
    angles = torch.empty((n, rot // 2, 2), dtype=torch.float32, device=DEV)
    native.rope_table(torch.tensor(positions, dtype=torch.int32, device=DEV), inv_freq.to(DEV), angles)
    reference = torch.stack((torch.cos(pos[:, None].double() * inv_freq.double()), torch.sin(pos[:, None].double() * inv_freq.double())), -1)
    torch.testing.assert_close(angles.double().cpu(), reference, atol=2e-6, rtol=0)
    again, k2, v2 = qkv.clone().to(DEV), torch.zeros_like(k_cache), torch.zeros_like(v_cache)
    native.qk_rope_cache(
        again, qw.to(DEV) if norm else None, kw.to(DEV) if norm else None, eps, inv_freq.to(DEV), rot,
        torch.tensor(positions, dtype=torch.int32, device=DEV), torch.tensor(entry, dtype=torch.int32, device=DEV),
        k2, v2, table, nq, True, status, table=angles,
    )
    assert torch.equal(again, dev_qkv) and torch.equal(k2, k_cache) and torch.equal(v2, v_cache)
    # slots that no token of this step owns stay untouched (zero)
    assert float(k_cache[2].abs().sum()) == 0 and float(k_cache[3].abs().sum()) == 0
    assert float(k_cache[4, :, :5].abs().sum()) == 0    # positions 8..12 of request 0 live in page 1 (pages 4,1,6)
    # a position beyond the table is reported, not written
    bad_pos = torch.tensor([40], dtype=torch.int32, device=DEV)
    native.qk_rope_cache(dev_qkv[:1].contiguous(), None, None, eps, None, 0, bad_pos,
                         torch.tensor([0], dtype=torch.int32, device=DEV), k_cache, v_cache, table, nq, True, status)
    assert int(status.item()) & 4


@pytest.mark.parametrize("nq,nkv,d,norm,with_table,write", [(32, 8, 128, True, True, True), (6, 2, 64, True, False, True),
                                                            (3, 1, 256, True, True, True), (5, 1, 128, False, True, True),
                                                            (7, 3, 64, True, True, False)])
def test_qk_rope_cache_from_sums(native, nq, nkv, d, norm, with_table, write) -> None:
    """The form that reads 32-bit sums (where a projection's k-splits were added) and leaves
    zeros behind: queries as bfloat16 into the q columns of another buffer, k and v into
    their pages, against the plain norm and rotation of the same 32-bit numbers."""
    g = torch.Generator().manual_seed(d + nq)
    page, theta, eps = 8, 54321.0, 3e-6
    table = torch.tensor([[4, 1, 6, -1], [0, 5, -1, -1]], dtype=torch.int32, device=DEV)
    positions = list(range(13, 21)) + list(range(0, 9))
    entry = [0] * 8 + [1] * 9
    n = len(positions)
    width = (nq + 2 * nkv) * d
    x = torch.randn((n, width), generator=g)
    qw, kw = 1 + 0.1 * torch.randn(d, generator=g), 1 + 0.1 * torch.randn(d, generator=g)
    k_cache = torch.zeros((7, nkv, page, d), dtype=torch.bfloat16, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    inv_freq = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    dev_positions = torch.tensor(positions, dtype=torch.int32, device=DEV)
    angles = None
    if with_table:
        angles = torch.empty((n, d // 2, 2), dtype=torch.float32, device=DEV)
        native.rope_table(dev_positions, inv_freq.to(DEV), angles)
    sums = native.projection_sums(torch.device(DEV), n * width)
    assert float(sums.abs().max()) == 0          # zero when handed out, and after every use
    view = sums[: n * width].view(n, width)
    view.copy_(x)
    out = torch.full((n, width), 7.0, dtype=torch.bfloat16, device=DEV)
    status = status_word()
    native.qk_rope_cache_sums(view, out, qw.to(DEV) if norm else None, kw.to(DEV) if norm else None, eps, inv_freq.to(DEV),
                              dev_positions, torch.tensor(entry, dtype=torch.int32, device=DEV), k_cache, v_cache, table,
                              nq, write, status, table=angles)
    assert int(status.item()) == 0
    assert float(sums.abs().max()) == 0
    q = x[:, : nq * d].view(n, nq, d)
    k = x[:, nq * d : (nq + nkv) * d].view(n, nkv, d)
    v = x[:, (nq + nkv) * d :].view(n, nkv, d)
    if norm:
        q, k = plain.rms_norm(q, qw, eps), plain.rms_norm(k, kw, eps)
    cosine, sine = plain.rotary_tables(torch.tensor(positions), d, theta, torch.float32)
    rotate = lambda t: plain.apply_rotary(t.transpose(0, 1), cosine, sine).transpose(0, 1)   # noqa: E731
    bound = dict(atol=2e-2, rtol=1e-2)
    torch.testing.assert_close(out[:, : nq * d].float().cpu().view(n, nq, d), rotate(q), **bound)
    assert float((out[:, nq * d :].float() - 7.0).abs().max()) == 0      # the k and v columns are not written
    if not write:
        assert float(k_cache.abs().sum()) == 0 and float(v_cache.abs().sum()) == 0
        return
    k_ref = rotate(k)
    for i, (e, p) in enumerate(zip(entry, positions)):
        page_id = int(table[e, p // page])
        torch.testing.assert_close(k_cache[page_id, :, p % page].float().cpu(), k_ref[i], **bound)
        assert torch.equal(v_cache[page_id, :, p % page].cpu(), v[i].to(torch.bfloat16))
    assert float(k_cache[2].abs().sum()) == 0 and float(k_cache[3].abs().sum()) == 0
    # a position beyond the table is reported, nothing is written, and the sums are cleared all the same
    view[:1].fill_(1.0)
    native.qk_rope_cache_sums(view[:1], out[:1], None, None, eps, None, torch.tensor([40], dtype=torch.int32, device=DEV),
                              torch.tensor([0], dtype=torch.int32, device=DEV), k_cache, v_cache, table, nq, True, status)
    assert int(status.item()) & 4 and float(sums.abs().max()) == 0


def test_rope_angles_at_large_positions(native) -> None:
    """Angles are float(position) * inv_freq in 32-bit; cos and sin must stay accurate at
    positions in the hundred thousands (no fast-math range reduction)."""
    d, theta = 64, 1e6
    positions = [0, 1, 4095, 131071, 262143]
    n = len(positions)
    x = torch.zeros((n, 3 * d))
    x[:, :d] = 1.0
    x[:, d : 2 * d] = 1.0
    inv_freq = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    table = torch.zeros((1, 262144 // 16), dtype=torch.int32, device=DEV)
    k_cache = torch.zeros((1, 1, 16, d), device=DEV)
    v_cache = torch.zeros_like(k_cache)
    dev = x.clone().to(DEV)
    native.qk_rope_cache(dev, None, None, 1e-6, inv_freq.to(DEV), d, torch.tensor(positions, dtype=torch.int32, device=DEV),
                         torch.zeros(n, dtype=torch.int32, device=DEV), k_cache, v_cache, table, 1, False, status_word())
    angles = (torch.tensor(positions).float()[:, None] * inv_freq[None]).double()
    ref = torch.cat((torch.cos(angles) - torch.sin(angles), torch.cos(angles) + torch.sin(angles)), -1)
    torch.testing.assert_close(dev[:, :d].double().cpu(), ref, atol=2e-6, rtol=0)


# ---------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------

def twin_uniform(seed: int, counter: int) -> float:
    """Same hash as the kernel, written out again for the test."""
    mask = (1 << 64) - 1

    def mix(z):
        z = (z + 0x9E3779B97F4A7C15) & mask
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        return z ^ (z >> 31)

    return (mix(mix(seed & mask) ^ ((counter * 0xD1342543DE82EF95) & mask)) >> 40) / 16777216.0


def twin_draw(logits_row, temperature, top_k, top_p, min_p, seed, counter):
    """Draw from the plain implementation's filtered distribution with the kernel's uniform:
    first index, in index order, whose running probability sum exceeds u."""
    filtered = plain.filter_logits(logits_row[None], temperature, top_k, top_p, min_p)[0]
    weights = torch.exp(filtered.double())
    target = twin_uniform(seed, counter) * float(weights.sum())
    running = torch.cumsum(weights, 0)
    index = int(torch.searchsorted(running, torch.tensor(target, dtype=torch.float64), right=True))
    survivors = torch.nonzero(weights > 0).flatten()
    return min(index, int(survivors[-1])), running, target


def test_uniform_twin_matches_kernel_hash(native) -> None:
    from forge_engine_b200.sampling.rng import uniform

    for seed, counter in [(0, 0), (1, 2), (2**63 - 1, 17), (123456789, 2**40)]:
        host = native.lib().fe_uniform_host(seed, counter)
        assert host == pytest.approx(twin_uniform(seed, counter), abs=0)
        assert uniform(seed, counter) == twin_uniform(seed, counter)
        assert 0.0 <= host < 1.0


def test_greedy_is_argmax_with_lowest_index_on_ties(native) -> None:
    g = torch.Generator().manual_seed(3)
    logits = torch.randn((9, 151936), generator=g)
    logits[2, 500] = logits[2, 70000] = 9.0
    logits[3, :] = -1.0
    logits[4, 151935] = 20.0
    out = torch.empty(9, dtype=torch.int32, device=DEV)
    status = status_word()
    native.sample(logits.to(DEV), out, status)
    expected = logits.argmax(-1)
    expected[2], expected[3] = 500, 0
    assert out.cpu().tolist() == expected.tolist() and int(status.item()) == 0
    bad = logits.clone()
    bad[1, 7] = float("nan")
    native.sample(bad.to(DEV), out, status)
    assert int(status.item()) & 16


@pytest.mark.parametrize("temperature,top_k,top_p,min_p", [
    (0.8, None, 1.0, 0.0), (1.0, 5, 1.0, 0.0), (1.3, None, 0.7, 0.0), (0.7, None, 1.0, 0.1),
    (1.0, 40, 0.9, 0.02), (2.0, 1, 1.0, 0.0),
])
def test_sampling_matches_filtered_distribution(native, temperature, top_k, top_p, min_p) -> None:
    vocab, rows = 331, 400
    g = torch.Generator().manual_seed(11)
    base = torch.randn(vocab, generator=g) * 2.0
    logits = base[None].repeat(rows, 1).contiguous()
    seeds = torch.arange(rows, dtype=torch.int64) * 7919 + 5
    counters = torch.arange(rows, dtype=torch.int64) % 13
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    native.sample(
        logits.to(DEV), out, status_word(),
        temperature=torch.full((rows,), temperature, device=DEV),
        top_k=torch.full((rows,), top_k or 0, dtype=torch.int32, device=DEV),
        top_p=torch.full((rows,), top_p, device=DEV), min_p=torch.full((rows,), min_p, device=DEV),
        seeds=seeds.to(DEV), counters=counters.to(DEV),
    )
    got = out.cpu().tolist()
    filtered = plain.filter_logits(base[None], temperature, top_k, top_p, min_p)[0]
    survivors = set(torch.nonzero(torch.isfinite(filtered)).flatten().tolist())
    assert set(got) <= survivors
    agree = 0
    for r in range(rows):
        want, running, target = twin_draw(base, temperature, top_k, top_p, min_p, int(seeds[r]), int(counters[r]))
        if got[r] == want:
            agree += 1
        else:
            # only a target within rounding of a boundary of the running sum may differ
            gap = float((running - target).abs().min())
            assert gap < 1e-5 * float(running[-1]), (r, got[r], want, gap)
    assert agree >= rows - 2
    if top_k == 1:
        assert set(got) == {int(base.argmax())}


@pytest.mark.parametrize("temperature,top_k,top_p,min_p", [(0.9, None, 1.0, 0.0), (1.0, 30, 1.0, 0.0), (1.1, None, 0.8, 0.0),
                                                           (0.8, 50, 0.9, 0.01)])
def test_sampling_large_vocabulary_over_a_cluster(native, temperature, top_k, top_p, min_p) -> None:
    """A vocabulary large enough that a row is cut over the blocks of a cluster: same draws
    as the plain filter."""
    vocab, rows = 70001, 12
    g = torch.Generator().manual_seed(21)
    base = torch.randn(vocab, generator=g) * 2.5
    logits = base[None].repeat(rows, 1).contiguous()
    seeds = torch.arange(rows, dtype=torch.int64) * 104729 + 3
    counters = torch.arange(rows, dtype=torch.int64) * 5
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    status = status_word()
    native.sample(
        logits.to(DEV), out, status,
        temperature=torch.full((rows,), temperature, device=DEV),
        top_k=torch.full((rows,), top_k or 0, dtype=torch.int32, device=DEV),
        top_p=torch.full((rows,), top_p, device=DEV), min_p=torch.full((rows,), min_p, device=DEV),
        seeds=seeds.to(DEV), counters=counters.to(DEV),
    )
    assert int(status.item()) == 0
    got = out.cpu().tolist()
    filtered = plain.filter_logits(base[None], temperature, top_k, top_p, min_p)[0]
    survivors = set(torch.nonzero(torch.isfinite(filtered)).flatten().tolist())
    assert set(got) <= survivors
    for r in range(rows):
        want, running, target = twin_draw(base, temperature, top_k, top_p, min_p, int(seeds[r]), int(counters[r]))
        if got[r] != want:
            gap = float((running - target).abs().min())
            assert gap < 1e-5 * float(running[-1]), (r, got[r], want, gap)


def test_sampling_rows_are_independent(native) -> None:
    """Different parameters per row in one launch; greedy rows beside sampled ones."""
    vocab = 1000
    g = torch.Generator().manual_seed(5)
    logits = torch.randn((4, vocab), generator=g) * 3
    params = [(0.0, 0, 1.0, 0.0), (1.0, 10, 1.0, 0.0), (0.5, 0, 0.5, 0.0), (1.5, 0, 1.0, 0.3)]
    out = torch.empty(4, dtype=torch.int32, device=DEV)
    native.sample(
        logits.to(DEV), out, status_word(),
        temperature=torch.tensor([p[0] for p in params], device=DEV),
        top_k=torch.tensor([p[1] for p in params], dtype=torch.int32, device=DEV),
        top_p=torch.tensor([p[2] for p in params], device=DEV),
        min_p=torch.tensor([p[3] for p in params], device=DEV),
        seeds=torch.tensor([1, 2, 3, 4], dtype=torch.int64, device=DEV),
        counters=torch.tensor([0, 5, 9, 2], dtype=torch.int64, device=DEV),
    )
    got = out.cpu().tolist()
    assert got[0] == int(logits[0].argmax())
    for r in (1, 2, 3):
        t, k, p, m = params[r]
        want, _, _ = twin_draw(logits[r], t, k or None, p, m, r + 1, [0, 5, 9, 2][r])
        assert got[r] == want


# ---------------------------------------------------------------------------
# tensor-core products for few rows
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("n,o,k,ksplit", [(1, 256, 128, 1), (8, 331, 72, 1), (5, 384, 200, 2), (33, 640, 2560, 4),
                                            (64, 2560, 4096, 8), (100, 331, 72, 1), (300, 1000, 512, 2), (128, 2560, 4096, 8),
                                            (100, 640, 2560, 4), (70, 384, 9728, 3)])
def test_gemm_tc5(native, n, o, k, ksplit) -> None:
    g = torch.Generator().manual_seed(n + o)
    x = torch.randn((n, k), generator=g).bfloat16().to(DEV)
    w = (torch.randn((o, k), generator=g) * 0.1).bfloat16().to(DEV)
    bias = torch.randn(o, generator=g).to(DEV)
    ref = x.double() @ w.double().t()
    status = status_word()
    out = torch.full((n, o), float("nan"), dtype=torch.float32, device=DEV)
    native.gemm_tc5(x, w, out, native.TC5_STORE_F32, status, ksplit=ksplit)
    torch.testing.assert_close(out.double(), ref, atol=2e-4, rtol=1e-5)
    out16 = torch.empty((n, o), dtype=torch.bfloat16, device=DEV)
    native.gemm_tc5(x, w, out16, native.TC5_STORE_BF16, status, bias=bias, ksplit=ksplit)
    torch.testing.assert_close(out16.double(), ref + bias.double(), atol=3e-2, rtol=1e-2)
    base = torch.randn((n, o), generator=g).to(DEV)
    acc = base.clone()
    native.gemm_tc5(x, w, acc, native.TC5_ADD_F32, status, ksplit=ksplit)
    torch.testing.assert_close(acc.double(), ref + base.double(), atol=2e-4, rtol=1e-5)
    # a second launch finds the arrival counters zeroed again
    native.gemm_tc5(x, w, out, native.TC5_STORE_F32, status, ksplit=ksplit)
    torch.testing.assert_close(out.double(), ref, atol=2e-4, rtol=1e-5)
    assert int(status.item()) == 0


@pytest.mark.parametrize("n,nq,nkv,k,ksplit,norm,rotate", [(1, 2, 1, 128, 1, True, True), (17, 4, 2, 200, 2, True, True),
                                                          (8, 32, 8, 2560, 4, True, True), (64, 3, 3, 512, 8, False, True),
                                                          (33, 4, 1, 256, 3, True, False)])
def test_gemm_tc5_qkv_rope(native, n, nq, nkv, k, ksplit, norm, rotate) -> None:
    """The q/k/v projection with the per-head norms, the rotation and the page write in its
    epilogue, against the same steps in 64-bit from the same bfloat16 inputs."""
    d, page, theta, eps = 128, 8, 54321.0, 3e-6
    g = torch.Generator().manual_seed(n + k)
    x = torch.randn((n, k), generator=g).bfloat16()
    w = (torch.randn(((nq + 2 * nkv) * d, k), generator=g) * (k ** -0.5)).bfloat16()
    bias = torch.randn((nq + 2 * nkv) * d, generator=g) * 0.1
    qw, kw = 1 + 0.1 * torch.randn(d, generator=g), 1 + 0.1 * torch.randn(d, generator=g)
    inv_freq = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    # two requests: the first already holds 37 tokens; pages in scrambled order
    first = (n + 1) // 2
    positions = list(range(37, 37 + first)) + list(range(0, n - first))
    entry = [0] * first + [1] * (n - first)
    pages_each = -(-(37 + n) // page)
    order = torch.randperm(2 * pages_each, generator=g).to(torch.int32)
    table = order.view(2, pages_each).to(DEV)
    k_cache = torch.zeros((2 * pages_each, nkv, page, d), dtype=torch.bfloat16, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    qkv = torch.full((n, (nq + 2 * nkv) * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    status = status_word()
    cos_sin = None
    if rotate:
        cos_sin = torch.empty((n, d // 2, 2), dtype=torch.float32, device=DEV)
        native.rope_table(torch.tensor(positions, dtype=torch.int32, device=DEV), inv_freq.to(DEV), cos_sin)
    native.gemm_tc5_qkv_rope(
        x.to(DEV), w.to(DEV), bias.to(DEV), qkv, qw.to(DEV) if norm else None, kw.to(DEV) if norm else None, eps,
        cos_sin, torch.tensor(positions, dtype=torch.int32, device=DEV),
        torch.tensor(entry, dtype=torch.int32, device=DEV), k_cache, v_cache, table, nq, True, status, ksplit=ksplit)
    assert int(status.item()) == 0
    y = x.double() @ w.double().t() + bias.double()
    q = y[:, : nq * d].view(n, nq, d)
    kk = y[:, nq * d : (nq + nkv) * d].view(n, nkv, d)
    v = y[:, (nq + nkv) * d :].view(n, nkv, d)
    if norm:
        q = q * torch.rsqrt(q.square().mean(-1, keepdim=True) + eps) * qw.double()
        kk = kk * torch.rsqrt(kk.square().mean(-1, keepdim=True) + eps) * kw.double()
    if rotate:
        angles = torch.tensor(positions, dtype=torch.float64)[:, None] * inv_freq.double()[None, :]
        cosine, sine = torch.cat((angles, angles), -1).cos()[:, None, :], torch.cat((angles, angles), -1).sin()[:, None, :]
        turn = lambda t: t * cosine + torch.cat((-t[..., d // 2 :], t[..., : d // 2]), -1) * sine
        q, kk = turn(q), turn(kk)
    bound = dict(atol=2e-2, rtol=1e-2)
    torch.testing.assert_close(qkv[:, : nq * d].double().cpu().view(n, nq, d), q, **bound)
    for i, (e, p) in enumerate(zip(entry, positions)):
        page_id = int(table[e, p // page])
        torch.testing.assert_close(k_cache[page_id, :, p % page].double().cpu(), kk[i], **bound)
        torch.testing.assert_close(v_cache[page_id, :, p % page].double().cpu(), v[i], **bound)
    # nothing else was written: as many slots are non-zero as tokens were stored
    assert int((k_cache.abs().sum((1, 3)) > 0).sum()) == n
    # a row's result does not depend on the rows beside it
    if n > 1:
        alone = torch.empty((1, (nq + 2 * nkv) * d), dtype=torch.bfloat16, device=DEV)
        k2, v2 = torch.zeros_like(k_cache), torch.zeros_like(v_cache)
        native.gemm_tc5_qkv_rope(
            x[:1].contiguous().to(DEV), w.to(DEV), bias.to(DEV), alone, qw.to(DEV) if norm else None,
            kw.to(DEV) if norm else None, eps, cos_sin[:1].contiguous() if rotate else None,
            torch.tensor(positions[:1], dtype=torch.int32, device=DEV), torch.tensor(entry[:1], dtype=torch.int32, device=DEV),
            k2, v2, table, nq, True, status, ksplit=ksplit)
        assert torch.equal(alone[:, : nq * d], qkv[:1, : nq * d])
        page_id = int(table[0, positions[0] // page])
        assert torch.equal(k2[page_id, :, positions[0] % page], k_cache[page_id, :, positions[0] % page])
    assert int(status.item()) == 0


@pytest.mark.parametrize("n,inter,k,ksplit", [(3, 64, 96, 1), (24, 256, 256, 2), (64, 9728, 2560, 1), (128, 9728, 2560, 1),
                                              (90, 512, 640, 2)])
def test_gemm_tc5_silu_mul(native, n, inter, k, ksplit) -> None:
    from forge_engine_b200.parts.linear import interleave_rows

    g = torch.Generator().manual_seed(inter)
    x = torch.randn((n, k), generator=g).bfloat16().to(DEV)
    gate = (torch.randn((inter, k), generator=g) * 0.05).bfloat16().to(DEV)
    up = (torch.randn((inter, k), generator=g) * 0.05).bfloat16().to(DEV)
    w = interleave_rows(gate, up, 16)
    ref = torch.nn.functional.silu(x.double() @ gate.double().t()) * (x.double() @ up.double().t())
    out = torch.empty((n, inter), dtype=torch.bfloat16, device=DEV)
    status = status_word()
    native.gemm_tc5(x, w, out, native.TC5_SILU_MUL, status, ksplit=ksplit)
    torch.testing.assert_close(out.double(), ref, atol=2e-2, rtol=1e-2)
    assert int(status.item()) == 0


@pytest.mark.parametrize("n,hidden,heads,inter", [(1, 64, 64, 128), (8, 2560, 4096, 9728), (16, 2560, 4096, 9728),
                                                  (5, 200, 136, 304), (13, 1024, 768, 19200), (3, 2048, 2048, 6144),
                                                  (2, 72, 96, 48)])
def test_decode_chain(native, n, hidden, heads, inter) -> None:
    """Output projection (+= residual), RMS norm + gate/up with SiLU*mul, down projection
    (+= residual) as one persistent kernel, against the same steps in 64-bit from the same
    bfloat16 inputs: sizes with fewer tiles than blocks, with more (whole tiles and shares of
    the left-over ones), widths that are no multiple of a tile, and two launches in a row (the
    second finds counters and staging tiles zeroed again)."""
    from forge_engine_b200.parts.linear import interleave_rows

    eps = 2e-6
    g = torch.Generator().manual_seed(n + hidden)
    x = torch.randn((n, heads), generator=g).bfloat16()
    w_o = (torch.randn((hidden, heads), generator=g) * heads ** -0.5).bfloat16()
    w_gate = (torch.randn((inter, hidden), generator=g) * hidden ** -0.5).bfloat16()
    w_up = (torch.randn((inter, hidden), generator=g) * hidden ** -0.5).bfloat16()
    w_down = (torch.randn((hidden, inter), generator=g) * inter ** -0.5).bfloat16()
    norm_w = 1 + 0.1 * torch.randn(hidden, generator=g)
    h0 = torch.randn((n, hidden), generator=g)
    shapes = [(hidden, heads, native.CHAIN_SRC_ACTIVATIONS, native.CHAIN_ADD),
              (2 * inter, hidden, native.CHAIN_SRC_NORM, native.CHAIN_SILU_MUL),
              (hidden, inter, native.CHAIN_SRC_ACTIVATIONS, native.CHAIN_ADD)]
    assert native.decode_chain_takes(shapes, n)
    h1 = h0.double() + x.double() @ w_o.double().t()
    normed = (h1 * torch.rsqrt(h1.square().mean(-1, keepdim=True) + eps) * norm_w.double()).bfloat16().double()
    gate, up = normed @ w_gate.double().t(), normed @ w_up.double().t()
    act_ref = (torch.nn.functional.silu(gate) * up)
    h2 = h1 + act_ref.bfloat16().double() @ w_down.double().t()
    w_gu = interleave_rows(w_gate, w_up, 16).to(DEV)
    status = status_word()
    for _ in range(2):
        h = h0.clone().to(DEV)
        act = torch.full((n, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
        native.decode_chain(
            [dict(w=w_o.to(DEV), x=x.to(DEV), out=h, src=native.CHAIN_SRC_ACTIVATIONS, epi=native.CHAIN_ADD),
             dict(w=w_gu, x=h, norm_w=norm_w.to(DEV), eps=eps, out=act, src=native.CHAIN_SRC_NORM, epi=native.CHAIN_SILU_MUL),
             dict(w=w_down.to(DEV), x=act, out=h, src=native.CHAIN_SRC_ACTIVATIONS, epi=native.CHAIN_ADD)],
            n, status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        torch.testing.assert_close(act.double().cpu(), act_ref, atol=2e-2, rtol=1e-2)
        # the residual: 32-bit sums of bfloat16 products; the bfloat16 rounding of the operands in
        # between (norm output, activation) may fall the other way than in the 64-bit restatement
        torch.testing.assert_close(h.double().cpu(), h2, atol=2e-2, rtol=1e-2)
    assert native.damaged_canaries() == []
    # what it does not take: more than 16 tokens, a norm wider than its operand buffer
    assert not native.decode_chain_takes(shapes, 17)
    assert not native.decode_chain_takes([(256, 4096, native.CHAIN_SRC_NORM, native.CHAIN_ADD)], 4)
