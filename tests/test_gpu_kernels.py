"""Each CUDA kernel alone against a plain float32 statement of the same operation,
at sizes other than the engine's tiny models use."""

import pytest
import torch

import plain_model
from dryft_flash_infer_b200.cache import LayerCache

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 1.6e-2) * scale


def rounded(x, dtype):
    return x.to(dtype).float()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows, dim", [(1, 8), (7, 100), (33, 2560), (5, 3001), (70, 2560), (64, 40), (65, 8192), (66, 4100),
                                       (67, 1032), (130, 4096), (259, 264), (2049, 1536)])
def test_rms_norm_and_add(dtype, rows, dim):
    from dryft_flash_infer_b200.ops import kernels

    g = torch.Generator().manual_seed(rows * dim)
    x = rounded(torch.randn(rows, dim, generator=g) * 3, dtype)
    d = rounded(torch.randn(rows, dim, generator=g), dtype)
    w = 1 + 0.2 * torch.randn(dim, generator=g)
    eps = 1e-5
    got = kernels.rms_norm(x.to(dtype).cuda(), w.cuda(), eps)
    assert torch.allclose(got.float().cpu(), plain_model.rms_norm(x, w, eps), atol=tol(dtype, 4), rtol=tol(dtype))
    res = x.to(dtype).cuda()
    got = kernels.add_rms_norm(res, d.to(dtype).cuda(), w.cuda(), eps)
    summed = rounded(x + d, dtype)
    assert torch.equal(res.float().cpu(), summed)                       # the residual is the rounded float32 sum
    assert torch.allclose(got.float().cpu(), plain_model.rms_norm(summed, w, eps), atol=tol(dtype, 4), rtol=tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows, inter", [(3, 200), (1, 9728), (9, 37)])
def test_swiglu(dtype, rows, inter):
    from dryft_flash_infer_b200.ops import kernels

    g = torch.Generator().manual_seed(inter)
    gu = rounded(torch.randn(rows, 2 * inter, generator=g) * 2, dtype)
    want = gu[:, :inter] / (1 + torch.exp(-gu[:, :inter])) * gu[:, inter:]
    got = kernels.swiglu(gu.to(dtype).cuda())
    assert torch.allclose(got.float().cpu(), want, atol=tol(dtype, 2), rtol=tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_gather(dtype):
    from dryft_flash_infer_b200.ops import kernels

    table = torch.randn(321, 100).to(dtype)
    ids = torch.tensor([0, 320, 17, 17, 5], dtype=torch.int32)
    got = kernels.embedding(table.cuda(), ids.cuda())
    assert torch.equal(got.cpu(), table[ids.long()])
    rows = torch.tensor([4, 0, 2], dtype=torch.int32)
    assert torch.equal(kernels.gather_rows(got, rows.cuda()).cpu(), table[ids.long()][rows.long()])
    odd = torch.randn(9, 33).to(dtype)                                  # a width with no 16-byte rows
    assert torch.equal(kernels.gather_rows(odd.cuda(), rows.cuda()).cpu(), odd[rows.long()])


def paged_cache(n_seqs, lengths, n_kv, dim, dtype, ring_tokens=0, seed=0, page_size=64):
    """A cache with pages handed out in a scrambled order, NaN everywhere nothing was written."""
    width = max(-(-(ring_tokens or n) // page_size) for n in lengths)
    n_pages = 1 + n_seqs * width
    g = torch.Generator().manual_seed(seed)
    order = (1 + torch.randperm(n_pages - 1, generator=g)).tolist()
    table = torch.zeros(n_seqs, width, dtype=torch.int32)
    for s in range(n_seqs):
        need = -(-(ring_tokens or lengths[s]) // page_size)
        table[s, :need] = torch.tensor([order.pop() for _ in range(need)], dtype=torch.int32)
    k = torch.full((n_pages, n_kv, page_size, dim), float("nan"), dtype=dtype)
    v = torch.full((n_pages, n_kv, page_size, dim), float("nan"), dtype=dtype)
    return LayerCache(k.cuda(), v.cuda(), table.cuda(), page_size, ring_tokens, True), table


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q, n_kv, dim", [(6, 3, 48), (4, 4, 16), (16, 2, 128), (5, 1, 256), (3, 1, 20)])
@pytest.mark.parametrize("lengths, starts", [([70, 3, 130], [60, 0, 127]), ([170, 3, 130], [60, 0, 127]), ([171, 3, 130], [60, 0, 127])])
def test_qk_norm_rope_write(dtype, n_q, n_kv, dim, lengths, starts):
    """Few rows take the kernel with a warp per head, many rows the one with half a warp per head and
    four rows per thread (116 rows fill its threads, 117 leave three of the last four without a row)."""
    from dryft_flash_infer_b200.ops import kernels
    from dryft_flash_infer_b200.parts.rotary import RotaryEmbedding

    # the new rows cross page borders
    new = [l - s for l, s in zip(lengths, starts)]
    rows = sum(new)
    g = torch.Generator().manual_seed(dim)
    qkv = rounded(torch.randn(rows, (n_q + 2 * n_kv) * dim, generator=g), dtype)
    qw, kw = 1 + 0.3 * torch.randn(dim, generator=g), 1 + 0.3 * torch.randn(dim, generator=g)
    eps, theta = 1e-5, 12345.0
    row_seq = torch.cat([torch.full((n,), i) for i, n in enumerate(new)]).int()
    row_pos = torch.cat([torch.arange(s, l) for s, l in zip(starts, lengths)]).int()
    cache, table = paged_cache(3, lengths, n_kv, dim, dtype, seed=dim)
    rotary = RotaryEmbedding(0, dim, theta)
    rotary.prepare(256, "cuda")
    dev = qkv.to(dtype).cuda()
    q = kernels.qk_norm_rope_write(dev, n_q, n_kv, dim, qw.cuda(), kw.cuda(), eps, rotary.cos, rotary.sin,
                                   row_pos.cuda(), row_seq.cuda(), cache)
    x = qkv.view(rows, n_q + 2 * n_kv, dim)
    angles = plain_model.rope_angles(row_pos, dim, theta)
    want_q = plain_model.apply_rope(plain_model.head_norm(x[:, :n_q], qw, eps), angles)
    want_k = plain_model.apply_rope(plain_model.head_norm(x[:, n_q:n_q + n_kv], kw, eps), angles)
    want_v = x[:, n_q + n_kv:]
    t = tol(dtype, 4)
    assert torch.allclose(q.float().cpu().view(rows, n_q, dim), want_q, atol=t, rtol=tol(dtype))
    k_cache, v_cache = cache.k.float().cpu(), cache.v.float().cpu()
    written = torch.zeros(k_cache.shape[0], 64, dtype=torch.bool)
    for r in range(rows):
        page = int(table[row_seq[r], row_pos[r] // 64])
        assert torch.allclose(k_cache[page, :, row_pos[r] % 64], want_k[r], atol=t, rtol=tol(dtype))
        assert torch.equal(v_cache[page, :, row_pos[r] % 64], want_v[r])
        written[page, row_pos[r] % 64] = True
    assert torch.isnan(k_cache.transpose(1, 2)[~written]).all() and torch.isnan(v_cache.transpose(1, 2)[~written]).all()   # nothing else was touched
    # without weights and tables the heads pass through unchanged, and writes=False leaves the cache alone
    cache2, _ = paged_cache(3, lengths, n_kv, dim, dtype, seed=dim)
    cache2.writes = False
    dev = qkv.to(dtype).cuda()
    q = kernels.qk_norm_rope_write(dev, n_q, n_kv, dim, None, None, eps, None, None, row_pos.cuda(), row_seq.cuda(), cache2)
    assert torch.equal(q.float().cpu(), qkv[:, :n_q * dim]) and torch.isnan(cache2.k).all()


def plain_attention_rows(q, keys, values, positions, starts, scale, window):
    """q [rows, n_q, D] of one sequence at ``positions``; keys/values [len, n_kv, D]."""
    n_q, n_kv = q.shape[1], keys.shape[1]
    out = torch.empty_like(q)
    for r, pos in enumerate(positions):
        first = max(0, pos - window + 1) if window else 0
        for h in range(n_q):
            s = (keys[first:pos + 1, h // (n_q // n_kv)] @ q[r, h]) * scale
            out[r, h] = torch.softmax(s, 0) @ values[first:pos + 1, h // (n_q // n_kv)]
    return out


def attention_case(dtype, n_q, n_kv, dim, lengths, new, window=0, ring_tokens=0, seed=0, sharp=None):
    g = torch.Generator().manual_seed(seed)
    keys = [rounded(torch.randn(l, n_kv, dim, generator=g), dtype) for l in lengths]
    values = [rounded(torch.randn(l, n_kv, dim, generator=g), dtype) for l in lengths]
    qs = [rounded(torch.randn(n, n_q, dim, generator=g), dtype) for n in new]
    if sharp is not None:                          # the last query of sequence 0 looks for one far key
        qs[0][-1] = keys[0][sharp].repeat_interleave(n_q // n_kv, 0) * 4.0
    cache, table = paged_cache(len(lengths), lengths, n_kv, dim, dtype, ring_tokens, seed)
    k_host, v_host = cache.k.cpu(), cache.v.cpu()
    for s, l in enumerate(lengths):
        first = max(0, l - ring_tokens) if ring_tokens else 0
        for p in range(first, l):
            place = p % ring_tokens if ring_tokens else p
            page = int(table[s, place // 64])
            k_host[page, :, place % 64] = keys[s][p].to(dtype)
            v_host[page, :, place % 64] = values[s][p].to(dtype)
    cache.k.copy_(k_host)
    cache.v.copy_(v_host)
    row_seq = torch.cat([torch.full((n,), i) for i, n in enumerate(new)]).int().cuda()
    row_pos = torch.cat([torch.arange(l - n, l) for l, n in zip(lengths, new)]).int().cuda()
    q = torch.cat(qs).reshape(sum(new), n_q * dim).to(dtype).cuda()
    scale = dim ** -0.5
    want = torch.cat([plain_attention_rows(qs[s], keys[s], values[s], list(range(l - n, l)), None, scale, window)
                      for s, (l, n) in enumerate(zip(lengths, new))]).reshape(sum(new), n_q * dim)
    return q, cache, row_seq, row_pos, scale, want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q, n_kv, dim", [(6, 3, 48), (4, 4, 16), (8, 2, 128), (3, 1, 256)])
def test_attention_generic_prefill_and_decode(dtype, n_q, n_kv, dim):
    from dryft_flash_infer_b200.ops import kernels

    for lengths, new in (([70, 3, 130], [70, 3, 130]), ([70, 3, 130], [10, 3, 3]), ([257, 64, 1], [1, 1, 1])):
        q, cache, row_seq, row_pos, scale, want = attention_case(dtype, n_q, n_kv, dim, lengths, new, seed=dim)
        got = kernels.attention_generic(q, cache, row_seq, row_pos, n_q, n_kv, dim, scale)
        assert torch.isfinite(got).all()
        assert torch.allclose(got.float().cpu(), want, atol=tol(dtype, 2), rtol=tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_generic_far_key_and_window_edge(dtype):
    from dryft_flash_infer_b200.ops import kernels

    # one key at position 5 of 600 takes nearly all the weight
    q, cache, row_seq, row_pos, scale, want = attention_case(dtype, 8, 2, 64, [600, 90], [1, 1], seed=3, sharp=5)
    got = kernels.attention_generic(q, cache, row_seq, row_pos, 8, 2, 64, scale)
    assert torch.allclose(got.float().cpu(), want, atol=tol(dtype, 2), rtol=tol(dtype))
    # a window of 100 over a ring of 192 places: the key just outside must not count, the one just inside must
    for window, ring in ((100, 192), (64, 128), (1, 64)):
        q, cache, row_seq, row_pos, scale, want = attention_case(
            dtype, 4, 2, 32, [500, 131, 40], [3, 2, 40], window=window, ring_tokens=ring, seed=window)
        got = kernels.attention_generic(q, cache, row_seq, row_pos, 4, 2, 32, scale, window)
        assert torch.isfinite(got).all()
        assert torch.allclose(got.float().cpu(), want, atol=tol(dtype, 2), rtol=tol(dtype))


def test_argmax_and_sampling():
    from dryft_flash_infer_b200.ops import kernels

    g = torch.Generator().manual_seed(0)
    logits = torch.randn(5, 151936, generator=g)
    logits[1, 7] = logits[1, 90000] = 50.0                              # a tie: the lowest index wins
    logits[2, 151935] = 60.0
    got = kernels.argmax(logits.cuda()).cpu()
    assert got.tolist() == [int(logits[0].argmax()), 7, 151935, int(logits[3].argmax()), int(logits[4].argmax())]
    small = torch.randn(3, 37, generator=g)
    assert kernels.argmax(small.cuda()).cpu().tolist() == small.argmax(-1).tolist()
    wide = torch.randn(4, 1000, generator=g)[:, :700]                   # rows with a stride
    assert kernels.argmax(wide.cuda()[:, :700]).cpu().tolist() == wide.argmax(-1).tolist()
    # sampling: the token's CDF interval holds its uniform number
    for vocab, temperature in ((320, 0.8), (151936, 1.3), (5, 0.1), (4097, 0.7), (12289, 2.0)):
        logits = torch.randn(64, vocab, generator=g) * 3
        if vocab == 12289:
            logits[:, 4096:8192] = float("-inf")                     # a whole segment without weight
            logits[3, :12288] = float("-inf")                        # all the weight on the last element
        u = torch.rand(64, generator=g)
        u[0], u[1] = 0.0, 1.0 - 2 ** -24
        got = kernels.sample_temperature(logits.cuda(), u.cuda(), temperature).cpu()
        cdf = torch.cumsum(plain_model.temperature_probabilities(logits, temperature), -1)
        for r in range(64):
            t = int(got[r])
            low = float(cdf[r, t - 1]) if t else 0.0
            assert low - 2e-5 <= float(u[r]) <= float(cdf[r, t]) + 2e-5, (vocab, r, t)
    # a row's draw does not depend on the other rows
    alone = kernels.sample_temperature(logits[5:6].cuda(), u[5:6].cuda(), temperature).cpu()
    assert int(alone[0]) == int(got[5])
    assert int(got[3]) == 12288
    # more rows than one launch holds, rows with a stride, and the same call twice
    many = torch.randn(300, 1000, generator=g)[:, :777] * 2
    u = torch.rand(300, generator=g)
    got = kernels.sample_temperature(many.cuda()[:, :777], u.cuda(), 0.9).cpu()
    cdf = torch.cumsum(plain_model.temperature_probabilities(many, 0.9), -1)
    for r in range(300):
        t = int(got[r])
        assert (float(cdf[r, t - 1]) if t else 0.0) - 2e-5 <= float(u[r]) <= float(cdf[r, t]) + 2e-5, r
    assert torch.equal(kernels.sample_temperature(many.cuda()[:, :777], u.cuda(), 0.9).cpu(), got)


def test_sizes_a_kernel_does_not_take_are_refused():
    from dryft_flash_infer_b200.ops import KernelError, kernels

    cache, _ = paged_cache(1, [10], 1, 20, torch.bfloat16)
    q = torch.zeros(1, 20, dtype=torch.bfloat16).cuda()
    pos = torch.zeros(1, dtype=torch.int32).cuda()
    with pytest.raises(KernelError, match="head_dim"):
        kernels.attention_generic(q, cache, pos, pos, 1, 1, 20, 1.0)
    with pytest.raises(KernelError, match="CUDA device"):
        kernels.rms_norm(torch.zeros(2, 8), torch.ones(8), 1e-6)
    with pytest.raises(KernelError, match="dtype"):
        kernels.rms_norm(torch.zeros(2, 8, dtype=torch.float16).cuda(), torch.ones(8).cuda(), 1e-6)


def step_like(lengths, new):
    """The few per-step numbers the tensor-core attention reads from a StepContext."""
    from types import SimpleNamespace

    cu = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32)
    return SimpleNamespace(cu_rows=cu.cuda(), seq_start=torch.tensor([l - n for l, n in zip(lengths, new)],
                                                                   dtype=torch.int32).cuda(),
                           n_seqs=len(lengths), max_q_len=max(new), max_kv_len=max(lengths),
                           all_decode=all(n == 1 for n in new))


@pytest.mark.parametrize("n_q, n_kv, dim", [(6, 3, 48), (4, 4, 16), (8, 2, 128), (3, 1, 64), (16, 1, 32), (5, 5, 112)])
def test_attention_tensor_core_prefill(n_q, n_kv, dim):
    from dryft_flash_infer_b200.ops import kernels

    dtype = torch.bfloat16
    for lengths, new in (([70, 3, 130], [70, 3, 130]), ([70, 3, 200], [10, 3, 67]), ([257, 64, 1], [1, 1, 1]),
                         ([300], [300])):
        q, cache, row_seq, row_pos, scale, want = attention_case(dtype, n_q, n_kv, dim, lengths, new, seed=dim)
        got = kernels.attention_prefill(q, cache, step_like(lengths, new), n_q, n_kv, dim, scale)
        assert torch.isfinite(got).all()
        assert torch.allclose(got.float().cpu(), want, atol=tol(dtype, 2), rtol=tol(dtype)), (lengths, new)


@pytest.mark.parametrize("n_q, n_kv, dim", [(6, 3, 48), (4, 4, 16), (8, 2, 128), (32, 8, 128), (16, 1, 32), (3, 1, 64)])
def test_attention_tensor_core_decode_dealt_to_any_number_of_ctas(n_q, n_kv, dim):
    from dryft_flash_infer_b200.ops import kernels

    dtype = torch.bfloat16
    lengths, new = [257, 64, 1, 1000, 65], [1, 1, 1, 1, 1]
    q, cache, row_seq, row_pos, scale, want = attention_case(dtype, n_q, n_kv, dim, lengths, new, seed=dim, sharp=5)
    ctx = step_like(lengths, new)
    for ctas in (None, 1, 2, 3, 16, 40, 1000):         # however the pages are dealt out
        got = kernels.attention_decode(q, cache, ctx, n_q, n_kv, dim, scale, n_ctas=ctas)
        assert torch.isfinite(got).all()
        assert torch.allclose(got.float().cpu(), want, atol=tol(dtype, 2), rtol=tol(dtype)), ctas
        again = kernels.attention_decode(q, cache, ctx, n_q, n_kv, dim, scale, n_ctas=ctas)
        assert torch.equal(again, got)                 # the counters were left ready; the order of the merge is fixed


@pytest.mark.parametrize("n_q, n_kv, dim", [(8, 2, 128), (4, 4, 32)])
def test_attention_decode_with_more_groups_than_ctas_takes_whole_groups(n_q, n_kv, dim):
    """Many short sequences of one length: with more (sequence, head) groups than CTAs a CTA takes whole groups,
    one after another, and nothing is merged.  The CTA counts are chosen so that the busiest CTA holds two
    or three groups and some hold one fewer; a count that does not qualify (few CTAs, long runs) runs beside them."""
    from dryft_flash_infer_b200.ops import kernels

    dtype = torch.bfloat16
    n_seqs = 40
    lengths, new = [170] * n_seqs, [1] * n_seqs                  # three pages each, the last one a third full
    q, cache, row_seq, row_pos, scale, want = attention_case(dtype, n_q, n_kv, dim, lengths, new, seed=dim + 1, sharp=60)
    ctx = step_like(lengths, new)
    groups = n_seqs * n_kv
    for ctas in (groups, groups // 2, groups // 2 + 7, groups // 3 + 1, 5):
        got = kernels.attention_decode(q, cache, ctx, n_q, n_kv, dim, scale, n_ctas=ctas)
        assert torch.isfinite(got).all()
        assert torch.allclose(got.float().cpu(), want, atol=tol(dtype, 2), rtol=tol(dtype)), ctas
        assert torch.equal(kernels.attention_decode(q, cache, ctx, n_q, n_kv, dim, scale, n_ctas=ctas), got)


@pytest.mark.parametrize("n_q, n_kv, dim", [(4, 4, 16), (16, 1, 32), (3, 1, 64), (32, 8, 128)])
@pytest.mark.parametrize("qk_norm, rotary, window, ring", [(True, True, 0, 0), (False, False, 0, 0), (True, True, 100, 192)])
def test_attention_decode_that_prepares_the_tokens_itself(n_q, n_kv, dim, qk_norm, rotary, window, ring):
    """The decode kernel given the raw projection (norm, rotation and cache write inside) against
    qk_norm_rope_write followed by the same kernel: outputs, and the rows written into the cache."""
    from dryft_flash_infer_b200.ops import kernels
    from dryft_flash_infer_b200.parts.rotary import RotaryEmbedding

    dtype = torch.bfloat16
    # the new token is the last of its page (64, 128), the first of one (65, 257, 1), or in the middle
    lengths = [257, 64, 1, 1000, 65, 128, 300]
    new = [1] * len(lengths)
    _, cache, row_seq, row_pos, scale, _ = attention_case(dtype, n_q, n_kv, dim, lengths, new, window=window,
                                                          ring_tokens=ring, seed=dim + window)
    table = cache.block_table.cpu()
    for s_, l in enumerate(lengths):                    # nothing is known yet about the new token's place
        place = (l - 1) % ring if ring else l - 1
        cache.k[int(table[s_, place // 64]), :, place % 64] = float("nan")
        cache.v[int(table[s_, place // 64]), :, place % 64] = float("nan")
    g = torch.Generator().manual_seed(dim)
    qkv = torch.randn(len(lengths), (n_q + 2 * n_kv) * dim, generator=g).to(dtype).cuda()
    qw = (1 + 0.3 * torch.randn(dim, generator=g)).cuda() if qk_norm else None
    kw = (1 + 0.3 * torch.randn(dim, generator=g)).cuda() if qk_norm else None
    eps = 1e-5
    rot = RotaryEmbedding(0, dim, 4321.0)
    rot.prepare(1024, "cuda")
    cos, sin = (rot.cos, rot.sin) if rotary else (None, None)
    ctx = step_like(lengths, new)

    two = LayerCache(cache.k.clone(), cache.v.clone(), cache.block_table, 64, ring, True)
    q = kernels.qk_norm_rope_write(qkv.clone(), n_q, n_kv, dim, qw, kw, eps, cos, sin, row_pos, row_seq, two)
    want = kernels.attention_decode(q, two, ctx, n_q, n_kv, dim, scale, window)
    assert torch.isfinite(want).all()
    for ctas in (None, 1, 3, 40):
        one = LayerCache(cache.k.clone(), cache.v.clone(), cache.block_table, 64, ring, True)
        prep = kernels.TokenPrep(qkv, qw, kw, eps, cos, sin)
        assert kernels.decode_prepares_tokens(qkv, ctx, n_q, n_kv, dim)
        got = kernels.attention_decode(None, one, ctx, n_q, n_kv, dim, scale, window, n_ctas=ctas, prep=prep)
        assert torch.allclose(got.float(), want.float(), atol=tol(dtype, 2), rtol=tol(dtype)), ctas
        assert torch.allclose(one.k.float(), two.k.float(), atol=tol(dtype), rtol=tol(dtype), equal_nan=True)
        assert torch.equal(one.v.float().nan_to_num(7.0), two.v.float().nan_to_num(7.0))
    # a layer that only reads the cache (another one wrote the token): queries prepared, cache untouched
    read_only = LayerCache(two.k.clone(), two.v.clone(), cache.block_table, 64, ring, False)
    got = kernels.attention_decode(None, read_only, ctx, n_q, n_kv, dim, scale, window,
                                   prep=kernels.TokenPrep(qkv, qw, kw, eps, cos, sin))
    assert torch.allclose(got.float(), want.float(), atol=tol(dtype, 2), rtol=tol(dtype))
    assert torch.equal(read_only.k.float().nan_to_num(7.0), two.k.float().nan_to_num(7.0))


@pytest.mark.parametrize("n_q, n_kv, dim", [(4, 4, 16), (8, 2, 128), (16, 2, 64), (32, 2, 32)])
def test_attention_decode_with_equal_lengths_merges_in_clusters(n_q, n_kv, dim):
    """Sequences of one length: every group is cut into the same number of parts; with 16 CTAs that is
    four parts, which meet in a cluster (groups of up to 8 query heads) or through scratch memory (16)."""
    from dryft_flash_infer_b200.ops import kernels

    dtype = torch.bfloat16
    n_seqs = 4 // n_kv if n_kv <= 4 else 1
    lengths, new = [1270] * n_seqs, [1] * n_seqs                # 20 pages each
    q, cache, row_seq, row_pos, scale, want = attention_case(dtype, n_q, n_kv, dim, lengths, new, seed=dim, sharp=700)
    ctx = step_like(lengths, new)
    for ctas in (16, 12, None):
        got = kernels.attention_decode(q, cache, ctx, n_q, n_kv, dim, scale, n_ctas=ctas)
        assert torch.isfinite(got).all()
        assert torch.allclose(got.float().cpu(), want, atol=tol(dtype, 2), rtol=tol(dtype)), ctas
        again = kernels.attention_decode(q, cache, ctx, n_q, n_kv, dim, scale, n_ctas=ctas)
        assert torch.equal(again, got)


def test_attention_tensor_core_window_edges():
    from dryft_flash_infer_b200.ops import kernels

    dtype = torch.bfloat16
    for window, ring in ((100, 192), (64, 128), (1, 64), (130, 320)):
        lengths, new = [500, 131, 40], [3, 2, 40]
        q, cache, row_seq, row_pos, scale, want = attention_case(dtype, 4, 2, 32, lengths, new, window=window,
                                                                 ring_tokens=ring, seed=window)
        got = kernels.attention_prefill(q, cache, step_like(lengths, new), 4, 2, 32, scale, window)
        assert torch.isfinite(got).all()
        assert torch.allclose(got.float().cpu(), want, atol=tol(dtype, 2), rtol=tol(dtype)), window
        lengths, new = [500, 131, 40, 1], [1, 1, 1, 1]
        q, cache, row_seq, row_pos, scale, want = attention_case(dtype, 4, 2, 32, lengths, new, window=window,
                                                                 ring_tokens=ring, seed=window + 1)
        for ctas in (1, 3, 11, None):
            got = kernels.attention_decode(q, cache, step_like(lengths, new), 4, 2, 32, scale, window, n_ctas=ctas)
            assert torch.isfinite(got).all()
            assert torch.allclose(got.float().cpu(), want, atol=tol(dtype, 2), rtol=tol(dtype)), (window, ctas)


@pytest.mark.parametrize("m", [1, 3, 8, 9, 17, 33, 64])
@pytest.mark.parametrize("n, k", [(64, 96), (100, 200), (2560, 4096), (320, 2560), (37, 72)])
def test_skinny_gemm(m, n, k):
    from dryft_flash_infer_b200.ops import kernels

    g = torch.Generator().manual_seed(m * n + k)
    x = (torch.randn(m, k, generator=g)).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16)
    want = x.float() @ w.float().T
    for ctas in (None, 1, 2, 3, 7, 500):             # however the units are dealt out, the sum is the same
        got = kernels.skinny_linear(x.cuda(), w.cuda(), torch.float32, n_ctas=ctas)
        assert torch.allclose(got.cpu(), want, atol=2e-3, rtol=1e-3), (ctas, float((got.cpu() - want).abs().max()))
        again = kernels.skinny_linear(x.cuda(), w.cuda(), torch.float32, n_ctas=ctas)
        assert torch.equal(again, got)                 # counters were left ready, and the order of sums is fixed
    got = kernels.skinny_linear(x.cuda(), w.cuda())
    assert got.dtype == torch.bfloat16 and torch.allclose(got.float().cpu(), want, atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("m", [1, 8, 20, 64])
@pytest.mark.parametrize("inter, k", [(200, 96), (128, 64), (9728, 2560), (33, 40)])
def test_skinny_gemm_with_swiglu(m, inter, k):
    from dryft_flash_infer_b200.ops import kernels

    g = torch.Generator().manual_seed(m + inter)
    x = (torch.randn(m, k, generator=g)).to(torch.bfloat16)
    w = (torch.randn(2 * inter, k, generator=g) * 0.1).to(torch.bfloat16)
    gu = x.float() @ w.float().T
    want = gu[:, :inter] / (1 + torch.exp(-gu[:, :inter])) * gu[:, inter:]
    for ctas in (None, 1, 2, 5, 333):
        got = kernels.skinny_linear(x.cuda(), w.cuda(), torch.float32, swiglu=True, n_ctas=ctas)
        assert torch.allclose(got.cpu(), want, atol=3e-3, rtol=2e-3), (ctas, float((got.cpu() - want).abs().max()))
    got = kernels.linear_swiglu(x.cuda(), w.cuda())
    assert got.dtype == torch.bfloat16 and torch.allclose(got.float().cpu(), want, atol=3e-2, rtol=1e-2)


@pytest.mark.parametrize("m, n, k", [(256, 256, 64), (300, 320, 200), (2048, 2560, 4096), (1, 8, 8), (700, 6144, 96),
                                     (5000, 520, 264)])
def test_tcgen05_pair_gemm(m, n, k):
    """The persistent kernel that runs a 256 x 256 tile on a pair of SMs: one tile, ragged edges, more
    tiles than clusters (each cluster walks several, through both accumulators)."""
    from dryft_flash_infer_b200.ops import kernels

    g = torch.Generator().manual_seed(m + n + k)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16)
    want = x.float() @ w.float().T
    got = kernels.pair_linear(x.cuda(), w.cuda())
    assert kernels.pair_error() == 0
    assert got.dtype == torch.bfloat16 and torch.allclose(got.float().cpu(), want, atol=2e-2, rtol=1e-2)
    assert torch.equal(kernels.pair_linear(x.cuda(), w.cuda()), got)


@pytest.mark.parametrize("m, inter, k", [(256, 128, 64), (300, 200, 96), (2048, 9728, 2560), (5, 72, 40), (1000, 1000, 520)])
def test_tcgen05_pair_gemm_swiglu(m, inter, k):
    from dryft_flash_infer_b200.ops import kernels

    g = torch.Generator().manual_seed(m + inter + k)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * inter, k, generator=g) * 0.1).to(torch.bfloat16)
    gu = x.float() @ w.float().T
    want = gu[:, :inter] / (1 + torch.exp(-gu[:, :inter])) * gu[:, inter:]
    got = kernels.pair_linear(x.cuda(), w.cuda(), swiglu=True)
    assert kernels.pair_error() == 0
    assert torch.allclose(got.float().cpu(), want, atol=0.02 * float(want.abs().max()), rtol=2e-2)


@pytest.mark.parametrize("m", [1, 3, 8, 17, 33, 64])
@pytest.mark.parametrize("n, k", [(128, 64), (100, 200), (2560, 4096), (320, 2560), (37, 72)])
def test_tcgen05_decode_gemm(m, n, k):
    from dryft_flash_infer_b200.ops import kernels

    g = torch.Generator().manual_seed(m * n + k)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16)
    want = x.float() @ w.float().T
    for ctas in (None, 1, 2, 3, 7, 500):             # however the units are dealt out, the sum is the same
        got = kernels.decode_linear(x.cuda(), w.cuda(), torch.float32, n_ctas=ctas)
        assert kernels.tc_error() == 0
        assert torch.allclose(got.cpu(), want, atol=2e-3, rtol=1e-3), (ctas, float((got.cpu() - want).abs().max()))
        again = kernels.decode_linear(x.cuda(), w.cuda(), torch.float32, n_ctas=ctas)
        assert torch.equal(again, got)
    got = kernels.decode_linear(x.cuda(), w.cuda())
    assert got.dtype == torch.bfloat16 and torch.allclose(got.float().cpu(), want, atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("m", [1, 8, 20, 64])
@pytest.mark.parametrize("inter, k", [(200, 96), (128, 64), (9728, 2560), (40, 40)])
def test_tcgen05_decode_gemm_with_swiglu(m, inter, k):
    from dryft_flash_infer_b200.ops import kernels

    g = torch.Generator().manual_seed(m + inter)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * inter, k, generator=g) * 0.1).to(torch.bfloat16)
    gu = x.float() @ w.float().T
    want = gu[:, :inter] / (1 + torch.exp(-gu[:, :inter])) * gu[:, inter:]
    for ctas in (None, 1, 2, 5, 333):
        got = kernels.decode_linear(x.cuda(), w.cuda(), torch.float32, swiglu=True, n_ctas=ctas)
        assert kernels.tc_error() == 0
        assert torch.allclose(got.cpu(), want, atol=3e-3, rtol=2e-3), (ctas, float((got.cpu() - want).abs().max()))


@pytest.mark.parametrize("m", [1, 8, 33, 64])
@pytest.mark.parametrize("hidden, k, n2", [(200, 96, 72), (128, 64, 256), (2560, 4096, 640), (40, 40, 40)])
def test_tcgen05_decode_gemm_with_the_norm_fused_around_it(m, hidden, k, n2):
    """A product that adds its result to the residual and prepares the norm, then products that finish
    that norm (plain and with SwiGLU), against add -> rms_norm -> product done one after the other."""
    from dryft_flash_infer_b200.ops import kernels

    g = torch.Generator().manual_seed(m + hidden + k)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(hidden, k, generator=g) * 0.1).to(torch.bfloat16)
    residual = (torch.randn(m, hidden, generator=g) * 3).to(torch.bfloat16)
    norm_w = 1 + 0.3 * torch.randn(hidden, generator=g)
    w2 = (torch.randn(n2, hidden, generator=g) * 0.1).to(torch.bfloat16)
    gate_up = (torch.randn(2 * n2, hidden, generator=g) * 0.1).to(torch.bfloat16)
    eps = 1e-5
    for ctas in (None, 1, 3, 500):
        res = residual.clone().cuda()
        scaled = kernels.decode_linear(x.cuda(), w.cuda(), n_ctas=ctas, add_norm=(res, norm_w.cuda(), eps))
        assert kernels.tc_error() == 0 and isinstance(scaled, kernels.ScaledRows)
        delta = (x.float() @ w.float().T).to(torch.bfloat16).float()
        want_res = (residual.float() + delta).to(torch.bfloat16).float()
        got_res = res.float().cpu()
        # the delta may round the other way where the float32 sums differ in their last bits
        assert torch.allclose(got_res, want_res, atol=0.04, rtol=1e-2)
        assert torch.equal(scaled.rows.float().cpu(), (got_res * norm_w).to(torch.bfloat16).float())
        ssq = scaled.ssq.cpu()[:, :m].sum(0)
        assert torch.allclose(ssq, (got_res ** 2).sum(-1), rtol=1e-5)
        normed = plain_model.rms_norm(got_res, norm_w, eps)
        y = kernels.decode_linear(scaled, w2.cuda(), torch.float32, n_ctas=ctas)
        want = normed @ w2.float().T
        assert torch.allclose(y.cpu(), want, atol=0.02 * float(want.abs().max()), rtol=1e-2), float((y.cpu() - want).abs().max())
        z = kernels.linear_swiglu(scaled, gate_up.cuda())
        gu = normed @ gate_up.float().T
        want = gu[:, :n2] / (1 + torch.exp(-gu[:, :n2])) * gu[:, n2:]
        assert torch.allclose(z.float().cpu(), want, atol=0.03 * float(want.abs().max()), rtol=2e-2)
    with pytest.raises(kernels.KernelError, match="plain bfloat16"):
        kernels.decode_linear(x.cuda(), w.cuda(), torch.float32, add_norm=(residual.cuda(), norm_w.cuda(), eps))


@pytest.mark.parametrize("m, hidden, k, n2", [(65, 200, 96, 72), (300, 2560, 512, 136), (129, 40, 40, 40)])
def test_product_over_many_rows_with_the_residual_as_its_addend(m, hidden, k, n2, monkeypatch):
    """More rows than the decode kernel takes: ``linear(..., add_norm=...)`` adds the product to the residual
    in place and hands on the complete rows of the norm, which the products after it take as they are."""
    from dryft_flash_infer_b200.ops import kernels

    g = torch.Generator().manual_seed(m + hidden + k)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(hidden, k, generator=g) * 0.1).to(torch.bfloat16)
    residual = (torch.randn(m, hidden, generator=g) * 3).to(torch.bfloat16)
    norm_w = 1 + 0.3 * torch.randn(hidden, generator=g)
    w2 = (torch.randn(n2, hidden, generator=g) * 0.1).to(torch.bfloat16)
    gate_up = (torch.randn(2 * n2, hidden, generator=g) * 0.1).to(torch.bfloat16)
    eps = 1e-5
    assert kernels.add_norm_fusable(residual.cuda()) and not kernels.add_norm_fusable(residual.float().cuda())
    for gemm in ("library", "own"):
        monkeypatch.setattr(kernels, "PREFILL_GEMM", gemm)
        res = residual.clone().cuda()
        normed = kernels.linear(x.cuda(), w.cuda(), add_norm=(res, norm_w.cuda(), eps))
        assert isinstance(normed, kernels.ScaledRows) and normed.ssq is None and normed.rows.shape == (m, hidden)
        want_res = residual.float() + x.float() @ w.float().T
        got_res = res.float().cpu()
        assert torch.allclose(got_res, want_res, atol=0.04, rtol=1e-2), gemm     # one rounding of the float32 sum
        want = plain_model.rms_norm(got_res, norm_w, eps)
        assert torch.allclose(normed.rows.float().cpu(), want, atol=tol(torch.bfloat16, 4), rtol=tol(torch.bfloat16)), gemm
        rows = normed.rows.float().cpu()
        y = kernels.linear(normed, w2.cuda())
        want = rows @ w2.float().T
        assert torch.allclose(y.float().cpu(), want, atol=0.02 * float(want.abs().max()), rtol=1e-2), gemm
        z = kernels.linear_swiglu(normed, gate_up.cuda())
        gu = rows @ gate_up.float().T
        want = gu[:, :n2] / (1 + torch.exp(-gu[:, :n2])) * gu[:, n2:]
        assert torch.allclose(z.float().cpu(), want, atol=0.03 * float(want.abs().max()), rtol=2e-2), gemm
        few = kernels.ScaledRows(normed.rows[:5].contiguous(), None, hidden, eps)
        y = kernels.decode_linear(few, w2.cuda(), torch.float32)            # the decode kernel takes complete rows too
        assert torch.allclose(y.cpu(), (rows[:5] @ w2.float().T), atol=0.02 * float(want.abs().max()) + 0.02, rtol=1e-2)


@pytest.mark.parametrize("n_q, n_kv, dim", [(8, 2, 128), (3, 1, 64), (4, 4, 128), (32, 8, 128)])
def test_attention_tcgen05_prefill(n_q, n_kv, dim):
    from dryft_flash_infer_b200.ops import kernels

    dtype = torch.bfloat16
    for lengths, new in (([70, 3, 130], [70, 3, 130]), ([70, 3, 200], [10, 3, 67]), ([257, 64, 1], [1, 1, 1]),
                         ([300], [300]), ([700, 129], [257, 128])):
        q, cache, row_seq, row_pos, scale, want = attention_case(dtype, n_q, n_kv, dim, lengths, new, seed=dim, sharp=5)
        for tiles in (0, 1, 2):          # the launch's choice, one query tile a CTA, two
            got = kernels.attention_prefill_tc(q, cache, step_like(lengths, new), n_q, n_kv, dim, scale, tiles_per_cta=tiles)
            assert kernels.attention_tc_error(dim) == 0
            assert torch.isfinite(got).all(), (lengths, new, tiles)
            assert torch.allclose(got.float().cpu(), want, atol=tol(dtype, 2), rtol=tol(dtype)), (lengths, new, tiles)
    for window, ring in ((100, 192), (64, 128), (130, 320)):
        lengths, new = [500, 131, 40], [3, 2, 40]
        q, cache, row_seq, row_pos, scale, want = attention_case(dtype, n_q, n_kv, dim, lengths, new, window=window,
                                                                 ring_tokens=ring, seed=window)
        for tiles in (1, 2):
            got = kernels.attention_prefill_tc(q, cache, step_like(lengths, new), n_q, n_kv, dim, scale, window, tiles_per_cta=tiles)
            assert kernels.attention_tc_error(dim) == 0
            assert torch.isfinite(got).all()
            assert torch.allclose(got.float().cpu(), want, atol=tol(dtype, 2), rtol=tol(dtype)), (window, tiles)


@pytest.mark.parametrize("m, n, k", [(1, 1, 1), (7, 130, 100), (64, 64, 16), (65, 63, 17), (300, 320, 200), (3, 1000, 2563)])
def test_plain_float32_pipe_gemm(m, n, k):
    """The product of the true 32-bit path, and of bfloat16 matrices whose width is no multiple of 8:
    float32 operands against a float64 product (no reduced-precision mode would pass this bound),
    bfloat16 operands with bfloat16 and float32 results."""
    from dryft_flash_infer_b200.ops import kernels

    g = torch.Generator().manual_seed(m + n + k)
    x = torch.randn(m, k, generator=g)
    w = torch.randn(n, k, generator=g) * 0.1
    want = (x.double() @ w.double().T)
    got = kernels.simt_linear(x.cuda(), w.cuda())
    assert got.dtype == torch.float32
    assert float((got.cpu().double() - want).abs().max()) <= 2e-6 * max(1.0, k ** 0.5) * float(want.abs().max() + 1)
    assert torch.equal(kernels.linear(x.cuda(), w.cuda()), got)            # float32 operands always run this kernel
    x16, w16 = x.to(torch.bfloat16), w.to(torch.bfloat16)
    want16 = x16.double() @ w16.double().T
    unrounded = kernels.simt_linear(x16.cuda(), w16.cuda(), torch.float32)
    assert float((unrounded.cpu().double() - want16).abs().max()) <= 2e-6 * max(1.0, k ** 0.5) * float(want16.abs().max() + 1)
    rounded = kernels.simt_linear(x16.cuda(), w16.cuda())
    assert rounded.dtype == torch.bfloat16 and torch.equal(rounded, unrounded.to(torch.bfloat16))
    if k % 8:
        assert torch.equal(kernels.linear(x16.cuda(), w16.cuda()), rounded)  # widths the TMA kernels do not take


@pytest.mark.parametrize("n_q, n_kv, dim", [(8, 2, 128), (32, 8, 128), (4, 1, 64)])
@pytest.mark.parametrize("length", [200, 330, 700, 960])
def test_attention_decode_of_short_sequences_in_four_parts(n_q, n_kv, dim, length):
    """Few short sequences of one length (4 to 15 pages): with CTAs to spare every group is cut into four
    parts of one to four pages, which meet in a cluster."""
    from dryft_flash_infer_b200.ops import kernels

    dtype = torch.bfloat16
    n_seqs = 2
    lengths, new = [length] * n_seqs, [1] * n_seqs
    q, cache, row_seq, row_pos, scale, want = attention_case(dtype, n_q, n_kv, dim, lengths, new, seed=dim + length, sharp=length // 3)
    ctx = step_like(lengths, new)
    for ctas in (None, 4 * n_seqs * n_kv, 4 * n_seqs * n_kv + 8, 7):
        got = kernels.attention_decode(q, cache, ctx, n_q, n_kv, dim, scale, n_ctas=ctas)
        assert torch.isfinite(got).all()
        assert torch.allclose(got.float().cpu(), want, atol=tol(dtype, 2), rtol=tol(dtype)), ctas
        assert torch.equal(kernels.attention_decode(q, cache, ctx, n_q, n_kv, dim, scale, n_ctas=ctas), got)


@pytest.mark.parametrize("m", [1, 8, 33, 64])
def test_a_word_about_the_next_product_changes_no_result(m):
    """``then=`` names the weights that the step streams next; the kernel asks some of them into L2.  Whatever
    those weights are (few tiles or many, SwiGLU rows, a matrix that ends inside a tile), the product's
    result is the same bit for bit, with every number of CTAs."""
    from dryft_flash_infer_b200.ops import kernels

    g = torch.Generator().manual_seed(m)
    x = torch.randn(m, 200, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(300, 200, generator=g) * 0.05).to(torch.bfloat16).cuda()
    gate_up = (torch.randn(2 * 72, 200, generator=g) * 0.1).to(torch.bfloat16).cuda()
    plain = kernels.decode_linear(x, w, torch.float32)
    plain_act = kernels.decode_linear(x, gate_up, swiglu=True)
    followers = [(torch.randn(n, k, generator=g).to(torch.bfloat16).cuda(), sw)
                 for n, k, sw in ((37, 72, False), (2560, 4096, False), (2 * 9728, 2560, True), (2 * 40, 40, True), (128, 64, False))]
    for follower, sw in followers:
        then = kernels.next_weights(follower, swiglu=sw)
        assert then.hint(m) is not None and then is kernels.next_weights(follower, swiglu=sw)
        for ctas in (None, 1, 3, 500):
            assert torch.equal(kernels.decode_linear(x, w, torch.float32, n_ctas=ctas, then=then),
                               kernels.decode_linear(x, w, torch.float32, n_ctas=ctas))
        assert torch.equal(kernels.decode_linear(x, w, torch.float32, then=then), plain)
        assert torch.equal(kernels.decode_linear(x, gate_up, swiglu=True, then=then), plain_act)
        assert kernels.tc_error() == 0
    # weights that the decode kernel would not take give no hint, and no hint is taken for more than 64 rows
    assert kernels.next_weights(torch.zeros(16, 12, dtype=torch.bfloat16, device="cuda")).hint(m) is None
    assert kernels.next_weights(torch.zeros(16, 16, dtype=torch.float32, device="cuda")).hint(m) is None
    assert kernels.next_weights(followers[1][0]).hint(65) is None
    assert kernels.next_weights(None) is None


@pytest.mark.parametrize("n_q, n_kv, dim", [(32, 8, 128), (8, 2, 64), (3, 1, 96), (4, 4, 32), (2, 2, 128)])
@pytest.mark.parametrize("length", [500, 513, 1270, 2049, 4100, 5100, 5200])
def test_attention_decode_of_few_groups_in_clusters_of_eight(n_q, n_kv, dim, length):
    """Few groups of up to four query heads and 8 to 80 pages each (a small batch at a middle context): the
    launch forms clusters of eight CTAs and every group is cut into eight parts that meet in their cluster;
    with more pages (5,200 keys) or with too few CTAs for that the parts meet as before."""
    from dryft_flash_infer_b200.ops import kernels

    dtype = torch.bfloat16
    n_seqs = max(1, 8 // n_kv) if length < 3000 else 1
    lengths, new = [length] * n_seqs, [1] * n_seqs
    q, cache, row_seq, row_pos, scale, want = attention_case(dtype, n_q, n_kv, dim, lengths, new, seed=dim + length,
                                                             sharp=length // 3)
    ctx = step_like(lengths, new)
    for ctas in (None, 64, 16):
        got = kernels.attention_decode(q, cache, ctx, n_q, n_kv, dim, scale, n_ctas=ctas)
        assert torch.isfinite(got).all()
        assert torch.allclose(got.float().cpu(), want, atol=tol(dtype, 2), rtol=tol(dtype)), ctas
        assert torch.equal(kernels.attention_decode(q, cache, ctx, n_q, n_kv, dim, scale, n_ctas=ctas), got)
    kernels.check_status()


@pytest.mark.parametrize("n_seqs, n_kv, group, dim", [(2, 8, 4, 128), (9, 8, 4, 128), (16, 8, 4, 128), (40, 4, 2, 64), (33, 8, 1, 32),
                                                     (70, 8, 4, 128), (70, 5, 3, 48), (3, 1, 16, 64), (20, 2, 8, 16)])
@pytest.mark.parametrize("spread", ["mild", "wild"])
def test_attention_decode_of_sequences_of_different_lengths(n_seqs, n_kv, group, dim, spread):
    """Lengths that differ, for every way the kernel deals them: few groups -> each cut into the parts of a
    cluster of 8, 4 or 2 CTAs (a sequence of one or two pages leaves parts empty); up to as many groups as
    CTAs -> one whole group a CTA; more -> several whole groups a CTA; and, where the longest group would
    hold a CTA too long, equal runs across groups with tickets.  With token preparation inside and without."""
    from dryft_flash_infer_b200.ops import kernels
    from dryft_flash_infer_b200.parts.rotary import RotaryEmbedding

    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(n_seqs * 131 + dim)
    if spread == "mild":
        lengths = [int(x) for x in torch.randint(520, 700, (n_seqs,), generator=g)]
    else:
        lengths = [int(x) for x in torch.randint(1, 1400, (n_seqs,), generator=g)]
        lengths[0], lengths[-1] = 1, 65
    new = [1] * n_seqs
    n_q = n_kv * group
    q, cache, row_seq, row_pos, scale, want = attention_case(dtype, n_q, n_kv, dim, lengths, new, seed=dim + n_seqs)
    ctx = step_like(lengths, new)
    for ctas in (None, 40):
        got = kernels.attention_decode(q, cache, ctx, n_q, n_kv, dim, scale, n_ctas=ctas)
        assert torch.isfinite(got).all()
        assert torch.allclose(got.float().cpu(), want, atol=tol(dtype, 2), rtol=tol(dtype)), ctas
        assert torch.equal(kernels.attention_decode(q, cache, ctx, n_q, n_kv, dim, scale, n_ctas=ctas), got)
    if dim in (16, 32, 64, 128) and group <= 16:
        # the raw projection in, norm + rotation + cache write inside: against the two kernels one after the other
        qkv = torch.randn(n_seqs, (n_q + 2 * n_kv) * dim, generator=g).to(dtype).cuda()
        qw, kw = (1 + 0.3 * torch.randn(dim, generator=g)).cuda(), (1 + 0.3 * torch.randn(dim, generator=g)).cuda()
        rot = RotaryEmbedding(0, dim, 4321.0)
        rot.prepare(2048, "cuda")
        two = LayerCache(cache.k.clone(), cache.v.clone(), cache.block_table, 64, 0, True)
        prepared = kernels.qk_norm_rope_write(qkv.clone(), n_q, n_kv, dim, qw, kw, 1e-5, rot.cos, rot.sin, row_pos, row_seq, two)
        want2 = kernels.attention_decode(prepared, two, ctx, n_q, n_kv, dim, scale, n_ctas=7)
        one = LayerCache(cache.k.clone(), cache.v.clone(), cache.block_table, 64, 0, True)
        got2 = kernels.attention_decode(None, one, ctx, n_q, n_kv, dim, scale,
                                        prep=kernels.TokenPrep(qkv, qw, kw, 1e-5, rot.cos, rot.sin))
        assert torch.allclose(got2.float(), want2.float(), atol=tol(dtype, 2), rtol=tol(dtype))
        assert torch.allclose(one.k.float(), two.k.float(), atol=tol(dtype), rtol=tol(dtype), equal_nan=True)
        assert torch.equal(one.v.float().nan_to_num(7.0), two.v.float().nan_to_num(7.0))
    kernels.check_status()


@pytest.mark.parametrize("n_seqs, n_kv, group, dim", [(1, 8, 4, 128), (1, 4, 2, 64), (3, 2, 4, 128), (1, 8, 4, 96), (1, 15, 1, 32)])
def test_attention_decode_in_clusters_of_sixteen(n_seqs, n_kv, group, dim):
    """The groups of one sequence (fewer than sixteen) whose cache may grow past 2,048 keys, but not past ten
    pages for each of sixteen parts, are launched in clusters of sixteen CTAs: sixteen parts that meet in the
    cluster from 16 pages on, and the other ways of dealing where that does not apply (fewer pages; sequences
    of different lengths; a head size whose columns sixteen CTAs cannot share, which stays with eight).  With
    token preparation inside and without."""
    from dryft_flash_infer_b200.ops import kernels
    from dryft_flash_infer_b200.parts.rotary import RotaryEmbedding

    dtype = torch.bfloat16
    n_q = n_kv * group
    g = torch.Generator().manual_seed(dim + n_kv)
    lib = kernels._attention_library(dim)
    assert tuple(lib.dfi_attention_decode_kv_step(i) for i in range(4)) == kernels.DECODE_KV_STEPS + (0,)
    for longest, limit in ((2100, 2100), (4096, 4096), (9001, 10240), (600, 4096), (1023, 8000), (65, 4096), (40, 4096),
                           (1025, 2049)):
        lengths = [longest] + [max(1, longest // (3 * i + 2)) for i in range(n_seqs - 1)]
        new = [1] * n_seqs
        q, cache, row_seq, row_pos, scale, want = attention_case(dtype, n_q, n_kv, dim, lengths, new, seed=dim + longest,
                                                                 sharp=max(1, longest // 3))
        ctx = step_like(lengths, new)
        ctx.max_kv_len = limit
        for ctas in (None, 64):
            got = kernels.attention_decode(q, cache, ctx, n_q, n_kv, dim, scale, n_ctas=ctas)
            assert torch.isfinite(got).all()
            assert torch.allclose(got.float().cpu(), want, atol=tol(dtype, 2), rtol=tol(dtype)), (longest, limit, ctas)
            assert torch.equal(kernels.attention_decode(q, cache, ctx, n_q, n_kv, dim, scale, n_ctas=ctas), got)
        if dim in (32, 64, 128):
            qkv = torch.randn(n_seqs, (n_q + 2 * n_kv) * dim, generator=g).to(dtype).cuda()
            qw, kw = (1 + 0.3 * torch.randn(dim, generator=g)).cuda(), (1 + 0.3 * torch.randn(dim, generator=g)).cuda()
            rot = RotaryEmbedding(0, dim, 4321.0)
            rot.prepare(10240, "cuda")
            two = LayerCache(cache.k.clone(), cache.v.clone(), cache.block_table, 64, 0, True)
            prepared = kernels.qk_norm_rope_write(qkv.clone(), n_q, n_kv, dim, qw, kw, 1e-5, rot.cos, rot.sin, row_pos, row_seq, two)
            want2 = kernels.attention_decode(prepared, two, ctx, n_q, n_kv, dim, scale, n_ctas=7)
            one = LayerCache(cache.k.clone(), cache.v.clone(), cache.block_table, 64, 0, True)
            got2 = kernels.attention_decode(None, one, ctx, n_q, n_kv, dim, scale,
                                            prep=kernels.TokenPrep(qkv, qw, kw, 1e-5, rot.cos, rot.sin))
            assert torch.allclose(got2.float(), want2.float(), atol=tol(dtype, 2), rtol=tol(dtype)), (longest, limit)
            assert torch.equal(one.v.float().nan_to_num(7.0), two.v.float().nan_to_num(7.0))
    kernels.check_status()


@pytest.mark.parametrize("n_seqs, n_kv, group, dim, lengths", [
    (1, 8, 4, 128, [4096]), (8, 8, 4, 128, [1500] * 8), (3, 2, 4, 64, [3000, 700, 65]), (40, 4, 2, 64, None),
    (70, 5, 3, 48, None), (9, 8, 4, 128, None), (2, 1, 16, 32, [200, 200])])
def test_attention_decode_with_plans_worked_out_once_for_all_layers(n_seqs, n_kv, group, dim, lengths):
    """``ctx.decode_plans``: the first launch of a pass works the plans of all CTAs out in a kernel of its own, later
    launches (other layers: other queries and caches, the same sequences) read them.  Same results, bit for bit,
    as launches whose CTAs plan for themselves; and a second pass with other lengths gets plans of its own."""
    from dryft_flash_infer_b200.ops import kernels

    dtype = torch.bfloat16
    n_q = n_kv * group
    g = torch.Generator().manual_seed(n_seqs * 7 + dim)
    for round_ in range(2):
        if lengths is None or round_ == 1:
            lens = [int(x) for x in torch.randint(1, 1400, (n_seqs,), generator=g)]
        else:
            lens = list(lengths)
        new = [1] * n_seqs
        layers = [attention_case(dtype, n_q, n_kv, dim, lens, new, seed=dim + n_seqs + layer) for layer in range(3)]
        ctx = step_like(lens, new)
        for ctas in (None, 40):
            alone = [kernels.attention_decode(q, cache, ctx, n_q, n_kv, dim, scale, n_ctas=ctas)
                     for q, cache, _, _, scale, _ in layers]
            ctx.decode_plans = {}
            shared = [kernels.attention_decode(q, cache, ctx, n_q, n_kv, dim, scale, n_ctas=ctas)
                      for q, cache, _, _, scale, _ in layers]
            assert len(ctx.decode_plans) == 1
            ctx.decode_plans = None
            for layer, (a, b) in enumerate(zip(alone, shared)):
                assert torch.equal(a, b), (round_, ctas, layer)
                assert torch.allclose(b.float().cpu(), layers[layer][5], atol=tol(dtype, 2), rtol=tol(dtype)), (round_, ctas, layer)
    kernels.check_status()
