"""Each CUDA kernel alone against its plain PyTorch version (tests/ref_ops.py), in 32-bit and in
bfloat16, at sizes other than the models': head sizes 16..80, odd head counts, widths and
vocabularies that are no power of two, page sizes 4..32, spans that start and end inside pages."""
import random

import pytest
import torch

import ref_ops
from zig_ai_b200.cache.manager import CacheView
from zig_ai_b200.engine.batch import pack_step

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from zig_ai_b200.kernels import ops as o
    o.require()
    return o


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


def make_step(o, dtype, ctx_lens, q_lens, page_size, num_pages, seed, device="cuda", slots=None):
    """A step over fresh random block tables: request s holds ctx_lens[s] cached positions and
    brings q_lens[s] new ones."""
    g = random.Random(seed)
    free = list(range(1, num_pages))
    g.shuffle(free)
    spans, tables = [], []
    width = max(-(-(c + n) // page_size) for c, n in zip(ctx_lens, q_lens))
    for s, (c, n) in enumerate(zip(ctx_lens, q_lens)):
        need = -(-(c + n) // page_size)
        row = [free.pop() for _ in range(need)]
        tables.append(row + [0] * (width - need))
        spans.append((s, c, [0] * n, [], (slots[s] if slots else s + 1)))
    return pack_step(o, dtype, torch.device(device), spans, {0: tables})


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,H,V", [(7, 96, 517), (1, 1000, 33), (33, 2050, 129)])
def test_embed_and_gather(dtype, N, H, V):
    o = ops()
    g = torch.Generator().manual_seed(1)
    table = torch.randn(V, H, generator=g).to(dtype).cuda()
    ids = torch.randint(0, V, (N,), generator=g, dtype=torch.int32).cuda()
    h = o.embed(ids, table)
    assert torch.equal(h, ref_ops.embed(ids, table))
    pending = torch.randn(N, H, generator=g).to(dtype).cuda()
    rows = torch.tensor([N - 1, 0, N // 2], dtype=torch.int32).cuda()
    assert torch.equal(o.gather_add(h, pending, rows), ref_ops.gather_add(h, pending, rows))
    assert torch.equal(o.gather_add(h, None, rows), ref_ops.gather_add(h, None, rows))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,H,eps", [(5, 96, 1e-6), (3, 1000, 1e-5), (17, 4104, 1e-3), (1, 64, 1e-5),
                                     (70, 1024, 1e-5), (100, 1000, 1e-6), (65, 2048, 1e-5), (64, 1540, 1e-3), (300, 96, 1e-5),
                                     (600, 1024, 1e-5), (513, 1000, 1e-6), (2048, 2048, 1e-5), (519, 1536, 1e-3), (512, 4, 1e-5)])
def test_add_rmsnorm(dtype, N, H, eps):
    o = ops()
    g = torch.Generator().manual_seed(2)
    h = (torch.randn(N, H, generator=g) * 3).cuda()
    delta = torch.randn(N, H, generator=g).to(dtype).cuda()
    w = (1 + 0.1 * torch.randn(H, generator=g)).cuda()
    h1, h2 = h.clone(), h.clone()
    a = o.add_rmsnorm(h1, delta, w, eps, dtype)
    b = ref_ops.add_rmsnorm(h2, delta, w, eps, dtype)
    assert torch.equal(h1, h2)                       # the 32-bit residual sum is exact
    assert torch.allclose(a.float(), b.float(), **tol(dtype))
    a = o.add_rmsnorm(h1, None, w, eps, dtype)
    b = ref_ops.add_rmsnorm(h2, None, w, eps, dtype)
    assert torch.allclose(a.float(), b.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,F", [(3, 192), (9, 1000), (1, 4608)])
def test_silu_mul(dtype, N, F):
    o = ops()
    gu = (torch.randn(N, 2 * F, generator=torch.Generator().manual_seed(3)) * 2).to(dtype).cuda()
    assert torch.allclose(o.silu_mul(gu, F).float(), ref_ops.silu_mul(gu, F).float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("C,L,bias", [(96, 4, True), (64, 3, False), (200, 2, True), (48, 1, False), (130, 7, True)])
def test_short_conv_spans_and_state(dtype, C, L, bias):
    """Spans shorter than, equal to and longer than the state, beside single tokens; then a second
    step that continues from the state the first one left; then a step of single tokens only."""
    o = ops()
    g = torch.Generator().manual_seed(4)
    w = (torch.randn(C, L, generator=g) * 0.3).cuda()
    b = (torch.randn(C, generator=g) * 0.3).cuda() if bias else None
    rows = max(L - 1, 1)
    state_a = torch.randn(6, rows, C, generator=g).cuda()
    state_b = state_a.clone()
    for q_lens in ([1, L - 1 if L > 1 else 1, L, 2 * L + 3, 1], [5, 1, 1, 2, 9], [1, 1, 1, 1, 1]):
        step = make_step(o, dtype, [3] * 5, q_lens, 8, 64, 5)
        bcx = torch.randn(sum(q_lens), 3 * C, generator=g).to(dtype).cuda()
        za = o.short_conv(bcx, w, b, state_a, step, L, True)
        zb = ref_ops.short_conv(bcx, w, b, state_b, step, L, True)
        assert torch.allclose(za.float(), zb.float(), **tol(dtype)), q_lens
        assert torch.allclose(state_a, state_b, atol=1e-6, rtol=1e-6), q_lens
    assert torch.equal(state_a[0], state_b[0])       # the null slot was never touched


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,rot,ps", [(4, 2, 16, 16, 16), (3, 1, 32, 32, 8), (5, 5, 48, 24, 4),
                                              (6, 2, 80, 80, 32), (16, 8, 64, 64, 16), (2, 1, 128, 128, 16),
                                              (3, 3, 256, 256, 8)])
def test_qk_norm_rope_and_page_write(dtype, Hq, Hkv, D, rot, ps):
    o = ops()
    g = torch.Generator().manual_seed(6)
    ctx, q_lens = [0, ps - 1, 3 * ps, min(1000, 60 * ps)], [ps + 3, 2, 1, 5]
    num_pages = 128
    step = make_step(o, dtype, ctx, q_lens, ps, num_pages, 7)
    N = sum(q_lens)
    qkv = torch.randn(N, (Hq + 2 * Hkv) * D, generator=g).to(dtype).cuda()
    qw = (1 + 0.1 * torch.randn(D, generator=g)).cuda()
    kw = (1 + 0.1 * torch.randn(D, generator=g)).cuda()
    pages_a = torch.zeros(num_pages, 2, Hkv, ps, D, dtype=dtype, device="cuda")
    pages_b = pages_a.clone()
    va = CacheView(0, pages_a, step.block_tables[0], ps)
    vb = CacheView(0, pages_b, step.block_tables[0], ps)
    qa, ka = o.qk_norm_rope(qkv, qw, kw, 1e-5, rot, 10000.0, step, va, Hq, Hkv, D, True, True, True)
    qb, kb = ref_ops.qk_norm_rope(qkv, qw, kw, 1e-5, rot, 10000.0, step, vb, Hq, Hkv, D, True, True, True)
    t = tol(dtype) if dtype == torch.bfloat16 else dict(atol=3e-4, rtol=1e-4)   # 32-bit angles of the plain version at position 1000
    assert torch.allclose(qa.float(), qb.float(), **t)
    assert torch.allclose(ka.float(), kb.float(), **t)
    assert torch.allclose(pages_a.float(), pages_b.float(), **t)
    assert pages_a[0].abs().sum() == 0                # nothing was written to the null page
    # without norm and rotation, then written by the separate kernel
    qa, ka = o.qk_norm_rope(qkv, None, None, 1e-5, 0, 1.0, step, va, Hq, Hkv, D, True, False, True)
    assert torch.equal(qa, qkv[:, :Hq * D].contiguous())
    assert torch.equal(ka, qkv[:, Hq * D:(Hq + Hkv) * D].contiguous())
    pages_c = torch.zeros_like(pages_a)
    vc = CacheView(0, pages_c, step.block_tables[0], ps)
    o.kv_write(ka, qkv[:, (Hq + Hkv) * D:], step, vc, Hkv, D)
    pages_d = torch.zeros_like(pages_a)
    ref_ops.kv_write(ka, qkv[:, (Hq + Hkv) * D:], step, CacheView(0, pages_d, step.block_tables[0], ps), Hkv, D)
    assert torch.equal(pages_c, pages_d)


JUNK = 25.0


def fill_pages(step, ctx, q_lens, ps, Hkv, D, dtype, num_pages, g, junk=JUNK):
    """Random keys and values at every position the step's requests hold.  Everything else (pages no
    request owns, the null page, the unused end of a request's last page) holds a large finite value:
    a kernel that reads a position it should not see gets a score that drowns the rest."""
    pages = torch.full((num_pages, 2, Hkv, ps, D), float(junk), dtype=dtype, device="cuda")
    bt = step.block_tables[0].cpu().long()
    page_ids, offs = [], []
    for s, (c, n) in enumerate(zip(ctx, q_lens)):
        p = torch.arange(c + n)
        page_ids.append(bt[s, p // ps])
        offs.append(p % ps)
    page_ids, offs = torch.cat(page_ids), torch.cat(offs)
    if page_ids.numel():
        vals = torch.randn(page_ids.numel(), 2, Hkv, D, generator=g).to(dtype).cuda()
        pages[page_ids.cuda(), :, :, offs.cuda(), :] = vals
    return pages


def plant_key(pages, step, ps, s, pos, kv_head, key, value):
    """Put `key` and `value` at position `pos` of request s of the step, for one key/value head."""
    page = int(step.block_tables[0][s, pos // ps])
    pages[page, 0, kv_head, pos % ps, :] = key.to(pages.dtype)
    pages[page, 1, kv_head, pos % ps, :] = value.to(pages.dtype)


ATT_SHAPES = [(4, 2, 16, 16, None), (3, 1, 32, 8, None), (6, 3, 48, 4, 7), (8, 2, 80, 32, None),
              (16, 8, 64, 16, None), (2, 2, 128, 16, 40), (32, 2, 96, 16, None), (5, 5, 112, 16, None)]


@pytest.mark.parametrize("dtype,impl", [(torch.float32, None), (torch.bfloat16, None), (torch.bfloat16, "general")])
@pytest.mark.parametrize("Hq,Hkv,D,ps,window", ATT_SHAPES)
def test_paged_attention_mixed_spans(dtype, impl, Hq, Hkv, D, ps, window):
    """Spans that start at 0, inside a page and far into a request, of 1 to 150 rows (more than two
    query tiles), with and without a window."""
    o = ops()
    g = torch.Generator().manual_seed(8)
    ctx, q_lens = [0, ps - 1, 2 * ps, 301, 5, 63], [150, 2, 1, 1, 37, 66]
    num_pages = 256
    step = make_step(o, dtype, ctx, q_lens, ps, num_pages, 9)
    pages = fill_pages(step, ctx, q_lens, ps, Hkv, D, dtype, num_pages, g)
    q = torch.randn(sum(q_lens), Hq * D, generator=g).to(dtype).cuda()
    view = CacheView(0, pages, step.block_tables[0], ps)
    a = o.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, window, impl=impl)
    b = ref_ops.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, window)
    assert torch.allclose(a.float(), b.float(), **tol(dtype))


@pytest.mark.parametrize("impl", ["tcgen05", "mma"])
@pytest.mark.parametrize("Hq,Hkv,ps,window", [(16, 8, 16, None), (4, 1, 64, None), (2, 2, 8, 100), (6, 3, 128, None),
                                              (3, 1, 32, 300)])
def test_span_attention_head_size_64(impl, Hq, Hkv, ps, window):
    """The two span kernels for head size 64 (tcgen05 with TMEM accumulators, and mma.sync): spans of
    1 to 400 rows (more than three blocks of 128 query rows) at contexts of 0, inside a page, and over
    a thousand keys (many key tiles), with and without a window; the status word stays clear."""
    o = ops()
    dtype, D = torch.bfloat16, 64
    g = torch.Generator().manual_seed(28)
    ctx, q_lens = [0, ps - 1, 1100, 301, 5, 127, 640], [400, 2, 130, 1, 37, 129, 128]
    num_pages = (sum(c + n for c, n in zip(ctx, q_lens)) // ps) + 16
    step = make_step(o, dtype, ctx, q_lens, ps, num_pages, 29)
    pages = fill_pages(step, ctx, q_lens, ps, Hkv, D, dtype, num_pages, g)
    q = torch.randn(sum(q_lens), Hq * D, generator=g).to(dtype).cuda()
    view = CacheView(0, pages, step.block_tables[0], ps)
    a = o.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, window, impl=impl)
    b = ref_ops.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, window)
    assert torch.allclose(a.float(), b.float(), **tol(dtype))
    assert o.tc_status() == 0


@pytest.mark.parametrize("Hq,Hkv,D,ps,window", ATT_SHAPES)
def test_paged_attention_single_tokens(Hq, Hkv, D, ps, window):
    """Every span one token (the split-key kernel in bfloat16): contexts of 0 keys, one short of
    and exactly a chunk of 256, several chunks, and one that ends inside a tile."""
    o = ops()
    for dtype in DTYPES:
        g = torch.Generator().manual_seed(18)
        ctx = [0, 1, 254, 255, 256, 700, 63, 1029]
        q_lens = [1] * len(ctx)
        num_pages = 1024
        step = make_step(o, dtype, ctx, q_lens, ps, num_pages, 19)
        assert step.decode_only
        pages = fill_pages(step, ctx, q_lens, ps, Hkv, D, dtype, num_pages, g)
        q = torch.randn(len(ctx), Hq * D, generator=g).to(dtype).cuda()
        view = CacheView(0, pages, step.block_tables[0], ps)
        a = o.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, window)
        b = ref_ops.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, window)
        assert torch.allclose(a.float(), b.float(), **tol(dtype)), dtype
        # more chunks than any request needs (a captured graph is sized for the longest request allowed)
        step.max_kv_len = 3000
        a2 = o.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, window)
        assert torch.equal(a, a2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_len", [1, 3])
def test_attention_finds_one_far_key(dtype, q_len):
    """One key among hundreds, at a page's first position far back, is made to stand out by scaling
    it and the query; the output must be its value (both the single-token and the span kernels)."""
    o = ops()
    Hq, Hkv, D, ps = 4, 2, 64, 16
    g = torch.Generator().manual_seed(10)
    ctx, q_lens = [700], [q_len]
    step = make_step(o, dtype, ctx, q_lens, ps, 64, 11)
    pages = fill_pages(step, ctx, q_lens, ps, Hkv, D, dtype, 64, g)
    q = torch.randn(q_len, Hq * D, generator=g).to(dtype).cuda()
    far = 5 * ps
    bt = step.block_tables[0].cpu()
    for h in range(Hkv):
        pages[bt[0, far // ps], 0, h, 0, :] = (q[0, (h * 2) * D:(h * 2 + 1) * D].float() * 8).to(dtype)
    view = CacheView(0, pages, step.block_tables[0], ps)
    a = o.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, None).float()[0].view(Hq, D)
    for h in (0, 2):
        want = pages[bt[0, far // ps], 1, h // 2, 0, :].float()
        assert torch.allclose(a[h], want, atol=2e-2), h


@pytest.mark.parametrize("R,V", [(1, 517), (5, 65536), (3, 1000)])
def test_argmax_first_maximum(R, V):
    o = ops()
    logits = torch.randn(R, V, generator=torch.Generator().manual_seed(12)).cuda()
    logits[0, V // 3] = 50.0
    logits[0, V // 3 + 7] = 50.0                     # a tie: the first index wins
    assert torch.equal(o.argmax(logits), ref_ops.argmax(logits))
    assert int(o.argmax(logits)[0]) == V // 3


@pytest.mark.parametrize("V", [517, 16391, 50001, 65536])
def test_sampling_matches_plain_version(V):
    o = ops()
    g = torch.Generator().manual_seed(13)
    R = 12
    logits = (torch.randn(R, V, generator=g) * 3).cuda()
    temperature = torch.tensor([0.0, 1.0, 0.7, 1.5, 1.0, 1.0, 0.9, 1.0, 1.0, 2.0, 1.0, 0.5]).cuda()
    top_k = torch.tensor([0, 0, 0, 0, 5, 1, 40, 0, 0, 50, 0, 3], dtype=torch.int32).cuda()
    top_p = torch.tensor([1.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0, 0.5, 0.9, 0.8, 0.01, 0.3]).cuda()
    for trial in range(6):
        u = torch.rand(R, generator=g).cuda()
        a = o.sample(logits, temperature, top_k, top_p, u).cpu()
        b = ref_ops.sample(logits.cpu(), temperature.cpu(), top_k.cpu(), top_p.cpu(), u.cpu())
        for r in range(R):
            if int(a[r]) == int(b[r]):
                continue
            # The kernel sums in 32-bit and in another order than the plain version, so where u falls on
            # the edge between two tokens, or the top-p mass on the edge of its last token, it may take
            # the neighbour.  Nothing else is accepted: the token must be one of the kept set, and u must
            # lie in the token's own interval of the cumulative distribution (within 2e-5 of the mass),
            # for the plain version's kept set or for that set with its edge token dropped or added.
            assert float(temperature[r]) > 0
            ok = any(_u_in_interval(p, int(a[r]), float(u[r])) for p in _kept_distributions(
                logits[r].double().cpu(), float(temperature[r]), int(top_k[r]), float(top_p[r])))
            assert ok, (trial, r, int(a[r]), int(b[r]))


def test_sampling_many_rows_one_block_a_row():
    """More than 32 rows run with one block a row (fewer share a row among a cluster of eight blocks): the same
    checks at 40 rows with every kind of selection, some rows with a kept set beyond the list."""
    o = ops()
    V, R = 20011, 40
    g = torch.Generator().manual_seed(213)
    logits = (torch.randn(R, V, generator=g) * 3).cuda()
    temperature = torch.tensor([[0.0, 1.0, 0.7, 1.3, 2.5][r % 5] for r in range(R)]).cuda()
    top_k = torch.tensor([[0, 40, 0, 5, 6000, 1, 0, 300][r % 8] for r in range(R)], dtype=torch.int32).cuda()
    top_p = torch.tensor([[1.0, 1.0, 0.9, 0.5, 0.95, 1.0, 0.3][r % 7] for r in range(R)]).cuda()
    u = torch.rand(R, generator=g).cuda()
    a = o.sample(logits, temperature, top_k, top_p, u).cpu()
    b = ref_ops.sample(logits.cpu(), temperature.cpu(), top_k.cpu(), top_p.cpu(), u.cpu())
    for r in range(R):
        if int(a[r]) == int(b[r]):
            continue
        assert float(temperature[r]) > 0
        ok = any(_u_in_interval(p, int(a[r]), float(u[r])) for p in _kept_distributions(
            logits[r].double().cpu(), float(temperature[r]), int(top_k[r]), float(top_p[r])))
        assert ok, (r, int(a[r]), int(b[r]))


def test_sampling_large_kept_sets():
    """Rows whose kept set does not fit the kernel's list of 4096 tokens, which take its general way: a flat
    distribution under top-p (a nucleus of tens of thousands of tokens), a top-k above 4096, values with so many
    ties that the k largest are more than 4096 tokens; and beside them rows that fit, with ties at the floor."""
    o = ops()
    V, R = 65536, 6
    g = torch.Generator().manual_seed(113)
    logits = (torch.randn(R, V, generator=g) * 3)
    logits[2] = torch.round(logits[2])                      # a few dozen distinct values: thousands of ties each
    logits[3] = torch.round(logits[3] * 4) / 4
    logits = logits.cuda()
    temperature = torch.tensor([3.0, 1.0, 1.0, 1.0, 2.5, 1.0]).cuda()
    top_k = torch.tensor([0, 5000, 40, 40, 3000, 4096], dtype=torch.int32).cuda()
    top_p = torch.tensor([0.95, 1.0, 1.0, 0.7, 0.9, 0.99]).cuda()
    for trial in range(4):
        u = torch.rand(R, generator=g).cuda()
        a = o.sample(logits, temperature, top_k, top_p, u).cpu()
        b = ref_ops.sample(logits.cpu(), temperature.cpu(), top_k.cpu(), top_p.cpu(), u.cpu())
        for r in range(R):
            if int(a[r]) == int(b[r]):
                continue
            ok = any(_u_in_interval(p, int(a[r]), float(u[r])) for p in _kept_distributions(
                logits[r].double().cpu(), float(temperature[r]), int(top_k[r]), float(top_p[r])))
            assert ok, (trial, r, int(a[r]), int(b[r]))


def _kept_distributions(row, T, k, tp):
    """The probabilities of the kept tokens (zero elsewhere, not normalised) as the plain version
    keeps them, and the two neighbouring choices of the top-p edge."""
    V = row.numel()
    w = row / T
    if 0 < k < V:
        kth = torch.sort(w, descending=True).values[k - 1]
        w = torch.where(w >= kth, w, torch.full_like(w, float("-inf")))
    p = torch.softmax(w, -1)
    if tp >= 1.0:
        return [p]
    sp, _ = torch.sort(p, descending=True, stable=True)
    cum = torch.cumsum(sp, 0)
    cutoff = int((cum >= tp).nonzero()[0]) + 1 if bool((cum >= tp).any()) else V
    out = []
    for c in (cutoff, cutoff - 1, cutoff + 1):
        if 1 <= c <= V:
            out.append(torch.where(p >= sp[c - 1], p, torch.zeros_like(p)))
    return out


def _u_in_interval(p, token, u, eps=2e-5):
    if float(p[token]) <= 0.0:
        return False
    c = torch.cumsum(p, 0)
    total = float(c[-1])
    lo = float(c[token - 1]) if token > 0 else 0.0
    return lo - eps * total <= u * total <= float(c[token]) + eps * total


def test_repetition_penalty():
    o = ops()
    V = 300
    logits = torch.randn(2, V, generator=torch.Generator().manual_seed(14)).cuda()
    want = logits.clone()
    tokens = torch.tensor([3, 7, 299, 5], dtype=torch.int32).cuda()
    counts = torch.tensor([1, 3, 1, 2], dtype=torch.int32).cuda()
    offsets = torch.tensor([0, 3, 4], dtype=torch.int32).cuda()
    penalty = torch.tensor([1.3, 2.0]).cuda()
    for r, (a, b) in enumerate([(0, 3), (3, 4)]):
        for i in range(a, b):
            for _ in range(int(counts[i])):
                v = want[r, tokens[i]]
                want[r, tokens[i]] = v / penalty[r] if v > 0 else v * penalty[r]
    o.repetition_penalty(logits, tokens, counts, offsets, penalty)
    assert torch.allclose(logits, want, atol=1e-6)


# ----------------------------------------------------------------------------- few-rows products
def _lazy(h, delta, gamma, eps, rows=None):
    from zig_ai_b200.parts.base import LazyNorm, Residual
    return LazyNorm(Residual(h), delta, gamma, eps, torch.bfloat16, rows)


@pytest.mark.parametrize("M", [1, 3, 8, 13, 16, 40, 64])
@pytest.mark.parametrize("O,K", [(96, 96), (517, 1000), (1024, 1024), (3072, 1024), (1024, 4608), (130, 8),
                                 (1000, 2048), (130, 8192), (96, 6144), (2048, 7168), (40, 1536), (33, 12288), (16, 12296)])
def test_skinny_gemm_plain_input(M, O, K):
    o = ops()
    g = torch.Generator().manual_seed(20)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(O, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    want = x.float() @ w.float().t()
    if M <= 16:
        before = o.launches
        got = o.linear(x, w)
        assert o.launches == before + 1                 # the fused kernel ran, not the library
    else:
        got = o.linear(x, w)
    assert got.dtype == torch.bfloat16 and torch.allclose(got.float(), want, atol=2e-2, rtol=2e-2)
    got32 = o.linear(x, w, out_dtype=torch.float32)
    assert got32.dtype == torch.float32 and torch.allclose(got32, want, atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("M", [1, 8, 11, 64])
@pytest.mark.parametrize("F,K", [(192, 64), (256, 96), (4608, 1024), (100, 1000)])
def test_skinny_gemm_swiglu(M, F, K):
    o = ops()
    g = torch.Generator().manual_seed(21)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(2 * F, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    gu = x.float() @ w.float().t()
    want = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    got = o.linear_swiglu(x, w, F)
    assert got.shape == (M, F) and torch.allclose(got.float(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M", [2, 9, 16, 17, 33, 64])
@pytest.mark.parametrize("F,K,eps", [(4608, 1024, 1e-5), (100, 1000, 1e-3), (192, 64, 1e-6), (1536, 256, 1e-5)])
def test_norm_and_swiglu(M, F, K, eps):
    """Residual addition, norm, the gate/up product and SwiGLU: one kernel up to 16 rows, the norm
    kernel, the library's product and the activation kernel beyond."""
    o = ops()
    g = torch.Generator().manual_seed(24)
    h = (torch.randn(M, K, generator=g) * 3).cuda()
    delta = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    gamma = (1 + 0.1 * torch.randn(K, generator=g)).cuda()
    w = (torch.randn(2 * F, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    hsum = h + delta.float()
    xn = (hsum * torch.rsqrt((hsum * hsum).mean(-1, keepdim=True) + eps) * gamma).to(torch.bfloat16)
    gu = xn.float() @ w.float().t()
    want = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    lazy = _lazy(h.clone(), delta, gamma, eps)
    before = o.launches
    got = o.linear_swiglu(lazy, w, F)
    assert o.launches == before + (1 if M <= 16 else 2)        # (the library's product is not counted)
    assert got.shape == (M, F) and torch.allclose(got.float(), want, atol=3e-2, rtol=3e-2)
    assert torch.equal(lazy.residual.data, hsum)


@pytest.mark.parametrize("M", [1, 5, 8, 24, 64])
@pytest.mark.parametrize("O,K,eps", [(3072, 1024, 1e-5), (288, 96, 1e-6), (517, 1000, 1e-3)])
def test_skinny_gemm_with_norm_residual_and_gathered_rows(M, O, K, eps):
    o = ops()
    g = torch.Generator().manual_seed(22)
    h = (torch.randn(M, K, generator=g) * 3).cuda()
    delta = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    gamma = (1 + 0.1 * torch.randn(K, generator=g)).cuda()
    w = (torch.randn(O, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    hsum = h + delta.float()
    xn = (hsum * torch.rsqrt((hsum * hsum).mean(-1, keepdim=True) + eps) * gamma).to(torch.bfloat16)
    want = xn.float() @ w.float().t()
    lazy = _lazy(h.clone(), delta, gamma, eps)
    old = lazy.residual.data
    got = o.linear(lazy, w)
    assert torch.allclose(got.float(), want, atol=3e-2, rtol=3e-2)
    assert torch.equal(lazy.residual.data, hsum)                                      # the new residual stream
    if M <= 16:                                                                       # the fused kernel: a fresh buffer,
        assert lazy.residual.data is not old and torch.equal(old, h)                  # the old one is untouched
    # without a pending term the stream stays where it is
    lazy = _lazy(h.clone(), None, gamma, eps)
    old = lazy.residual.data
    xn0 = (h * torch.rsqrt((h * h).mean(-1, keepdim=True) + eps) * gamma).to(torch.bfloat16)
    assert torch.allclose(o.linear(lazy, w).float(), xn0.float() @ w.float().t(), atol=3e-2, rtol=3e-2)
    assert lazy.residual.data is old
    # gathered rows, 32-bit result (the head)
    rows = torch.tensor([M - 1, 0, M // 2][:min(3, M)], dtype=torch.int32).cuda()
    lazy = _lazy(h.clone(), delta, gamma, eps, rows)
    got = o.linear(lazy, w, out_dtype=torch.float32)
    assert got.dtype == torch.float32 and torch.allclose(got, want[rows.long()], atol=3e-2, rtol=3e-2)
    assert torch.equal(lazy.residual.data, h)


@pytest.mark.parametrize("M", [1, 5, 8, 13, 16])
@pytest.mark.parametrize("C,K,taps,bias,norm", [(1024, 1024, 3, False, True), (96, 96, 3, True, True), (100, 64, 4, True, False),
                                                (517, 1000, 2, False, True), (72, 40, 1, True, False)])
def test_projection_with_short_conv_epilogue(M, C, K, taps, bias, norm):
    """The short convolution's input projection with gates, taps and state update as its epilogue,
    against the product followed by the plain convolution; the slots of the rows are not in order and
    one state row more than needed is kept; with and without writing the state back."""
    o = ops()
    g = torch.Generator().manual_seed(23)
    w_in = (torch.randn(3 * C, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    conv_w = torch.randn(C, taps, generator=g).cuda()
    conv_b = torch.randn(C, generator=g).cuda() if bias else None
    slots = [3 * i + 2 for i in range(M)]
    slots.reverse()
    state0 = torch.randn(3 * M + 4, taps, C, generator=g).cuda()
    step = make_step(o, torch.bfloat16, [7 + i for i in range(M)], [1] * M, 16, 64, 24, slots=slots)
    h = (torch.randn(M, K, generator=g) * 2).cuda()
    delta = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    gamma = (1 + 0.1 * torch.randn(K, generator=g)).cuda()
    xb = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    for write in (False, True):
        # the projections with the kernel's own rounding points: x = bf16((h + delta) gamma), the row's
        # 1/rms applied to the 32-bit sums, B, C and x~ rounded to bfloat16 as when they are stored
        if norm:
            hsum = h + delta.float()
            xin = (hsum * gamma).to(torch.bfloat16)
            inv = torch.rsqrt((hsum * hsum).mean(-1, keepdim=True) + 1e-5)
        else:
            xin, inv = xb, 1.0
        bcx = ((xin.float() @ w_in.float().t()) * inv).to(torch.bfloat16)
        st_want = state0.clone()
        want = ref_ops.short_conv(bcx, conv_w, conv_b, st_want, step, taps, write)
        # the size of what is summed (the sum itself may cancel): |C| (|b| + sum |w_j s_j| + |w_last B x~|)
        Bf, Cf, Xf = bcx[:, :C].float(), bcx[:, C:2 * C].float(), bcx[:, 2 * C:].float()
        hist = state0[torch.tensor(slots, device="cuda")][:, :taps - 1]                       # [M, taps-1, C]
        size = (hist * conv_w.t()[None, :taps - 1]).abs().sum(1) + (conv_w[:, taps - 1][None] * Bf * Xf).abs()
        if bias:
            size = size + conv_b.abs()[None]
        size = Cf.abs() * size
        st_got = state0.clone()
        lazy = _lazy(h.clone(), delta, gamma, 1e-5) if norm else None
        before = o.launches
        got = o.linear_short_conv(lazy if norm else xb, w_in, conv_w, conv_b, st_got, step, taps, write)
        assert o.launches == before + 1                    # one kernel
        # B, C, x~ and z are each rounded to bfloat16 from 32-bit sums that may differ in their last
        # bits (another order of summation): a few steps of 2^-8 of what is summed
        assert ((got.float() - want.float()).abs() <= 2 ** -6 * size + 1e-3).all()
        assert torch.allclose(st_got, st_want, atol=1e-3, rtol=2 ** -6)
        if not write:
            assert torch.equal(st_got, state0)
        if norm:
            assert torch.equal(lazy.residual.data, h + delta.float())


# ----------------------------------------------------------------------------- many-rows products (tcgen05)
def _tc_call(o, y, w, x, epilogue):
    import ctypes
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    fn = o._fn("gemm_tc", "zai_gemm_tc")
    code = fn(y.data_ptr(), w.data_ptr(), x.data_ptr(), status.data_ptr(), x.shape[0], w.shape[0], w.shape[1], epilogue,
              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert code == 0 and int(status.item()) == 0, (code, int(status.item()))


def _pair_call(o, y, w, x, epilogue, wide):
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    fn = o._fn("gemm_tc_pair", "zai_gemm_pair")
    code = fn(y.data_ptr(), w.data_ptr(), x.data_ptr(), status.data_ptr(), x.shape[0], w.shape[0], w.shape[1], epilogue,
              wide, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert code == 0 and int(status.item()) == 0, (code, int(status.item()))


@pytest.mark.parametrize("wide", [1, 0, -1])
@pytest.mark.parametrize("N,O,K", [(256, 256, 64), (128, 128, 64), (512, 512, 1024), (300, 517, 1000), (2048, 1024, 1024),
                                   (1000, 3072, 1024), (129, 96, 96), (4096, 256, 136), (640, 1536, 4608),
                                   (5000, 2048, 512)])
def test_two_block_tensor_core_gemm_bf16_and_f32(N, O, K, wide):
    """The product whose tiles span two blocks: tiles that end inside the matrix in every direction
    (also a pair whose second block has no token at all), K that is no multiple of 64, more tiles
    than pairs, few tiles, both tile widths.  The inputs differ by token and by weight row, so a
    half of a tile that landed in the wrong block's rows or columns shows."""
    o = ops()
    g = torch.Generator().manual_seed(33)
    x = torch.randn(N, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(O, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    want = x.float() @ w.float().t()
    y = torch.full((N, O), float("nan"), dtype=torch.bfloat16, device="cuda")
    _pair_call(o, y, w, x, 0, wide)
    assert torch.allclose(y.float(), want, atol=2e-2, rtol=2e-2)
    y32 = torch.full((N, O), float("nan"), dtype=torch.float32, device="cuda")
    _pair_call(o, y32, w, x, 1, wide)
    assert torch.allclose(y32, want, atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("wide", [1, 0])
@pytest.mark.parametrize("N,F,K", [(256, 128, 64), (2048, 4608, 1024), (130, 100, 96), (700, 1000, 520), (3000, 1536, 256)])
def test_two_block_tensor_core_gemm_swiglu(N, F, K, wide):
    o = ops()
    g = torch.Generator().manual_seed(34)
    x = torch.randn(N, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(2 * F, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    gu = x.float() @ w.float().t()
    want = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    y = torch.full((N, F), float("nan"), dtype=torch.bfloat16, device="cuda")
    _pair_call(o, y, w, x, 2, wide)
    assert torch.allclose(y.float(), want, atol=3e-2, rtol=3e-2)
    if wide and N >= o.PAIR_SWIGLU_MIN_ROWS:
        # and through the op the parts call, with the switch that sends gate/up products to this kernel
        old, o.USE_PAIR_GEMM, o.PAIR_GEMM_ALWAYS = (o.USE_PAIR_GEMM, o.PAIR_GEMM_ALWAYS), True, True
        try:
            before = o.launches
            got = o.linear_swiglu(x, w, F)
            assert o.launches == before + 1 and torch.allclose(got.float(), want, atol=3e-2, rtol=3e-2)
        finally:
            o.USE_PAIR_GEMM, o.PAIR_GEMM_ALWAYS = old
        assert o.tc_status() == 0


@pytest.mark.parametrize("N,O,K", [(128, 128, 64), (256, 256, 1024), (300, 517, 1000), (2048, 1024, 1024),
                                   (1000, 3072, 1024), (129, 96, 96), (4096, 256, 136), (640, 1536, 4608)])
def test_tensor_core_gemm_bf16_and_f32(N, O, K):
    """Tiles that end inside the matrix in every direction, K that is no multiple of 64, more tiles
    than blocks (a block takes several), few tiles."""
    o = ops()
    g = torch.Generator().manual_seed(30)
    x = torch.randn(N, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(O, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    want = x.float() @ w.float().t()
    y = torch.full((N, O), float("nan"), dtype=torch.bfloat16, device="cuda")
    _tc_call(o, y, w, x, 0)
    assert torch.allclose(y.float(), want, atol=2e-2, rtol=2e-2)
    y32 = torch.full((N, O), float("nan"), dtype=torch.float32, device="cuda")
    _tc_call(o, y32, w, x, 1)
    assert torch.allclose(y32, want, atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("N,F,K", [(128, 128, 64), (2048, 4608, 1024), (130, 100, 96), (700, 1000, 520)])
def test_tensor_core_gemm_swiglu(N, F, K):
    o = ops()
    g = torch.Generator().manual_seed(31)
    x = torch.randn(N, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(2 * F, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    gu = x.float() @ w.float().t()
    want = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    y = torch.full((N, F), float("nan"), dtype=torch.bfloat16, device="cuda")
    _tc_call(o, y, w, x, 2)
    assert torch.allclose(y.float(), want, atol=3e-2, rtol=3e-2)
    # and through the op the parts call, with the switch that sends products to this kernel
    old, o.USE_TC_GEMM = o.USE_TC_GEMM, True
    try:
        before = o.launches
        got = o.linear_swiglu(x, w, F)
        assert o.launches == before + 1 and torch.allclose(got.float(), want, atol=3e-2, rtol=3e-2)
        assert torch.allclose(o.linear(x, w).float(), gu, atol=3e-2, rtol=3e-2)
    finally:
        o.USE_TC_GEMM = old
    assert o.tc_status() == 0


@pytest.mark.parametrize("Hq,Hkv,D,ps,window,rot,qk_norm", [
    (4, 2, 16, 16, None, 16, True), (3, 1, 32, 8, None, 32, True), (6, 3, 48, 4, 7, 24, False),
    (8, 2, 80, 32, None, 80, True), (16, 8, 64, 16, None, 64, True), (2, 2, 128, 16, 40, 64, True), (32, 2, 96, 16, None, 96, True),
    (4, 1, 64, 8, None, 64, True), (6, 2, 64, 32, 300, 32, False), (16, 1, 64, 64, None, 64, True)])
@pytest.mark.parametrize("tma", [True, False])
def test_fused_decode_attention(Hq, Hkv, D, ps, window, rot, qk_norm, tma):
    """The one-kernel decode attention against the plain versions of its three steps, at contexts of
    0 keys, around the chunk size of 256, several chunks, and with more chunks launched than needed;
    run twice on the same buffers (the ticket counters must come back to zero)."""
    o = ops()
    o.USE_TMA_ATTENTION = tma          # (head size 64 and pages of 8..64 positions go through TMA; the rest does not)
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(40)
    ctx = [0, 1, 254, 255, 256, 257, 700, 63, 1029]
    B = len(ctx)
    num_pages = 1024
    step = make_step(o, dtype, ctx, [1] * B, ps, num_pages, 41)
    pages_a = fill_pages(step, ctx, [0] * B, ps, Hkv, D, dtype, num_pages, g)     # the cached keys only
    pages_b = pages_a.clone()
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, generator=g).to(dtype).cuda()
    qw = (1 + 0.1 * torch.randn(D, generator=g)).cuda() if qk_norm else None
    kw = (1 + 0.1 * torch.randn(D, generator=g)).cuda() if qk_norm else None
    va, vb = CacheView(0, pages_a, step.block_tables[0], ps), CacheView(0, pages_b, step.block_tables[0], ps)
    qb, _ = ref_ops.qk_norm_rope(qkv, qw, kw, 1e-5, rot, 10000.0, step, vb, Hq, Hkv, D, True, True, False)
    want = ref_ops.paged_attention(qb, step, vb, Hq, Hkv, D, D ** -0.5, window)
    for max_kv in (step.max_kv_len, 3000):
        step.max_kv_len = max_kv
        pa = pages_a.clone()
        got = o.decode_attention_fused(qkv, qw, kw, 1e-5, rot, 10000.0, step, CacheView(0, pa, step.block_tables[0], ps),
                                       Hq, Hkv, D, D ** -0.5, window, True)
        assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2), max_kv
        assert torch.allclose(pa.float(), pages_b.float(), atol=2e-2, rtol=2e-2)       # the new keys and values
        assert torch.equal(pa[0], pages_a[0])                                          # the null page was not written
    # reading only (a layer that uses another layer's cache): the pages already hold the new position
    got = o.decode_attention_fused(qkv, qw, kw, 1e-5, rot, 10000.0, step, vb, Hq, Hkv, D, D ** -0.5, window, False)
    assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2)
    o.USE_TMA_ATTENTION = True
    assert o.tc_status() == 0


@pytest.mark.parametrize("ps", [16, 64])
def test_tma_decode_attention_long_contexts_repeat(ps):
    """Contexts of thousands of keys, so that every block's ring of stages goes round many times, on
    a pool larger than L2 so that loads land late and out of order; repeated launches must give the
    same bits each time, agree with the kernel that loads with plain copies, and never give up a wait."""
    o = ops()
    dtype = torch.bfloat16
    Hq, Hkv, D = 16, 8, 64
    g = torch.Generator().manual_seed(52)
    ctx = [4000 - 37 * i for i in range(32)]
    B = len(ctx)
    num_pages = (B * 4096) // ps + 1
    step = make_step(o, dtype, ctx, [1] * B, ps, num_pages, 53)
    pages = fill_pages(step, ctx, [0] * B, ps, Hkv, D, dtype, num_pages, g)
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, generator=g).to(dtype).cuda()
    qw = (1 + 0.1 * torch.randn(D, generator=g)).cuda()
    kw = (1 + 0.1 * torch.randn(D, generator=g)).cuda()
    view = CacheView(0, pages, step.block_tables[0], ps)
    step.max_kv_len = 4096
    o.USE_TMA_ATTENTION = False
    want = o.decode_attention_fused(qkv, qw, kw, 1e-5, D, 10000.0, step, view, Hq, Hkv, D, D ** -0.5, None, True)
    o.USE_TMA_ATTENTION = True
    flush = torch.empty(160 * 2 ** 20, dtype=torch.uint8, device="cuda")
    first = None
    for rep in range(40):
        flush.fill_(rep)
        got = o.decode_attention_fused(qkv, qw, kw, 1e-5, D, 10000.0, step, view, Hq, Hkv, D, D ** -0.5, None, True)
        if first is None:
            first = got.clone()
            assert torch.allclose(got.float(), want.float(), atol=2e-3, rtol=2e-2)
        assert torch.equal(got, first), rep
    assert o.tc_status() == 0


# ----------------------------------------------------------------------------- ids outside their bounds
def test_ids_outside_their_bounds_raise_the_status_word_and_touch_nothing():
    """Every kernel that indexes by page, slot, position or token id is told a pool four pages (a state
    two slots) smaller than the tensor that was really allocated, and is given an id in the part it was
    not told of: it must use id 0 instead, leave the part beyond its bound as it was, and raise the
    matching bit of the status word.  (Not even a missed check would touch foreign memory here.)"""
    o = ops()
    dtype, Hq, Hkv, D, ps = torch.bfloat16, 4, 2, 64, 16
    g = torch.Generator().manual_seed(90)
    num_pages, told = 40, 36
    assert o.read_status() == 0

    def fresh(q_lens, ctx):
        step = make_step(o, dtype, ctx, q_lens, ps, told, 91)            # tables from pages 1..35
        pages = fill_pages(step, ctx, q_lens, ps, Hkv, D, dtype, num_pages, g, junk=0.0)
        return step, pages

    # --- pages: spans (page write, the three span attention kernels), then single tokens
    for q_lens, ctx in (([20, 3], [5, 40]), ([1, 1, 1], [30, 70, 5])):
        step, pages = fresh(q_lens, ctx)
        N = sum(q_lens)
        bad = step.block_tables[0].clone()
        bad[1, 0] = told + 2                                             # allocated, but beyond what the kernels are told
        beyond = pages[told:].clone()
        view = CacheView(0, pages[:told], bad, ps)
        qkv = torch.randn(N, (Hq + 2 * Hkv) * D, generator=g).to(dtype).cuda()
        q = qkv[:, :Hq * D].contiguous()
        w = torch.ones(D, device="cuda")
        calls = [lambda: o.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, None, impl="general")]
        if step.decode_only:
            calls += [lambda: o.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, None)]
            for tma in (True, False):
                def fused(tma=tma):
                    old, o.USE_TMA_ATTENTION = o.USE_TMA_ATTENTION, tma
                    try:
                        o.decode_attention_fused(qkv, w, w, 1e-5, D, 1e4, step, view, Hq, Hkv, D, D ** -0.5, None, True)
                    finally:
                        o.USE_TMA_ATTENTION = old
                calls.append(fused)
        else:
            calls += [lambda: o.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, None, impl="mma"),
                      lambda: o.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, None, impl="tcgen05")]
        def run(which):
            for i, call in enumerate(which):
                call()
                assert o.read_status() == 4, (q_lens, i)
                assert torch.equal(pages[told:], beyond), (q_lens, i)

        run(calls)                                                       # kernels that read the request's first page
        bad[1, 0] = int(step.block_tables[0][1, 0])
        bad[1, ctx[1] // ps] = told + 1                                  # the page the request's new rows are written to
        run([lambda: o.qk_norm_rope(qkv, w, w, 1e-5, D, 1e4, step, view, Hq, Hkv, D, True, True, False),
             lambda: o.kv_write(qkv[:, Hq * D:(Hq + Hkv) * D], qkv[:, (Hq + Hkv) * D:], step, view, Hkv, D)])
        # --- positions: a table row narrower than the request's positions
        narrow = CacheView(0, pages[:told], step.block_tables[0][:, :1].contiguous(), ps)
        o.qk_norm_rope(qkv, w, w, 1e-5, D, 1e4, step, narrow, Hq, Hkv, D, True, True, False)
        assert o.read_status() & 16
        o.paged_attention(q, step, narrow, Hq, Hkv, D, D ** -0.5, None, impl="general")
        assert o.read_status() & 16
    # --- slots
    C, L = 64, 3
    conv_w = torch.randn(C, L, generator=g).cuda()
    state = torch.randn(8, L - 1, C, generator=g).cuda()
    for q_lens in ([1, 1, 1], [4, 1, 6]):
        step = make_step(o, dtype, [3] * 3, q_lens, ps, told, 92, slots=[1, 7, 2])        # slot 7 is beyond the six it is told
        bcx = torch.randn(sum(q_lens), 3 * C, generator=g).to(dtype).cuda()
        keep = state[6:].clone()
        o.short_conv(bcx, conv_w, None, state[:6], step, L, True)
        assert o.read_status() == 8 and torch.equal(state[6:], keep)
    step = make_step(o, dtype, [3] * 3, [1, 1, 1], ps, told, 92, slots=[1, 7, 2])
    K = 128
    x = torch.randn(3, K, generator=g).to(dtype).cuda()
    w_in = (torch.randn(3 * C, K, generator=g) * K ** -0.5).to(dtype).cuda()
    before = o.launches
    o.linear_short_conv(x, w_in, conv_w, None, state[:6], step, L, True)                # the product's convolution epilogue
    assert o.read_status() == 8 and torch.equal(state[6:], keep)
    # --- token ids
    table = torch.randn(50, 32, generator=g).to(dtype).cuda()
    out = o.embed(torch.tensor([3, 50, -1, 49], dtype=torch.int32).cuda(), table)
    assert o.read_status() == 2 and torch.equal(out[1], table[0].float()) and torch.equal(out[3], table[49].float())
    # --- and the word is what the step function reads: a raised bit voids the step
    o.status_tensor().fill_(1)
    assert o.tc_status() == 1 and o.read_status() == 0


# ----------------------------------------------------------------------------- 17 to 128 rows: the weight-streaming products
@pytest.fixture
def stream_gemm_on():
    """The ops send products of 17 to 128 rows to the weight-streaming kernel (an option, off by default)."""
    from zig_ai_b200.kernels import ops as o
    old, o.USE_STREAM_GEMM = o.USE_STREAM_GEMM, True
    yield
    o.USE_STREAM_GEMM = old


def _stream_call(o, y, w, x, epilogue):
    fn = o._fn("stream_gemm", "zai_stream_gemm")
    code = fn(y.data_ptr(), w.data_ptr(), x.data_ptr(), o.status_tensor().data_ptr(), x.shape[0], w.shape[0], w.shape[1], epilogue,
              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert code == 0 and o.read_status() == 0, code


@pytest.mark.parametrize("rows,ksplit", [(0, 0), (128, 1), (64, 2), (8, 8), (16, 4), (32, 1)])
@pytest.mark.parametrize("N,O,K", [(17, 128, 64), (64, 1024, 1024), (33, 517, 1000), (128, 1024, 4608), (100, 3072, 1024),
                                   (24, 96, 96), (65, 256, 136), (32, 65536, 1024), (1, 300, 72), (64, 2048, 1536)])
def test_stream_gemm_bf16_and_f32(N, O, K, rows, ksplit, stream_gemm_on):
    """Tiles that end inside the matrix in every direction, K that is no multiple of 64, one 64-k slice
    only, tiles of 8 to 128 weight rows, K cut across clusters of every size (`rows`, `ksplit`: asked
    for; 0 leaves the choice to the launcher) and more blocks in a cluster than slices."""
    o = ops()
    o._fn("stream_gemm", "zai_stream_force_cluster")(ksplit)
    o._fn("stream_gemm", "zai_stream_force_rows")(rows)
    g = torch.Generator().manual_seed(70)
    x = torch.randn(N, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(O, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    want = x.float() @ w.float().t()
    y = torch.full((N, O), float("nan"), dtype=torch.bfloat16, device="cuda")
    _stream_call(o, y, w, x, 0)
    assert torch.allclose(y.float(), want, atol=2e-2, rtol=2e-2)
    y32 = torch.full((N, O), float("nan"), dtype=torch.float32, device="cuda")
    _stream_call(o, y32, w, x, 1)
    assert torch.allclose(y32, want, atol=2e-3, rtol=2e-3)
    o._fn("stream_gemm", "zai_stream_force_cluster")(0)
    o._fn("stream_gemm", "zai_stream_force_rows")(0)
    if 17 <= N:
        before = o.launches
        assert torch.allclose(o.linear(x, w).float(), want, atol=2e-2, rtol=2e-2) and o.launches == before + 1


@pytest.mark.parametrize("rows", [0, 64, 8])
@pytest.mark.parametrize("N,F,K", [(17, 64, 64), (64, 4608, 1024), (40, 100, 96), (128, 1000, 520), (96, 8192, 2048)])
def test_stream_gemm_swiglu(N, F, K, rows, stream_gemm_on):
    o = ops()
    o._fn("stream_gemm", "zai_stream_force_rows")(rows)
    g = torch.Generator().manual_seed(71)
    x = torch.randn(N, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(2 * F, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    gu = x.float() @ w.float().t()
    want = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    y = torch.full((N, F), float("nan"), dtype=torch.bfloat16, device="cuda")
    _stream_call(o, y, w, x, 2)
    o._fn("stream_gemm", "zai_stream_force_rows")(0)
    assert torch.allclose(y.float(), want, atol=3e-2, rtol=3e-2)
    before = o.launches
    assert torch.allclose(o.linear_swiglu(x, w, F).float(), want, atol=3e-2, rtol=3e-2) and o.launches == before + 1


@pytest.mark.parametrize("rows", [0, 32, 8])
@pytest.mark.parametrize("M,C,K,L,bias", [(17, 64, 128, 3, False), (64, 1024, 1024, 3, False), (40, 200, 96, 4, True),
                                          (128, 96, 520, 2, True), (33, 48, 64, 1, False), (100, 2048, 2048, 3, False)])
def test_stream_gemm_short_conv_epilogue(M, C, K, L, bias, rows, stream_gemm_on):
    """The short convolution as the input projection's epilogue for 17 to 128 single tokens: against the
    plain product followed by the plain convolution, twice in a row (the state moves on), with slots in
    another order than the rows, and once without writing the state."""
    o = ops()
    g = torch.Generator().manual_seed(72)
    w_in = (torch.randn(3 * C, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    conv_w = (torch.randn(C, L, generator=g) * 0.3).cuda()
    conv_b = (torch.randn(C, generator=g) * 0.3).cuda() if bias else None
    rows = max(L - 1, 1)
    slots = list(range(1, M + 1))
    random.Random(73).shuffle(slots)
    state_a = torch.randn(M + 3, rows, C, generator=g).cuda()
    state_b = state_a.clone()
    step = make_step(o, torch.bfloat16, [3] * M, [1] * M, 16, 2 * M + 2, 74, slots=slots)
    o._fn("stream_gemm", "zai_stream_force_rows")(rows)
    for rep, write in enumerate((True, True, False)):
        x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
        before = o.launches
        za = o.linear_short_conv(x, w_in, conv_w, conv_b, state_a, step, L, write)
        assert o.launches == before + 1
        bcx = (x.float() @ w_in.float().t()).to(torch.bfloat16)
        zb = ref_ops.short_conv(bcx, conv_w, conv_b, state_b, step, L, write)
        assert torch.allclose(za.float(), zb.float(), atol=3e-2, rtol=3e-2), rep
        assert torch.allclose(state_a, state_b, atol=2e-2, rtol=2e-2), rep
    o._fn("stream_gemm", "zai_stream_force_rows")(0)
    assert torch.equal(state_a[0], state_b[0]) and o.read_status() == 0


@pytest.mark.parametrize("Hq,Hkv,D,ps,qk_norm", [(16, 8, 64, 64, True), (4, 2, 16, 16, True), (3, 1, 32, 8, False), (2, 1, 128, 16, True),
                                                  (3, 3, 256, 8, True)])
def test_qk_norm_rope_many_rows(Hq, Hkv, D, ps, qk_norm):
    """From 256 rows on the bfloat16 kernel works with 16-byte accesses: spans of hundreds of rows that
    start inside pages, against the plain version, pages included."""
    o = ops()
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(16)
    ctx, q_lens = [0, ps - 1, 3 * ps, 100], [300, 2, 1, 45]
    num_pages = sum(-(-(c + n) // ps) for c, n in zip(ctx, q_lens)) + 4
    step = make_step(o, dtype, ctx, q_lens, ps, num_pages, 17)
    N = sum(q_lens)
    qkv = torch.randn(N, (Hq + 2 * Hkv) * D, generator=g).to(dtype).cuda()
    qw = (1 + 0.1 * torch.randn(D, generator=g)).cuda() if qk_norm else None
    kw = (1 + 0.1 * torch.randn(D, generator=g)).cuda() if qk_norm else None
    pages_a = torch.zeros(num_pages, 2, Hkv, ps, D, dtype=dtype, device="cuda")
    pages_b = pages_a.clone()
    va, vb = CacheView(0, pages_a, step.block_tables[0], ps), CacheView(0, pages_b, step.block_tables[0], ps)
    qa, ka = o.qk_norm_rope(qkv, qw, kw, 1e-5, D, 10000.0, step, va, Hq, Hkv, D, True, True, True)
    qb, kb = ref_ops.qk_norm_rope(qkv, qw, kw, 1e-5, D, 10000.0, step, vb, Hq, Hkv, D, True, True, True)
    assert torch.allclose(qa.float(), qb.float(), **tol(dtype))
    assert torch.allclose(ka.float(), kb.float(), **tol(dtype))
    assert torch.allclose(pages_a.float(), pages_b.float(), **tol(dtype))
    assert pages_a[0].abs().sum() == 0 and o.read_status() == 0
