"""The attention kernels at the sizes the benchmark runs, each directly against the plain PyTorch version
(tests/ref_ops.py): one span of 2048 rows from an empty cache and one of 512 rows behind 3584 cached
positions for the two span kernels, and a batch of 64 single tokens at contexts of 2048..4095 for the
decode kernels (keys by TMA and by plain copies).

Random keys hide a dropped or an extra key among thousands (one key moves the output by 1e-3), so in
every case keys are planted that must decide the output if they are seen and must not if they are
not: a key aligned with the query (score about +24, every other score is about N(0, 1)) with a value
of its own, at the first and the last visible position, on both sides of every boundary the kernels
have (pages, tiles of 64 and 128 keys, chunks of 256 to 1024 keys, the window's edge), one per
request or per group of query rows.  Everything that no request owns holds a large finite value.

The operator: src/transformer/hybrid_attn.zig:571-609, src/cuda/paged_attention.cu:121-337.
"""
import pytest
import torch

import ref_ops
from test_gpu_kernels import fill_pages, make_step, ops, plant_key
from zig_ai_b200.cache.manager import CacheView

pytestmark = pytest.mark.gpu

Hq, Hkv, D = 16, 8, 64
G = Hq // Hkv
BF16 = torch.bfloat16


def distinct_value(i):
    """A value row that no average of random rows resembles: +-6 in a pattern of its own."""
    bits = torch.tensor([(i * 2654435761 >> d) & 1 for d in range(D)], dtype=torch.float32)
    return bits * 12.0 - 6.0


def boundaries(last, ps, window=None):
    """Positions on both sides of the kernels' boundaries that a query at position `last` may see."""
    cand = {0, 1, last, last - 1}
    for step in {ps, 64, 128, 256, 512, 1024}:
        for m in (1, 2, (last // step), (last // step) - 1):
            for d in (-1, 0):
                cand.add(m * step + d)
    lo = 0 if window is None else max(last - window + 1, 0)
    if window is not None:
        cand |= {lo, lo + 1}
    return sorted(p for p in cand if lo <= p <= last)


@pytest.mark.parametrize("impl", ["tcgen05", "mma"])
@pytest.mark.parametrize("ctx,q_len,ps,window", [(0, 2048, 64, None), (3584, 512, 64, None), (3584, 512, 16, 1000),
                                                  (1000, 700, 32, None)])
def test_span_attention_at_the_benchmark_sizes(impl, ctx, q_len, ps, window):
    o = ops()
    g = torch.Generator().manual_seed(61)
    num_pages = (ctx + q_len) // ps + 8
    step = make_step(o, BF16, [ctx], [q_len], ps, num_pages, 62)
    pages = fill_pages(step, [ctx], [q_len], ps, Hkv, D, BF16, num_pages, g)
    q = torch.randn(q_len, Hq * D, generator=g).to(BF16).cuda()
    # query row r (position ctx + r) of query head h = r % Hq: a key planted at one of the boundaries
    # that row can see, aligned with that row's query of that head
    planted = set()
    for r in range(0, q_len, max(q_len // 97, 1)):
        last = ctx + r
        cands = boundaries(last, ps, window)
        pos = cands[(r * 7) % len(cands)]
        h = r % Hq
        if (pos, h // G) in planted:
            continue
        planted.add((pos, h // G))
        plant_key(pages, step, ps, 0, pos, h // G, q[r, h * D:(h + 1) * D].float() * 3.0, distinct_value(r))
    view = CacheView(0, pages, step.block_tables[0], ps)
    got = o.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, window, impl=impl)
    want = ref_ops.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, window)
    assert want.float().abs().max() > 5.0                        # the planted values decide some rows
    assert torch.allclose(got.float(), want.float(), atol=3e-2, rtol=3e-2), (got.float() - want.float()).abs().max()
    assert o.read_status() == 0


@pytest.mark.parametrize("ps,window,padded", [(64, None, 0), (16, None, 3), (128, 5000, 0), (32, 700, 1)])
def test_span_attention_few_rows_over_long_contexts(ps, window, padded):
    """Few tiles of query rows over long contexts: several blocks share a tile's keys, leave their parts in
    scratch, and the one with the last ticket combines them.  Requests of 40 rows behind 16 000 positions
    (every block has keys), 3 rows behind 5 (all blocks but one have none), 130 rows behind 700 and 1 row
    behind 9000; a planted key on both sides of the boundaries between the blocks' shares; twice in a row
    (the tickets must be zero again), and with more tiles launched than the step has (a captured graph's
    grid is sized for its bucket)."""
    o = ops()
    from zig_ai_b200.kernels import ops as ops_module
    g = torch.Generator().manual_seed(71)
    ctx, q_lens = [16000, 5, 700, 9000], [40, 3, 130, 1]
    num_pages = sum(-(-(c + n) // ps) for c, n in zip(ctx, q_lens)) + 8
    step = make_step(o, BF16, ctx, q_lens, ps, num_pages, 72)
    pages = fill_pages(step, ctx, q_lens, ps, Hkv, D, BF16, num_pages, g)
    q = torch.randn(sum(q_lens), Hq * D, generator=g).to(BF16).cuda()
    n_tiles = sum(-(-n // 128) for n in q_lens)
    lib_splits = ops_module._fn("attention_tc", "zai_prefill_attention_tc_splits")(n_tiles + padded, Hq, step.block_tables[0].shape[1], ps)
    assert lib_splits > 1                                            # the case is one the shared tiles are made for
    key_tiles = -(-(ctx[0] + q_lens[0]) // 64)
    per = -(-key_tiles // lib_splits)
    starts = [0] + q_lens[:-1]
    row_of = [sum(q_lens[:i]) for i in range(len(q_lens))]
    planted = set()
    # request 0: one key per share boundary (last key of a share, first key of the next), seen by different rows and heads
    for z in range(1, lib_splits):
        for d, r in ((-1, (2 * z) % q_lens[0]), (0, (2 * z + 1) % q_lens[0])):
            pos = z * per * 64 + d
            if window is not None and pos < ctx[0] + r - window + 1:
                continue
            h = (z + d) % Hq
            if (pos, h // G) in planted:
                continue
            planted.add((pos, h // G))
            plant_key(pages, step, ps, 0, pos, h // G, q[row_of[0] + r, h * D:(h + 1) * D].float() * 3.0, distinct_value(z * 2 + d + 1))
    # the other requests: their first and last visible keys
    for s_i in (1, 2, 3):
        r = q_lens[s_i] - 1
        last = ctx[s_i] + r
        lo = 0 if window is None else max(last - window + 1, 0)
        for pos, h in ((lo, 1), (last, 2 + s_i)):
            plant_key(pages, step, ps, s_i, pos, h // G, q[row_of[s_i] + r, h * D:(h + 1) * D].float() * 3.0, distinct_value(40 + 2 * s_i + h))
    view = CacheView(0, pages, step.block_tables[0], ps)
    if padded:
        step.attn_tiles = n_tiles + padded
    want = ref_ops.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, window)
    assert want.float().abs().max() > 5.0
    for _ in range(2):
        got = o.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, window, impl="tcgen05")
        assert torch.allclose(got.float(), want.float(), atol=3e-2, rtol=3e-2), (got.float() - want.float()).abs().max()
        assert int(ops_module._span_tickets[q.device].abs().sum()) == 0
    assert o.read_status() == 0


@pytest.mark.parametrize("tma", [True, False])
@pytest.mark.parametrize("ps,window", [(64, None), (16, None), (64, 1500)])
def test_decode_attention_batch_64_at_contexts_2048_to_4095(tma, ps, window):
    o = ops()
    B = 64
    g = torch.Generator().manual_seed(63)
    ctx = [2048 + (i * 2047) // (B - 1) for i in range(B)]       # 2048 .. 4095
    ctx[5], ctx[6], ctx[7] = 2048 + 255, 2048 + 256, 4095 - 64
    num_pages = sum(-(-(c + 1) // ps) for c in ctx) + 8
    step = make_step(o, BF16, ctx, [1] * B, ps, num_pages, 64)
    pages = fill_pages(step, ctx, [0] * B, ps, Hkv, D, BF16, num_pages, g)
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, generator=g).to(BF16).cuda()
    qw = (1 + 0.1 * torch.randn(D, generator=g)).cuda()
    kw = (1 + 0.1 * torch.randn(D, generator=g)).cuda()
    table = step.block_tables[0]
    # the queries as the kernel will see them (normed and rotated), to aim the planted keys
    scratch = CacheView(0, pages.clone(), table, ps)
    q_ref, _ = ref_ops.qk_norm_rope(qkv, qw, kw, 1e-5, D, 1e6, step, scratch, Hq, Hkv, D, True, True, False)
    for b in range(B):
        cands = boundaries(ctx[b] - 1, ps, None if window is None else window - 1)   # cached positions the new token sees
        pos = cands[(b * 5) % len(cands)]
        h = b % Hq
        plant_key(pages, step, ps, b, pos, h // G, q_ref[b, h * D:(h + 1) * D].float() * 3.0, distinct_value(b))
        if window is not None:                                   # and one just outside the window: must not be seen
            out = ctx[b] - window
            plant_key(pages, step, ps, b, out, (h // G + 1) % Hkv, q_ref[b, ((h + G) % Hq) * D:((h + G) % Hq + 1) * D].float() * 3.0,
                      distinct_value(b + 100))
    pages_ref = pages.clone()
    view_ref = CacheView(0, pages_ref, table, ps)
    q_ref, _ = ref_ops.qk_norm_rope(qkv, qw, kw, 1e-5, D, 1e6, step, view_ref, Hq, Hkv, D, True, True, False)
    want = ref_ops.paged_attention(q_ref, step, view_ref, Hq, Hkv, D, D ** -0.5, window)
    assert want.float().abs().max() > 5.0
    step.max_kv_len = 4096
    old = o.USE_TMA_ATTENTION
    o.USE_TMA_ATTENTION = tma
    try:
        got = o.decode_attention_fused(qkv, qw, kw, 1e-5, D, 1e6, step, CacheView(0, pages, table, ps), Hq, Hkv, D, D ** -0.5,
                                       window, True)
    finally:
        o.USE_TMA_ATTENTION = old
    assert torch.allclose(got.float(), want.float(), atol=3e-2, rtol=3e-2), (got.float() - want.float()).abs().max()
    assert torch.allclose(pages.float(), pages_ref.float(), atol=2e-2, rtol=2e-2)      # the new keys and values, and nothing else
    assert o.read_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, BF16])
@pytest.mark.parametrize("heads,kv_heads,head_dim,ps,window", [(4, 2, 16, 16, None), (3, 1, 32, 8, 77), (6, 2, 80, 32, None),
                                                               (16, 8, 64, 16, 300), (2, 2, 128, 16, None)])
def test_planted_keys_at_every_edge_other_head_sizes(dtype, heads, kv_heads, head_dim, ps, window):
    """The same planting for the general kernel (32-bit) and the mma.sync kernels at other head sizes:
    spans and single tokens in one call each."""
    o = ops()
    g = torch.Generator().manual_seed(65)
    grp = heads // kv_heads
    for q_lens, ctx in (([1] * 6, [0, 63, 255, 256, 700, 1029]), ([150, 2, 37, 66], [0, 301, 5, 63])):
        num_pages = sum(-(-(c + n) // ps) for c, n in zip(ctx, q_lens)) + 4
        step = make_step(o, dtype, ctx, q_lens, ps, num_pages, 66)
        pages = fill_pages(step, ctx, q_lens, ps, kv_heads, head_dim, dtype, num_pages, g)
        q = torch.randn(sum(q_lens), heads * head_dim, generator=g).to(dtype).cuda()
        row0 = 0
        for s, (c, n) in enumerate(zip(ctx, q_lens)):
            seen = set()
            for i in range(0, n, max(n // 9, 1)):
                last = c + i
                cands = boundaries(last, ps, window)
                pos = cands[(i * 3 + s) % len(cands)]
                h = (i + s) % heads
                if (pos, h // grp) in seen:
                    continue
                seen.add((pos, h // grp))
                val = distinct_value(row0 + i)[:head_dim] if head_dim <= D else distinct_value(row0 + i).repeat(2)[:head_dim]
                plant_key(pages, step, ps, s, pos, h // grp, q[row0 + i, h * head_dim:(h + 1) * head_dim].float() * (24.0 / head_dim ** 0.5), val)
            row0 += n
        view = CacheView(0, pages, step.block_tables[0], ps)
        got = o.paged_attention(q, step, view, heads, kv_heads, head_dim, head_dim ** -0.5, window)
        want = ref_ops.paged_attention(q, step, view, heads, kv_heads, head_dim, head_dim ** -0.5, window)
        tol = dict(atol=2e-4, rtol=2e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
        assert want.float().abs().max() > 5.0
        assert torch.allclose(got.float(), want.float(), **tol), (q_lens, (got.float() - want.float()).abs().max())
