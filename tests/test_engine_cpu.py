"""The engine's host logic on the CPU: the step function, the cache and the batch description run
with the plain PyTorch kernels of tests/ref_ops.py in place of the CUDA kernels, and are compared
with the plain whole-sequence implementation under several ways of cutting the same requests."""
import random

import pytest
import torch

import plain_lfm2
import ref_ops
from tiny_configs import PAGE_SIZE
from zig_ai_b200.engine.runner import load_runner


def plain_logits(model_dir, tokens):
    c = plain_lfm2.read_config(model_dir)
    W = plain_lfm2.read_weights(model_dir)
    return plain_lfm2.forward(c, W, tokens)


def make_runner(model_dir, name, max_tokens=512):
    return load_runner(model_dir, "float32", max_tokens=max_tokens, max_requests=4,
                       page_size=PAGE_SIZE[name], device="cpu", ops=ref_ops)


def random_tokens(vocab, n, seed):
    g = random.Random(seed)
    return [g.randrange(vocab) for _ in range(n)]


@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_prompt_matches_plain(tiny_models, name):
    r = make_runner(tiny_models[name], name)
    toks = random_tokens(r.model.vocab_size, 37, 1)
    want = plain_logits(tiny_models[name], toks)
    r.add_request("a")
    got = r.step([("a", toks, list(range(len(toks))))])
    assert got.shape == want.shape
    assert torch.allclose(got.double(), want, atol=2e-4, rtol=0), (got.double() - want).abs().max()


@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_and_decode_match_plain(tiny_models, name):
    r = make_runner(tiny_models[name], name)
    toks = random_tokens(r.model.vocab_size, 61, 2)
    want = plain_logits(tiny_models[name], toks)
    r.add_request("a")
    cuts, g, left = [], random.Random(5), len(toks) - 12
    while left > 0:
        n = min(g.choice([2, 3, 5, 7, 11]), left)
        cuts.append(n)
        left -= n
    cuts += [1] * 12
    got, at = [], 0
    for n in cuts:
        got.append(r.step([("a", toks[at:at + n], list(range(n)))]))
        at += n
    got = torch.cat(got)
    assert torch.allclose(got.double(), want, atol=2e-4, rtol=0), (got.double() - want).abs().max()


@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_batches_with_page_reuse(tiny_models, name):
    ps = PAGE_SIZE[name]
    r = make_runner(tiny_models[name], name, max_tokens=6 * max(ps, 16))
    V = r.model.vocab_size
    g = random.Random(9)
    lengths = [23, 40, 9, 31, 17, 28]
    reqs = {f"r{i}": random_tokens(V, n, 100 + i) for i, n in enumerate(lengths)}
    want = {k: plain_logits(tiny_models[name], t) for k, t in reqs.items()}
    waiting = list(reqs)
    live, at, got = [], {}, {k: [] for k in reqs}
    budget_tokens = r.cache.num_pages * ps
    while waiting or live:
        # admit while fewer than three live and the pool can hold the whole request
        while waiting and len(live) < 3:
            k = waiting[0]
            held = sum(-(-len(reqs[x]) // ps) * ps for x in live)
            if held + -(-len(reqs[k]) // ps) * ps > budget_tokens:
                break
            waiting.pop(0)
            r.add_request(k)
            live.append(k)
            at[k] = 0
        entries = []
        for k in live:
            left = len(reqs[k]) - at[k]
            n = 1 if left <= 4 else min(g.choice([1, 2, 4, 6]), left)
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
        out = r.step(entries)
        row = 0
        for k, t, w in entries:
            got[k].append(out[row:row + len(w)])
            row += len(w)
            at[k] += len(t)
        for k in [k for k in live if at[k] == len(reqs[k])]:
            r.end_request(k)
            live.remove(k)
        r.cache.check()
    assert r.cache.pages_reused > 0
    for k in reqs:
        diff = (torch.cat(got[k]).double() - want[k]).abs().max()
        assert diff < 2e-4, (k, diff)


def test_step_graph_buckets():
    """What a step's bucket is made of: rows rounded up, spans and wanted rows rounded up coarsely,
    the leading one-token spans rounded down (and none for a step of single tokens only)."""
    from zig_ai_b200.engine.batch import leading_singles
    from zig_ai_b200.engine.graph import ShapeGraphs, round_count, round_rows
    assert [round_rows(n) for n in (1, 8, 9, 16, 17, 32, 33, 256, 257, 2048)] == [8, 8, 16, 16, 32, 32, 64, 256, 320, 2048]
    assert [round_count(n) for n in (0, 1, 8, 9, 16, 17, 33, 64, 65, 129)] == [8, 8, 8, 16, 16, 32, 64, 64, 128, 192]
    assert [leading_singles([1] * n + [5]) for n in (0, 7, 8, 9, 15, 16, 31, 33, 64, 65)] == [0, 0, 8, 8, 8, 16, 16, 32, 64, 64]
    assert leading_singles([1] * 9) == 0 and leading_singles([]) == 0 and leading_singles([3, 1, 1, 1, 1, 1, 1, 1, 1, 1]) == 0
    span = lambda n, wanted: ("r", 0, [0] * n, list(range(wanted)), 0)
    assert ShapeGraphs.key([span(1, 1)] * 9 + [span(30, 2)]) == (64, 16, 16, 8)
    assert ShapeGraphs.key([span(1, 1)] * 12 + [span(20, 1), span(18, 1)]) == (64, 16, 16, 8)
    assert ShapeGraphs.key([span(2000, 1)]) == (2048, 8, 8, 0)


@pytest.mark.parametrize("page_size", [8, 16, 64])
def test_padding_spans_stay_inside_their_table_rows(page_size):
    """The span of the null request that rounds a step's rows up lies at positions 0..pad-1; its row of
    every block table covers those positions (with null pages), in eager steps and in step graphs'
    buckets, also when the real requests are short and the pages small."""
    import numpy as np
    from zig_ai_b200.engine.batch import pack_host
    from zig_ai_b200.engine.graph import ShapeGraphs
    from zig_ai_b200.engine.runner import pad_rows

    def check(spans, tables, widths=None):
        flat, lay = pack_host(spans, tables, widths)
        for g, (off, w) in lay.tables.items():
            table = flat[off:off + lay.S * w].reshape(lay.S, w)
            for s, (c, n) in enumerate(zip(lay.ctx, lay.q_lens)):
                if n:
                    assert (c + n - 1) // page_size < w, (s, c, n, w)
            assert (table[len(spans_in):] == 0).all()              # the added spans see null pages only
        assert lay.total == flat.shape[0]

    for n_req, n_tok in [(4, 9), (3, 6), (17, 1), (1, 20), (2, 130), (5, 60)]:
        spans_in = [(f"r{i}", 0, [1] * n_tok, [n_tok - 1], i + 1) for i in range(n_req)]
        width = max(-(-n_tok // page_size), 1)
        tables_in = {0: np.arange(1, n_req * width + 1, dtype=np.int32).reshape(n_req, width)}
        spans, tables = pad_rows(spans_in, tables_in, page_size)
        assert sum(len(s[2]) for s in spans) % 32 == 0 or sum(len(s[2]) for s in spans) <= 16
        check(spans, tables)

        class Pool:
            pass
        pool = Pool()
        pool.page_size = page_size
        sg = ShapeGraphs(None, pool, None, None, None, {0: width})       # a pool of few positions: narrow tables
        k = sg.key(spans_in)
        spans, tables = sg._fill(k, spans_in, tables_in)
        assert sum(len(s[2]) for s in spans) == k[0] and len(spans) == k[1]
        check(spans, tables, sg.widths)


def test_a_raised_status_word_voids_the_step(tiny_models):
    """An id outside its bound is replaced by id 0 by the kernel that meets it and raises the status word;
    the step function reads the word with the step's results and raises (here on the plain stand-ins
    of the kernels, which keep the same word)."""
    from zig_ai_b200.engine.runner import StepError
    r = make_runner(tiny_models["A"], "A")
    V = r.model.vocab_size
    r.add_request("a")
    r.step([("a", random_tokens(V, 20, 3), [19])])
    # a block-table entry that points outside the pool (the host mirror of the request's table is spoilt)
    rc = r.cache.requests["a"]
    g = r.cache.paged_groups()[0]
    keep = int(r.cache._rows[g][rc.slot, 0])
    r.cache._rows[g][rc.slot, 0] = r.cache.num_pages + 7
    with pytest.raises(StepError, match="outside the page pool"):
        r.step([("a", [1], [0])])
    r.cache._rows[g][rc.slot, 0] = keep
    r.step([("a", [2], [0])])                                   # the word was cleared by the read: the next step is fine
    # a slot outside the slots
    slot, rc.slot = rc.slot, r.cache.max_requests + 3
    r.cache._rows[g] = __import__("numpy").vstack([r.cache._rows[g], r.cache._rows[g][:4]])
    with pytest.raises(StepError, match="slot outside"):
        r.step([("a", [3], [0])])
    rc.slot = slot
    # a token id outside the vocabulary that the host check was told to trust
    with pytest.raises(StepError, match="outside the vocabulary"):
        r.step([("a", [V + 5], [0])], trusted=True)
    assert ref_ops.read_status() == 0


def test_the_engine_reads_the_status_word_with_the_token_ids(tiny_models):
    from zig_ai_b200.engine.engine import Engine
    from zig_ai_b200.engine.runner import StepError
    from zig_ai_b200.sampling.sampler import SamplingParams
    eng = Engine(tiny_models["A"], "float32", max_num_seqs=2, max_tokens=256, page_size=16, device="cpu", ops=ref_ops)
    eng.add_request([1, 2, 3, 4, 5], SamplingParams(temperature=0.0, max_new_tokens=8))
    eng.step()
    eng.step()
    ref_ops._raise(1)                                             # as a kernel whose bounded wait ran out would
    with pytest.raises(StepError, match="bounded wait"):
        for _ in range(3):
            eng.step()
    assert ref_ops.read_status() == 0
