"""Whole-model checks through bin/trace_run: the same requests replayed whole, with the last 32
tokens decoded one by one, in portions of changing size, and mixed with other requests in a pool
so small that pages are used again; in 32-bit and in bfloat16; all compared with the plain
implementation (tests/plain_lfm2.py)."""
import numpy as np
import pytest
import torch

import plain_lfm2
import traces
from tiny_configs import PAGE_SIZE, TINY

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [70, 45, 128, 33, 7, 1, 2, 96], "B": [130, 61, 257, 40, 5, 1, 33, 90], "C": [300, 129, 64, 410, 1, 35]}


@pytest.fixture(scope="module")
def plain(tiny_models):
    out = {}
    for name, d in tiny_models.items():
        c, W = plain_lfm2.read_config(d), plain_lfm2.read_weights(d)
        reqs = traces.requests_for(c["vocab_size"], LENGTHS[name], 77)
        out[name] = (reqs, {k: plain_lfm2.forward(c, W, t).numpy() for k, t in reqs.items()})
    return out


def rows_of(got, tag, k, n):
    return np.stack([got[(tag + k, p)] for p in range(n)])


def compare(got, reqs, want, tag, dtype):
    for k, toks in reqs.items():
        traces.check_request(rows_of(got, tag, k, len(toks)), want[k], dtype, f"{dtype} schedule '{tag}' request {k}")


def compare_schedules(got, reqs, tag_a, tag_b, dtype):
    for k, toks in reqs.items():
        traces.check_same(rows_of(got, tag_a, k, len(toks)), rows_of(got, tag_b, k, len(toks)), dtype,
                          f"{dtype} schedules '{tag_a}'/'{tag_b}' request {k}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_schedules_agree_with_plain(tiny_models, plain, tmp_path, name, dtype):
    reqs, want = plain[name]
    vocab = TINY[name][0]["vocab_size"]
    steps = traces.number(traces.whole(reqs) + traces.decode_tail(reqs) + traces.portions(reqs, 3))
    got = traces.run_trace(tiny_models[name], dtype, steps, max_tokens=512, out_dir=str(tmp_path / "o"),
                           vocab=vocab, page_size=PAGE_SIZE[name])
    for tag in "wdp":
        compare(got, reqs, want, tag, dtype)
    compare_schedules(got, reqs, "w", "d", dtype)
    compare_schedules(got, reqs, "w", "p", dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_batches_in_a_small_pool(tiny_models, plain, tmp_path, name, dtype):
    reqs, want = plain[name]
    vocab = TINY[name][0]["vocab_size"]
    longest = -(-max(len(t) for t in reqs.values()) // 64) * 64
    max_tokens = longest + 128                       # a few requests at most: pages must be used again
    steps = traces.number(traces.mixed(reqs, 5, max_tokens))
    assert max(len(s["entries"]) for s in steps) >= 2
    stats = {}
    got = traces.run_trace(tiny_models[name], dtype, steps, max_tokens=max_tokens, out_dir=str(tmp_path / "o"),
                           vocab=vocab, page_size=PAGE_SIZE[name], stats=stats)
    compare(got, reqs, want, "m", dtype)
    # the pool is as small as asked for, every page of it was in use at some time, and pages that one
    # request gave back were handed to another
    assert stats["num_pages"] * stats["page_size"] == -(-max_tokens // PAGE_SIZE[name]) * PAGE_SIZE[name]
    assert stats["pages_reused"] > 0 and stats["slots_used"] == 0
    used = [v for k, v in stats.items() if k.endswith("_pages_used")]
    high = [v for k, v in stats.items() if k.endswith("_pages_high_water")]
    assert used and all(v == 0 for v in used) and all(v > stats["num_pages"] // 2 for v in high)
