"""Decode-only steps of more than 16 requests against the plain implementation.

From 17 rows on a step changes kernels entirely: the matrix products are the library's, the norm, the
activation, the convolution and the gather of wanted rows are kernels of their own, and the step's
graph belongs to the buckets of 32, 64, 128 and 256 rows.  Here 17, 24, 64 and 130 requests with
contexts that differ and cross page edges are prefilled in portions and then decoded together for
twelve steps (replayed from their graph); every decoded row is compared with tests/plain_lfm2.py, in
32-bit and in bfloat16, on Tiny B, the configuration with head size 64, and four layers of the
benchmark's widths.  And generation through the entry point with 24 requests at once gives the plain
greedy tokens in 32-bit.
"""
import random

import numpy as np
import pytest

import plain_lfm2
import traces
from tiny_configs import PAGE_SIZE, TINY

pytestmark = pytest.mark.gpu

DECODE_STEPS = 12


def prompt_lengths(n, page_size, g):
    """Lengths such that the decode steps cross page edges for some requests (a few tokens short of a
    multiple of the page size), start a page for others, and differ widely."""
    base = [page_size - 3, page_size, 2 * page_size - DECODE_STEPS + 1, 1, 2, 3 * page_size + 5, page_size + 1, 5 * page_size - 1]
    out = []
    for i in range(n):
        v = base[i % len(base)] + (i // len(base)) * g.choice([0, 1, 3]) % (3 * page_size)
        out.append(max(int(v), 1))
    return out


def run_wide_decode(model_dir, dtype, n_requests, page_size, seed, budget=512):
    from zig_ai_b200.engine.runner import load_runner
    c, W = plain_lfm2.read_config(model_dir), plain_lfm2.read_weights(model_dir)
    V = c["vocab_size"]
    g = random.Random(seed)
    lengths = prompt_lengths(n_requests, page_size, g)
    toks = {i: [g.randrange(V) for _ in range(n)] for i, n in enumerate(lengths)}
    total = sum(-(-(n + DECODE_STEPS + 1) // page_size) * page_size for n in lengths)
    runner = load_runner(model_dir, dtype, max_tokens=total + 4 * page_size, page_size=page_size,
                         max_requests=n_requests + 2)
    for k in toks:
        runner.add_request(k)
    # the prompts, several requests a step under a token budget, the longest cut into portions
    at = {k: 0 for k in toks}
    while any(at[k] < len(toks[k]) for k in toks):
        entries, left = [], budget
        for k in toks:
            n = min(len(toks[k]) - at[k], left, 3 * page_size + 1)
            if n <= 0:
                continue
            entries.append((k, toks[k][at[k]:at[k] + n], []))
            at[k] += n
            left -= n
        runner.step(entries)
    got, rows = {k: [] for k in toks}, {k: [] for k in toks}
    for step in range(DECODE_STEPS):
        entries = []
        for k in toks:
            t = g.randrange(V)
            toks[k].append(t)
            entries.append((k, [t], [0]))
        out = runner.step(entries).float().cpu().numpy()
        assert out.shape[0] == n_requests and np.isfinite(out).all()
        for i, k in enumerate(toks):
            got[k].append(out[i].copy())
            rows[k].append(len(toks[k]) - 1)
    if runner.use_graphs:
        assert runner.graphs.replays >= DECODE_STEPS - 2
    worst = 0.0
    for k in toks:
        want = plain_lfm2.forward(c, W, toks[k], rows=rows[k]).numpy()
        traces.check_request(np.stack(got[k]), want, dtype, f"{dtype} request {k} of {n_requests}")
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_requests", [17, 24, 64, 130])
@pytest.mark.parametrize("name", ["B", "C"])
def test_decode_steps_of_many_requests(tiny_models, name, n_requests, dtype):
    run_wide_decode(tiny_models[name], dtype, n_requests, PAGE_SIZE[name], seed=100 + n_requests)


@pytest.mark.parametrize("n_requests,dtype", [(17, "bfloat16"), (64, "bfloat16"), (130, "bfloat16"), (24, "float32")])
def test_decode_steps_of_many_requests_at_the_benchmark_widths(tmp_path_factory, n_requests, dtype):
    from test_gpu_full_width import FULL_WIDTH
    from zig_ai_b200.config import config_from_dict
    from zig_ai_b200.weights import write_random_model
    d = str(tmp_path_factory.mktemp("full_width_wide"))
    write_random_model(config_from_dict(FULL_WIDTH), 41, d, matrix_std="fan_in")
    run_wide_decode(d, dtype, n_requests, 64, seed=200 + n_requests, budget=2048)


@pytest.mark.parametrize("name", ["B", "C"])
def test_generation_with_24_requests_at_once_gives_the_plain_greedy_tokens(tiny_models, name):
    import zig_ai_b200 as z
    from test_gpu_generate import plain_greedy
    g = random.Random(31)
    V = TINY[name][0]["vocab_size"]
    prompts = [[g.randrange(V) for _ in range(1 + (7 * i) % 23)] for i in range(24)]
    eng = z.Engine(tiny_models[name], "float32", max_num_seqs=24, max_batched_tokens=64, max_model_len=64,
                   page_size=PAGE_SIZE[name])
    got = eng.generate(prompts, max_new_tokens=8, temperature=0.0)
    assert eng.stats()["steps_ahead"] > 0
    for p, out in zip(prompts, got):
        assert out == plain_greedy(tiny_models[name], p, 8)
