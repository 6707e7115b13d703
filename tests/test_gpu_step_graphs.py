"""Step graphs for steps with spans: more buckets than are kept, and back to the first.

A bucket's graph is captured the third time the bucket is met and the most recently used sixteen are
kept.  One request's prompt is fed in portions whose row counts and numbers of wanted rows walk
through eighteen buckets, three times each, and then returns to the first: that one was dropped, is
captured again and replayed.  Every wanted row of every step is compared with the plain
implementation in 32-bit, so a graph that was captured, dropped, recaptured or replayed with another
step's description shows."""
import random

import numpy as np
import pytest

import plain_lfm2
import traces

pytestmark = pytest.mark.gpu


def test_more_buckets_than_kept_graphs_and_back_to_the_first(tiny_models):
    from zig_ai_b200.engine.graph import ShapeGraphs
    from zig_ai_b200.engine.runner import load_runner
    d = tiny_models["C"]
    c, W = plain_lfm2.read_config(d), plain_lfm2.read_weights(d)
    V = c["vocab_size"]
    g = random.Random(71)
    runner = load_runner(d, "float32", max_tokens=4096, page_size=64, max_requests=4)
    assert runner.use_graphs
    sg = runner.shape_graphs
    shapes = [(n, w) for n in (5, 12, 20, 40, 70, 100, 130) for w in (3, 12, 24) if w <= n]     # (tokens, wanted rows)
    assert len({ShapeGraphs.key([("r", 0, [0] * n, list(range(w)), 1)]) for n, w in shapes}) == len(shapes) > ShapeGraphs.KEEP
    toks, got, rows = [], [], []
    runner.add_request("r")

    def feed(n, w):
        new = [g.randrange(V) for _ in range(n)]
        want = sorted(g.sample(range(n), w))
        out = runner.step([("r", new, want)]).float().cpu().numpy()
        assert out.shape[0] == w
        for i, p in enumerate(want):
            got.append(out[i].copy())
            rows.append(len(toks) + p)
        toks.extend(new)

    first = ShapeGraphs.key([("r", 0, [0] * shapes[0][0], list(range(shapes[0][1])), 1)])
    for n, w in shapes:
        for _ in range(3):
            feed(n, w)
        if (n, w) == shapes[0]:
            assert first in sg.graphs                      # captured at its third step
    assert len(sg.graphs) == ShapeGraphs.KEEP and first not in sg.graphs      # the oldest were dropped
    replays = sg.replays
    for _ in range(4):
        feed(*shapes[0])                                   # seen before, captured again, then replayed
    assert first in sg.graphs and sg.replays > replays and len(sg.graphs) == ShapeGraphs.KEEP
    want = plain_lfm2.forward(c, W, toks, rows=rows).numpy()
    traces.check_request(np.stack(got), want, "float32", "portions through step graphs")
