"""Traces for the replay program: the same requests cut into steps in different ways, and a helper
that runs bin/trace_run on a trace and collects the logits by (request, position)."""
from __future__ import annotations

import json
import os
import random
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def requests_for(vocab, lengths, seed):
    g = random.Random(seed)
    return {f"q{i}": [g.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


def whole(reqs, tag="w"):
    """Each request alone and whole."""
    steps = []
    for k, toks in reqs.items():
        steps.append({"entries": [{"id": tag + k, "tokens": toks, "want": list(range(len(toks)))}], "end": [tag + k]})
    return steps


def decode_tail(reqs, tail=32, tag="d"):
    """Most of a request in one step, its last `tail` tokens one by one."""
    steps = []
    for k, toks in reqs.items():
        head = max(len(toks) - tail, 0)
        at = 0
        if head:
            steps.append({"entries": [{"id": tag + k, "tokens": toks[:head], "want": list(range(head))}], "end": []})
            at = head
        while at < len(toks):
            steps.append({"entries": [{"id": tag + k, "tokens": toks[at:at + 1], "want": [0]}], "end": []})
            at += 1
        steps[-1]["end"] = [tag + k]
    return steps


def portions(reqs, seed, tag="p", sizes=(2, 3, 5, 7, 13, 29, 64)):
    """Portions of changing size, down to two tokens."""
    g = random.Random(seed)
    steps = []
    for k, toks in reqs.items():
        at = 0
        while at < len(toks):
            n = min(g.choice(sizes), len(toks) - at)
            steps.append({"entries": [{"id": tag + k, "tokens": toks[at:at + n], "want": list(range(n))}], "end": []})
            at += n
        steps[-1]["end"] = [tag + k]
    return steps


def mixed(reqs, seed, max_tokens, round_to=64, max_live=4, tag="m"):
    """Up to `max_live` live requests: portions of some beside single decoded tokens of others,
    admitted only while the rounded-up sizes of the live requests fit `max_tokens`, so that pages
    of finished requests are used again."""
    g = random.Random(seed)
    waiting = list(reqs)
    live, at, steps = [], {}, []
    size = lambda k: -(-len(reqs[k]) // round_to) * round_to
    while waiting or live:
        while waiting and len(live) < max_live and sum(size(x) for x in live) + size(waiting[0]) <= max_tokens:
            k = waiting.pop(0)
            live.append(k)
            at[k] = 0
        if not live:
            raise ValueError("a request does not fit max_tokens")
        entries = []
        for k in live:
            if len(live) > 1 and g.random() < 0.2:
                continue                                  # left out of this step, goes on later
            left = len(reqs[k]) - at[k]
            decoding = left <= len(reqs[k]) // 3          # the last third comes one token at a time
            n = 1 if decoding else min(g.choice([2, 3, 4, 6, 9, 17]), left)
            entries.append({"id": tag + k, "tokens": reqs[k][at[k]:at[k] + n], "want": list(range(n))})
            at[k] += n
        if not entries:
            continue
        ended = [k for k in live if at[k] == len(reqs[k])]
        for k in ended:
            live.remove(k)
        steps.append({"entries": entries, "end": [tag + k for k in ended]})
    return steps


def number(steps, first=0):
    return [dict(s, step=first + i) for i, s in enumerate(steps)]


def run_trace(model_dir, dtype, steps, max_tokens, out_dir, vocab, page_size=16, timeout=900, stats=None):
    """Run bin/trace_run on the numbered steps; returns {(request id, position): logits row}.  `stats`:
    a dict that receives the counters the program writes when its input ends."""
    os.makedirs(out_dir, exist_ok=True)
    env = dict(os.environ)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens), "--page-size", str(page_size)]
    if stats is not None:
        cmd += ["--stats", os.path.join(out_dir, "stats.json")]
    p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    got, pos = {}, {}
    try:
        for s in steps:
            p.stdin.write(json.dumps(s) + "\n")
            p.stdin.flush()
            line = p.stdout.readline()
            assert line.strip() == f"done {s['step']}", f"trace_run said {line!r} (exit {p.poll()})"
            n_want = sum(len(e["want"]) for e in s["entries"])
            path = os.path.join(out_dir, f"{s['step']}.f32")
            if n_want:
                data = np.fromfile(path, dtype="<f4").reshape(n_want, vocab)
                row = 0
                for e in s["entries"]:
                    base = pos.get(e["id"], 0)
                    for w in e["want"]:
                        got[(e["id"], base + w)] = data[row]
                        row += 1
            for e in s["entries"]:
                pos[e["id"]] = pos.get(e["id"], 0) + len(e["tokens"])
            for k in s["end"]:
                pos.pop(k, None)
        p.stdin.close()
        assert p.wait(timeout=timeout) == 0
        if stats is not None:
            with open(os.path.join(out_dir, "stats.json")) as f:
                stats.update(json.load(f))
    finally:
        if p.poll() is None:
            p.kill()
    return got


# How far logits may be from the plain implementation's.
#   float32: every row within 5e-5 of its largest logit (rounding of sums of a few hundred terms
#   through a handful of layers stays far below that).  Two ways of cutting the same request agree
#   within 2e-5.
#   bfloat16: every stored activation is rounded to 8 bits of mantissa (relative 2^-9), and the
#   absolute error that this leaves in a row of logits follows the size of the activations, not the
#   size of that row's logits.  So a row's error is measured against the request's logit scale (the
#   root mean square over all its rows).  Measured on the tiny models: 2 % on average, up to 5-6 %
#   for single rows, the same whether the request runs whole, token by token or in portions, and
#   moving by a per cent when another kernel takes a product.  Asserted: the mean over a request's
#   rows below 3 %, every row below 10 %.  A fault of the cache or of the batch moves a row by tens
#   of per cent; smaller faults are the 32-bit path's to show, which runs the same cache and batch
#   code, and the tensor-core kernels have their own tests against plain versions with tight limits.
def request_errors(got_rows, want_rows):
    """Per row: root-mean-square error over the request's root-mean-square logit."""
    want = np.asarray(want_rows, dtype=np.float64)
    got = np.asarray(got_rows, dtype=np.float64)
    scale = max(float(np.sqrt((want ** 2).mean())), 1e-30)
    return np.sqrt(((got - want) ** 2).mean(axis=1)) / scale


def check_request(got_rows, want_rows, dtype, where):
    """All rows of one request against the plain implementation."""
    want = np.asarray(want_rows, dtype=np.float64)
    got = np.asarray(got_rows, dtype=np.float64)
    if dtype == "float32":
        err = np.abs(got - want).max(axis=1) / np.maximum(np.abs(want).max(axis=1), 1e-30)
        assert err.max() < 5e-5, f"{where}: position {int(err.argmax())} is off by {err.max():.3e} of its largest logit"
    else:
        e = request_errors(got, want)
        assert e.max() < 1e-1, f"{where}: position {int(e.argmax())} is off by {e.max():.3e} of the request's logit scale"
        assert e.mean() < 3e-2, f"{where}: rows are off by {e.mean():.3e} of the request's logit scale on average"


def check_same(a_rows, b_rows, dtype, where):
    """Two ways of running the same request.  In 32-bit they agree to the rounding of the sums.  In
    bfloat16 the two runs may go through different kernels (library product or few-rows kernel,
    span or single-token attention) and are two independent roundings; their distance is held to
    twice the limit of one run."""
    a, b = np.asarray(a_rows, dtype=np.float64), np.asarray(b_rows, dtype=np.float64)
    if dtype == "float32":
        err = np.abs(a - b).max(axis=1) / np.maximum(np.abs(b).max(axis=1), 1e-30)
        assert err.max() < 2e-5, f"{where}: position {int(err.argmax())} differs by {err.max():.3e}"
    else:
        e = request_errors(a, b)
        assert e.max() < 2e-1 and e.mean() < 6e-2, f"{where}: two ways of cutting differ by {e.max():.3e} (mean {e.mean():.3e})"
