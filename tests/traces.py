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


def run_trace(model_dir, dtype, steps, max_tokens, out_dir, vocab, page_size=16, timeout=900):
    """Run bin/trace_run on the numbered steps; returns {(request id, position): logits row}."""
    os.makedirs(out_dir, exist_ok=True)
    env = dict(os.environ)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens), "--page-size", str(page_size)]
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
    finally:
        if p.poll() is None:
            p.kill()
    return got


# How far logits may be from the plain implementation's, per row of logits.
#   float32: rounding of sums of a few hundred terms through a handful of layers, far below 5e-5 of
#   the largest logit.
#   bfloat16: every stored activation is rounded to 8 bits of mantissa (relative 2^-9); over the
#   layers this adds up to a relative error of the row (L2) near 2 % on average with a tail to 5 %
#   among 600 rows, the same whether the request runs whole or token by token.  A fault of the
#   cache or the batch moves a row by tens of per cent; faults smaller than this noise are the 32-bit
#   path's to show.  Rows of different ways of cutting the same request are also compared with each
#   other: in 32-bit they agree to rounding of the sums; in bfloat16 a span and a single token run
#   through different attention kernels (other orders of summation, probabilities rounded to
#   bfloat16 at other places), so two runs differ like two independent roundings of the same row and
#   get the same limit as a run against the plain implementation.
def row_error(got, want):
    """(relative L2 error of the row, largest absolute error over the row's largest |logit|)"""
    err = np.abs(got.astype(np.float64) - want)
    return float(np.linalg.norm(err) / max(np.linalg.norm(want), 1e-30)), float(err.max() / max(np.abs(want).max(), 1e-30))


def check_row(got, want, dtype, where):
    l2, mx = row_error(got, want)
    if dtype == "float32":
        assert mx < 5e-5, f"{where}: error {mx:.3e} of the row's largest logit"
    else:
        assert l2 < 6e-2 and mx < 8e-2, f"{where}: relative L2 error {l2:.3e}, largest {mx:.3e}"


def check_same(a, b, dtype, where):
    """Two ways of running the same position."""
    l2, mx = row_error(a, b.astype(np.float64))
    lim_l2, lim_mx = (2e-5, 2e-5) if dtype == "float32" else (6e-2, 8e-2)
    assert l2 < lim_l2 and mx < lim_mx, f"{where}: two ways of cutting differ by L2 {l2:.3e}, largest {mx:.3e}"
