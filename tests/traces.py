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
