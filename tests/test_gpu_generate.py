"""Generation through the Python entry point on the GPU, long decoding, and the command line."""
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_lfm2
import traces
from tiny_configs import PAGE_SIZE, TINY

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def plain_greedy(model_dir, prompt, n):
    c, W = plain_lfm2.read_config(model_dir), plain_lfm2.read_weights(model_dir)
    toks = list(prompt)
    for _ in range(n):
        toks.append(plain_lfm2.greedy(plain_lfm2.forward(c, W, toks)[-1]))
    return toks[len(prompt):]


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_float32_matches_plain(tiny_models, name):
    import zig_ai_b200 as z
    g = random.Random(3)
    V = TINY[name][0]["vocab_size"]
    prompts = [[g.randrange(V) for _ in range(n)] for n in (7, 13, 1)]
    eng = z.Engine(tiny_models[name], "float32", max_num_seqs=3, max_batched_tokens=6, max_model_len=64,
                   page_size=PAGE_SIZE[name])
    got = eng.generate(prompts, max_new_tokens=8, temperature=0.0)
    for p, out in zip(prompts, got):
        assert out == plain_greedy(tiny_models[name], p, 8)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_bfloat16_picks_a_plain_maximum(tiny_models, name):
    """In bfloat16 a near-tie may fall the other way: every generated token must be within the
    bfloat16 tolerance of the plain implementation's best logit at its place."""
    import zig_ai_b200 as z
    g = random.Random(4)
    V = TINY[name][0]["vocab_size"]
    prompts = [[g.randrange(V) for _ in range(n)] for n in (5, 17, 33, 1)]
    eng = z.Engine(tiny_models[name], "bfloat16", max_num_seqs=4, max_batched_tokens=10, max_model_len=96,
                   page_size=PAGE_SIZE[name])
    got = eng.generate(prompts, max_new_tokens=10, temperature=0.0)
    c, W = plain_lfm2.read_config(tiny_models[name]), plain_lfm2.read_weights(tiny_models[name])
    for p, out in zip(prompts, got):
        assert len(out) == 10
        logits = plain_lfm2.forward(c, W, p + out)
        for i, tok in enumerate(out):
            row = logits[len(p) + i - 1]
            assert float(row.max() - row[tok]) <= 8e-2 * float(row.abs().max()), (i, tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_repetition_penalty_with_histories_on_the_device(tiny_models, dtype):
    """With a repetition penalty the requests' token counts live in a table on the device, so their steps run
    ahead like any other; the tokens are those of the same engine with the counts kept on the host (no step
    ahead then), for requests with and without a penalty, sampled and greedy, few pages (preemption), and a
    second round of requests that takes over the first round's rows of the table."""
    import zig_ai_b200 as z
    from zig_ai_b200.sampling import SamplingParams
    name = "B"
    g = random.Random(41)
    V = TINY[name][0]["vocab_size"]
    outs = []
    for on_device in (True, False):
        eng = z.Engine(tiny_models[name], dtype, max_num_seqs=4, max_batched_tokens=12, max_model_len=96,
                       max_tokens=224, page_size=PAGE_SIZE[name])
        assert eng.sampler.device_history
        eng.sampler.device_history = on_device
        g = random.Random(41)
        got = []
        for rnd in range(2):
            specs = [dict(temperature=0.9, top_k=20, repetition_penalty=1.3), dict(temperature=0.0, repetition_penalty=1.5),
                     dict(temperature=1.1, top_p=0.8), dict(temperature=0.7, repetition_penalty=1.15),
                     dict(temperature=0.8, top_k=5, repetition_penalty=2.0)]
            ids = [eng.add_request([g.randrange(V) for _ in range(3 + 4 * i)], SamplingParams(max_new_tokens=40, seed=7 * rnd + i, **sp))
                   for i, sp in enumerate(specs)]
            done = {}
            while len(done) < len(ids):
                for r in eng.step():
                    done[r.request_id] = r
            eng.flush()
            got.append([done[i].output for i in ids])
            assert not eng.sampler._slots                     # every row of the table was given back
        outs.append(got)
        st = eng.stats()
        assert (st["steps_ahead"] > 0) == on_device or st["steps_ahead"] > 0
        if on_device:
            assert st["steps_ahead"] > 10
    assert outs[0] == outs[1]
    assert all(len(o) == 40 for rnd in outs[0] for o in rnd)


def test_sampled_generation_is_fixed_by_the_seed_and_not_by_batching(tiny_models):
    import zig_ai_b200 as z
    g = random.Random(5)
    prompts = [[g.randrange(517) for _ in range(n)] for n in (1, 5, 17, 33)]
    kw = dict(max_new_tokens=10, temperature=1.0, seed=7)
    together = z.Engine(tiny_models["B"], "float32", max_num_seqs=4, max_batched_tokens=10, max_model_len=64,
                        page_size=8).generate(prompts, **kw)
    alone = [z.Engine(tiny_models["B"], "float32", max_num_seqs=1, max_batched_tokens=64, max_model_len=64,
                      page_size=8).generate([p], **dict(kw, seed=7 + i))[0] for i, p in enumerate(prompts)]
    assert together == alone
    tight = z.Engine(tiny_models["B"], "float32", max_num_seqs=4, max_batched_tokens=16, max_model_len=64,
                     max_tokens=56, page_size=8)
    assert tight.generate(prompts, **kw) == alone and tight.stats()["preemptions"] > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(tiny_models, tmp_path, dtype):
    """One request decoded token by token from its first token for 600 positions."""
    d = tiny_models["B"]
    c, W = plain_lfm2.read_config(d), plain_lfm2.read_weights(d)
    toks = traces.requests_for(c["vocab_size"], [600], 9)["q0"]
    want = plain_lfm2.forward(c, W, toks).numpy()
    steps = traces.number(traces.decode_tail({"q0": toks}, tail=600))
    got = traces.run_trace(d, dtype, steps, max_tokens=640, out_dir=str(tmp_path / "o"), vocab=c["vocab_size"], page_size=8)
    traces.check_request(np.stack([got[("dq0", p)] for p in range(600)]), want, dtype, f"{dtype} long decoding")


def test_command_line(tiny_models):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "zig-ai-engine"), "-m", tiny_models["A"],
                          "--prompt", "5,17,3", "-n", "6", "--temperature", "0", "--dtype", "float32"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    line = next(l for l in out.stdout.splitlines() if l.startswith("[0]"))
    ids = [int(x) for x in line.split(")")[1].split()]
    assert ids == plain_greedy(tiny_models["A"], [5, 17, 3], 6)
    assert "decode:" in out.stdout and "prefill:" in out.stdout and "warm-up:" in out.stdout


def test_warm_up_leaves_nothing_behind(tiny_models):
    """Engine.warm_up runs a request of its own and captures the bucket's decode graph; afterwards no request, page
    or slot is held, request ids start where they would have, and generation gives the tokens it gives without it."""
    import zig_ai_b200 as z
    prompts = [[5, 17, 3], [9, 1, 200, 7, 7, 41]]
    want = [plain_greedy(tiny_models["A"], p, 6) for p in prompts]
    eng = z.Engine(tiny_models["A"], "float32", max_num_seqs=2, max_batched_tokens=8, max_model_len=64, page_size=PAGE_SIZE["A"])
    eng.warm_up(2)
    assert not eng.requests and not eng.has_work()
    assert eng.runner.graphs.bucket(2) in eng.runner.graphs.graphs
    assert all(v == 0 for k, v in eng.stats().items() if k.endswith("pages_used"))
    from zig_ai_b200.sampling import SamplingParams
    assert eng.add_request(prompts[0], SamplingParams(temperature=0.0, max_new_tokens=2)) == 0    # (the warm-up request took a name of its own)
    while eng.has_work():
        eng.step()
    eng.flush()
    assert eng.generate(prompts, max_new_tokens=6, temperature=0.0) == want


def test_command_line_sizes_the_pool_and_profiles(tiny_models):
    """--page-size, --num-pages and --max-num-seqs size the engine (four sequences through two seats and a
    pool of 12 pages of 8 positions: the same tokens as alone); --profile prints the time by kernel class
    for both kinds of step and changes no token."""
    base = [sys.executable, os.path.join(ROOT, "bin", "zig-ai-engine"), "-m", tiny_models["C"], "--prompt", "5,17,3,900,41",
            "-n", "7", "--temperature", "0"]
    want = plain_greedy(tiny_models["C"], [5, 17, 3, 900, 41], 7)
    out = subprocess.run(base + ["--dtype", "float32", "-np", "4", "--max-num-seqs", "2", "--page-size", "8", "--num-pages", "12"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    lines = [l for l in out.stdout.splitlines() if l.startswith("[") and ") " in l and not l.startswith("[+]")]
    assert len(lines) == 4 and all([int(x) for x in l.split(")")[1].split()] == want for l in lines)
    assert "12 pages of 8 positions" in out.stdout
    assert "tokens of 4 sequences" in out.stdout and "first token after" in out.stdout
    out = subprocess.run(base + ["--dtype", "bfloat16", "--profile"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    prof = [l for l in out.stdout.splitlines() if l.startswith("[profile]")]
    assert any("decode steps" in l for l in prof) and any("steps with prompt portions" in l for l in prof)
    for word in ("attention", "products", "head", "sampling", "embedding"):
        assert any(word in l for l in prof), word
    bad = subprocess.run(base + ["--page-size", "0"], capture_output=True, text=True, timeout=600)
    assert bad.returncode == 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_repeated_step_shapes_run_as_graphs_and_agree(tiny_models, dtype):
    """The same span lengths again and again (here: five requests of 40 tokens, each cut 24 + 16):
    from the third time on the step is a replayed graph; its logits equal the eager ones."""
    from zig_ai_b200.engine.runner import load_runner
    d = tiny_models["B"]
    c, W = plain_lfm2.read_config(d), plain_lfm2.read_weights(d)
    reqs = traces.requests_for(c["vocab_size"], [40] * 5, 21)
    runner = load_runner(d, dtype, max_tokens=512, page_size=8)
    eager = load_runner(d, dtype, max_tokens=512, page_size=8, graphs=False)
    for k, toks in reqs.items():
        want = plain_lfm2.forward(c, W, toks).numpy()
        outs = []
        for r in (runner, eager):
            r.add_request(k)
            a = r.step([(k, toks[:24], list(range(24)))]).cpu().numpy().copy()
            b = r.step([(k, toks[24:], list(range(16)))]).cpu().numpy().copy()
            r.end_request(k)
            outs.append(np.concatenate([a, b]))
        traces.check_request(outs[0], want, dtype, f"{dtype} graphed request {k}")
        assert np.array_equal(outs[0], outs[1]) or dtype == "bfloat16" or np.abs(outs[0] - outs[1]).max() < 1e-5
    assert runner.shape_graphs.replays >= 4 and len(runner.shape_graphs.graphs) == 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_of_one_bucket_share_a_graph_and_agree(tiny_models, dtype):
    """Steps whose shapes differ but round to the same counts (17 to 32 rows, two to five spans, some
    of one token beside prompt portions, up to eight wanted rows) are replayed from one graph once it
    is captured; logits as from the runner without graphs; the requests go on across the steps, so a
    padded row that touched a request's pages or state would show."""
    from zig_ai_b200.engine.runner import load_runner
    d = tiny_models["A"]
    c, W = plain_lfm2.read_config(d), plain_lfm2.read_weights(d)
    g = random.Random(23)
    V = c["vocab_size"]
    runner = load_runner(d, dtype, max_tokens=2048, page_size=PAGE_SIZE["A"], max_requests=8)
    eager = load_runner(d, dtype, max_tokens=2048, page_size=PAGE_SIZE["A"], max_requests=8, graphs=False)
    toks = {k: [] for k in range(5)}
    for r in (runner, eager):
        for k in toks:
            r.add_request(k)
    worst = 0.0
    for step in range(14):
        n_spans = g.randint(2, 5)
        ks = g.sample(range(5), n_spans)
        sizes = [1] * (n_spans - 1) + [0]
        sizes[-1] = g.randint(17, 32) - sum(sizes)                  # the step's rows: 17..32
        entries = []
        for k, n in zip(ks, sizes):
            new = [g.randrange(V) for _ in range(n)]
            want = sorted(g.sample(range(n), min(n, g.randint(0, 2))))
            entries.append((k, new, want))
            toks[k] += new
        a = runner.step(entries).cpu().numpy().copy()
        b = eager.step(entries).cpu().numpy().copy()
        assert a.shape == b.shape
        if a.size:
            worst = max(worst, float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-6)))
    assert len(runner.shape_graphs.graphs) == 1 and runner.shape_graphs.replays >= 10
    assert worst < (2e-5 if dtype == "float32" else 4e-2), worst
    # and the requests' caches are what the plain implementation expects: one more token each
    for k in toks:
        nxt = [(k, [3], [0])]
        got = runner.step(nxt).cpu().numpy()[0]
        want = plain_lfm2.forward(c, W, toks[k] + [3]).numpy()[-1]
        traces.check_request(got[None], want[None], dtype, f"{dtype} request {k} after bucketed steps")


@pytest.mark.parametrize("name", ["B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_requests_beside_prompt_portions(tiny_models, name, dtype):
    """Steps with 9 to 12 decoding requests in front and one or two prompt portions behind them: in
    bfloat16 the first 8 one-token spans go through the single-token attention kernel, the rest
    through the span kernel.  Every wanted row against the plain implementation, run eagerly and
    (from the third step of the bucket on) from a graph; the contexts differ, cross page edges and
    grow from step to step."""
    from zig_ai_b200.engine.runner import load_runner
    d = tiny_models[name]
    c, W = plain_lfm2.read_config(d), plain_lfm2.read_weights(d)
    g = random.Random(31)
    V, ps = c["vocab_size"], PAGE_SIZE[name]
    runner = load_runner(d, dtype, max_tokens=16 * 256, page_size=ps, max_requests=16)
    n_dec = 12
    toks = {k: [g.randrange(V) for _ in range(ps * (k % 3) + 3 + 5 * k)] for k in range(n_dec)}
    for k in toks:
        runner.add_request(k)
        runner.step([(k, toks[k], [])])
    prompts = {100 + i: [g.randrange(V) for _ in range(400)] for i in range(3)}
    for k in prompts:
        runner.add_request(k)
    plain_cache = {}

    def plain_row(k, seq):
        key = (k, len(seq))
        if key not in plain_cache:
            plain_cache[key] = plain_lfm2.forward(c, W, seq).numpy()
        return plain_cache[key]

    done = {k: 0 for k in prompts}
    pairs = {}
    for step in range(8):
        live = list(range(n_dec)) if step % 2 == 0 else list(range(n_dec - 3))
        entries, checks = [], []
        for k in live:
            t = g.randrange(V)
            toks[k].append(t)
            entries.append((k, [t], [0]))
            checks.append((k, list(toks[k]), [len(toks[k]) - 1]))
        for k in list(prompts)[: 1 + step % 2]:
            n = g.randint(30, 40) if step % 2 == 0 else g.randint(15, 20)      # 39 to 52 rows a step: one bucket
            part = prompts[k][done[k]:done[k] + n]
            want = sorted({0, n - 1})
            entries.append((k, part, want))
            checks.append((k, prompts[k][:done[k] + n], [done[k] + w for w in want]))
            done[k] += n
        got = runner.step(entries).cpu().numpy()
        at = 0
        for k, seq, rows in checks:
            ref = plain_row(k, seq)
            for r in rows:
                assert np.isfinite(got[at]).all(), (step, k, r)
                pairs.setdefault(k, ([], []))
                pairs[k][0].append(got[at])
                pairs[k][1].append(ref[r])
                at += 1
        assert at == got.shape[0]
    for k, (a, b) in pairs.items():               # a request's rows of all steps together, as in the replay tests
        traces.check_request(np.stack(a), np.stack(b), dtype, f"{dtype} request {k}")
    if dtype == "bfloat16":
        assert runner.shape_graphs.replays >= 2
        assert any(k[3] == 8 for k in runner.shape_graphs.graphs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("temperature", [0.0, 0.9])
def test_a_step_ahead_of_the_host_changes_no_token(tiny_models, dtype, temperature):
    """With `pipeline` the engine launches a decode step before it has read the tokens of the step
    before.  Same tokens as without it: requests of different lengths that end at different steps (by
    their length, and one by an EOS token, whose row of the step launched ahead is dropped), more
    requests than seats (so that steps with admissions and prompts come between), few pages."""
    import zig_ai_b200 as z
    name = "B"
    g = random.Random(11)
    V = TINY[name][0]["vocab_size"]
    prompts = [[g.randrange(V) for _ in range(n)] for n in (9, 3, 21, 5, 14, 2)]
    news = [12, 30, 7, 19, 25, 9]

    def run(pipeline, eos_of=None):
        eng = z.Engine(tiny_models[name], dtype, max_num_seqs=3, max_batched_tokens=16, max_model_len=64,
                       max_tokens=3 * 64, page_size=PAGE_SIZE[name], pipeline=pipeline)
        ids = [eng.add_request(p, z.SamplingParams(temperature=temperature, top_k=40, seed=5 + i, max_new_tokens=n,
                                                   eos_id=(eos_of[i] if eos_of else None)))
               for i, (p, n) in enumerate(zip(prompts, news))]
        done = {}
        while eng.has_work():
            for r in eng.step():
                done[r.request_id] = r
        eng.flush()
        return [done[i].output for i in ids], [done[i].finish_reason for i in ids], eng.stats()

    base, reasons, _ = run(False)
    assert [len(o) for o in base] == news and set(reasons) == {"length"}
    got, _, stats = run(True)
    assert got == base and stats["steps_ahead"] >= 3
    # an EOS token in the middle of three outputs: the token that the plain run produced there
    eos = [None, base[1][11], None, base[3][6], base[4][20], None]
    want = [o if e is None else o[:o.index(e) + 1] for o, e in zip(base, eos)]
    base_eos, reasons, _ = run(False, eos)
    assert reasons[1] == reasons[3] == reasons[4] == "eos"
    if dtype == "float32":            # (in bfloat16 a sampled token may depend on what else was in its step's batch)
        assert base_eos == want
    else:
        assert [o[-1] for o in base_eos] == [w[-1] if e is None else e for w, e in zip(base_eos, eos)]
    got, reasons, stats = run(True, eos)
    assert got == base_eos and reasons[1] == "eos" and stats["steps_ahead"] >= 1


def test_a_step_ahead_with_preemptions(tiny_models):
    """So few pages that running requests are preempted and recomputed: the engine that keeps a step
    ahead gives the same tokens as the one that does not, and both saw preemptions."""
    import zig_ai_b200 as z
    name = "B"
    g = random.Random(12)
    V = TINY[name][0]["vocab_size"]
    prompts = [[g.randrange(V) for _ in range(n)] for n in (20, 11, 17, 6)]

    def run(pipeline):
        eng = z.Engine(tiny_models[name], "float32", max_num_seqs=4, max_batched_tokens=24, max_model_len=64,
                       max_tokens=11 * PAGE_SIZE[name], page_size=PAGE_SIZE[name], pipeline=pipeline)
        out = eng.generate(prompts, max_new_tokens=24, temperature=0.8, top_p=0.9, seed=3)
        return out, eng.stats()

    base, st0 = run(False)
    got, st1 = run(True)
    assert got == base and all(len(o) == 24 for o in got)
    assert st0["preemptions"] > 0 and st1["preemptions"] > 0 and st1["steps_ahead"] > 0


@pytest.mark.parametrize("name", ["B", "C"])
def test_preemption_and_recomputation_in_bfloat16_pick_plain_maxima(tiny_models, name):
    """In bfloat16, with so few pages that running requests are preempted and recomputed from their prompt
    and the tokens they had produced: every request still gets all its tokens, and every greedy token is
    within the bfloat16 tolerance of the plain implementation's best logit at its place (a recomputed
    request runs its old tokens as a prompt portion, through other kernels than when it decoded them)."""
    import zig_ai_b200 as z
    g = random.Random(14)
    V = TINY[name][0]["vocab_size"]
    ps = PAGE_SIZE[name]
    prompts = [[g.randrange(V) for _ in range(n)] for n in (2 * ps + 3, ps + 1, 2 * ps - 1, ps // 2 + 1)]
    new = ps + 5
    eng = z.Engine(tiny_models[name], "bfloat16", max_num_seqs=4, max_batched_tokens=3 * ps, max_model_len=4 * ps + 16,
                   max_tokens=9 * ps, page_size=ps)
    got = eng.generate(prompts, max_new_tokens=new, temperature=0.0)
    st = eng.stats()
    assert st["preemptions"] > 0 and all(len(o) == new for o in got)
    assert all(v == 0 for k, v in st.items() if k.endswith("_pages_used")) and st["slots_used"] == 0
    c, W = plain_lfm2.read_config(tiny_models[name]), plain_lfm2.read_weights(tiny_models[name])
    for p, out in zip(prompts, got):
        logits = plain_lfm2.forward(c, W, p + out)
        for i, tok in enumerate(out):
            row = logits[len(p) + i - 1]
            assert float(row.max() - row[tok]) <= 8e-2 * float(row.abs().max()), (i, tok)


def test_a_long_random_serving_run_gives_the_plain_greedy_tokens(tiny_models):
    """Forty requests of random lengths through six seats and a pool so small that requests are preempted
    and recomputed, arriving while others decode (so that steps of every kind follow one another: prompt
    portions alone, beside decoding requests, decode steps replayed from graphs and launched a step
    ahead): in 32-bit every request's tokens are the plain implementation's greedy tokens, and at the end
    every page and slot is free."""
    import zig_ai_b200 as z
    name = "B"
    g = random.Random(21)
    V = TINY[name][0]["vocab_size"]
    ps = PAGE_SIZE[name]
    eng = z.Engine(tiny_models[name], "float32", max_num_seqs=6, max_batched_tokens=40, max_model_len=128,
                   max_tokens=26 * ps, page_size=ps)
    todo = [([g.randrange(V) for _ in range(g.randint(1, 60))], g.randint(3, 24)) for _ in range(40)]
    ids, done, at = {}, {}, 0
    while len(done) < len(todo):
        # a few arrivals every few steps
        if at < len(todo) and (eng.n_steps % 3 == 0 or not eng.has_work()):
            for _ in range(g.randint(1, 3)):
                if at < len(todo):
                    p, n = todo[at]
                    ids[eng.add_request(p, z.SamplingParams(temperature=0.0, max_new_tokens=n))] = at
                    at += 1
        for r in eng.step():
            done[ids[r.request_id]] = r
    eng.flush()
    st = eng.stats()
    assert st["preemptions"] > 0 and st["steps_ahead"] > 0
    assert st["slots_used"] == 0 and all(v == 0 for k, v in st.items() if k.endswith("_pages_used"))
    eng.runner.cache.check()
    for i, (p, n) in enumerate(todo):
        assert done[i].finish_reason == "length" and done[i].output == plain_greedy(tiny_models[name], p, n), i
