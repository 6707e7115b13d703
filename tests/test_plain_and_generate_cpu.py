"""The plain implementation's own parts, and generation through the engine's entry point on the
CPU (kernels replaced by their plain PyTorch versions) compared with plain greedy decoding."""
import math
import random

import pytest
import torch

import plain_lfm2
import ref_ops
from tiny_configs import PAGE_SIZE, TINY
from zig_ai_b200.engine.engine import Engine
from zig_ai_b200.sampling import SamplingParams, uniform


def test_plain_parts():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(plain_lfm2.rms_norm(x, torch.ones(2, dtype=torch.float64), 0.0),
                          x / math.sqrt(12.5))
    # rotation keeps the norm and position 0 is the identity (src/transformer/rope.zig:226-253)
    v = torch.randn(5, 2, 8, dtype=torch.float64)
    r = plain_lfm2.rotary_half_split(v, torch.arange(5), 10000.0)
    assert torch.allclose(r.norm(dim=-1), v.norm(dim=-1)) and torch.allclose(r[0], v[0])
    # pair (i, i + D/2), angle pos * theta^(-2i/D)
    e = torch.zeros(1, 1, 4, dtype=torch.float64)
    e[0, 0, 1] = 1.0
    out = plain_lfm2.rotary_half_split(e, torch.tensor([3]), 100.0)
    ang = 3 * 100.0 ** (-2 / 4)
    assert torch.allclose(out[0, 0], torch.tensor([0, math.cos(ang), 0, math.sin(ang)], dtype=torch.float64))
    # convolution: tap L-1 multiplies the current token, earlier taps earlier tokens, zeros before the start
    u = torch.tensor([[1.0], [10.0], [100.0]], dtype=torch.float64)
    w = torch.tensor([[0.5, 2.0, 3.0]], dtype=torch.float64)
    y = plain_lfm2.causal_depthwise_conv(u, w, None)
    assert y[:, 0].tolist() == [3.0, 32.0, 320.5]
    # attention: the first position attends only to itself; query head h reads kv head h // group
    q, k, vv = torch.randn(4, 4, 8, dtype=torch.float64), torch.randn(4, 2, 8, dtype=torch.float64), \
        torch.randn(4, 2, 8, dtype=torch.float64)
    o = plain_lfm2.causal_attention(q, k, vv, 8 ** -0.5)
    assert torch.allclose(o[0, 3], vv[0, 1]) and torch.allclose(o[0, 0], vv[0, 0])
    o_w = plain_lfm2.causal_attention(q, k, vv, 8 ** -0.5, window=1)
    assert torch.allclose(o_w[:, 2], vv[:, 1])


def test_plain_sampler_follows_the_reference_order():
    logits = torch.tensor([1.0, 3.0, 3.0, -2.0, 0.5])
    assert plain_lfm2.greedy(logits) == 1                                   # first maximum
    assert plain_lfm2.sample(logits, 0.3, temperature=0.0) == 1
    p = torch.softmax(logits.double(), -1)
    assert plain_lfm2.sample(logits, float(p[0]) - 1e-9) == 0 and plain_lfm2.sample(logits, float(p[0]) + 1e-9) == 1
    assert plain_lfm2.sample(logits, 0.999, top_k=2) in (1, 2)
    assert plain_lfm2.sample(logits, 0.999, top_p=0.5) in (1, 2)
    pen = plain_lfm2.sample(logits, 0.0, temperature=0.0, repetition_penalty=4.0, history=[1, 3])
    assert pen == 2                                                         # 3.0/4 drops below the other 3.0
    counts = [0] * 5
    g = random.Random(0)
    for _ in range(4000):
        counts[plain_lfm2.sample(logits, g.random(), temperature=1.0)] += 1
    assert all(abs(c / 4000 - float(pi)) < 0.03 for c, pi in zip(counts, p))


def test_uniform_numbers_are_fixed_by_seed_and_index():
    a = [uniform(42, i) for i in range(1000)]
    assert a == [uniform(42, i) for i in range(1000)] and a != [uniform(43, i) for i in range(1000)]
    assert all(0.0 <= x < 1.0 for x in a) and 0.45 < sum(a) / 1000 < 0.55
    assert all(float(torch.tensor(x, dtype=torch.float32)) == x for x in a)  # exact in 32-bit


def plain_greedy(model_dir, prompt, n):
    c, W = plain_lfm2.read_config(model_dir), plain_lfm2.read_weights(model_dir)
    toks = list(prompt)
    for _ in range(n):
        toks.append(plain_lfm2.greedy(plain_lfm2.forward(c, W, toks)[-1]))
    return toks[len(prompt):]


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_matches_plain(tiny_models, name):
    g = random.Random(3)
    V = TINY[name][0]["vocab_size"]
    prompts = [[g.randrange(V) for _ in range(n)] for n in (7, 13, 1)]
    eng = Engine(tiny_models[name], "float32", max_num_seqs=3, max_batched_tokens=6, max_model_len=64,
                 page_size=PAGE_SIZE[name], device="cpu", ops=ref_ops)
    got = eng.generate(prompts, max_new_tokens=8, temperature=0.0)
    for p, out in zip(prompts, got):
        assert out == plain_greedy(tiny_models[name], p, 8)
    st = eng.stats()
    assert st["slots_used"] == 0 and st["generated"] == 24


def test_sampled_tokens_do_not_depend_on_batching_or_preemption(tiny_models):
    name = "B"
    g = random.Random(4)
    V = TINY[name][0]["vocab_size"]
    prompts = [[g.randrange(V) for _ in range(n)] for n in (1, 5, 17, 33)]
    kw = dict(max_new_tokens=10, temperature=1.0, seed=123)
    alone = []
    for i, p in enumerate(prompts):
        eng = Engine(tiny_models[name], "float32", max_num_seqs=1, max_batched_tokens=64, max_model_len=64,
                     page_size=8, device="cpu", ops=ref_ops)
        alone.append(eng.generate([p], **dict(kw, seed=123 + i))[0])
    eng = Engine(tiny_models[name], "float32", max_num_seqs=4, max_batched_tokens=6 + 4, max_model_len=64,
                 page_size=8, device="cpu", ops=ref_ops)
    assert eng.generate(prompts, **kw) == alone
    # a pool so small that requests are preempted and recomputed
    tight = Engine(tiny_models[name], "float32", max_num_seqs=4, max_batched_tokens=16, max_model_len=64,
                   max_tokens=56, page_size=8, device="cpu", ops=ref_ops)
    assert tight.generate(prompts, **kw) == alone
    assert tight.stats()["preemptions"] > 0


def test_top_k_top_p_and_penalty_through_the_entry_point(tiny_models):
    eng = Engine(tiny_models["A"], "float32", max_num_seqs=2, max_batched_tokens=32, max_model_len=64,
                 device="cpu", ops=ref_ops)
    a = eng.generate([[1, 2, 3]], max_new_tokens=12, temperature=0.8, top_k=5, top_p=0.9, repetition_penalty=1.3)
    b = eng.generate([[1, 2, 3]], max_new_tokens=12, temperature=0.8, top_k=5, top_p=0.9, repetition_penalty=1.3)
    assert a == b and len(a[0]) == 12
    assert eng.generate([[1, 2, 3]], max_new_tokens=4, temperature=1.0, top_k=1) == \
        eng.generate([[1, 2, 3]], max_new_tokens=4, temperature=0.0)


def test_array_uniforms_and_incremental_histories():
    """The array form of the per-request random numbers gives the scalar form's numbers, and a history kept up
    token by token (also across a list that was replaced by a shorter one) counts what a recount counts."""
    import random
    from collections import Counter
    import numpy as np
    from zig_ai_b200.sampling.sampler import _History, uniform, uniforms
    g = random.Random(5)
    seeds = [g.randrange(-9, 1 << 70) for _ in range(500)]
    idx = [g.randrange(0, 1 << 22) for _ in range(500)]
    assert [float(np.float32(uniform(s, i))) for s, i in zip(seeds, idx)] == [float(v) for v in uniforms(seeds, idx)]
    h, out = _History(), []
    for step in range(300):
        out.append(g.randrange(40) if step % 3 else g.randrange(100000))
        if step in (120, 250):
            out = out[:7]                                    # (a request that was started again)
        h.update(out)
        got = dict(zip(h.tokens[:h.n].tolist(), h.counts[:h.n].tolist()))
        assert got == dict(Counter(out)), step
