"""The layer sizes that the benchmark runs (hidden 1024, 16 query and 8 key/value heads of 64,
feed-forward 4608, vocabulary 65536), four layers deep, against the plain implementation: the kernels
are tested one by one at these sizes elsewhere; here they run as the model's chain of dependent
launches (prompt portions beside decoding requests, then decode steps replayed from graphs), where
one kernel's early start can meet another kernel's data."""
import random

import numpy as np
import pytest

import plain_lfm2
import traces

pytestmark = pytest.mark.gpu

FULL_WIDTH = {
    "architectures": ["Lfm2ForCausalLM"], "hidden_size": 1024, "num_hidden_layers": 4,
    "layer_types": ["conv", "full_attention", "full_attention", "conv"],
    "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 64,
    "block_ff_dim": 6656, "block_auto_adjust_ff_dim": True, "block_multiple_of": 256, "vocab_size": 65536,
    "rope_theta": 1000000.0, "conv_L_cache": 3, "conv_bias": False, "use_qk_norm": True, "norm_eps": 1e-5,
    "tie_embedding": True, "max_position_embeddings": 4096,
}


# the widths of the three model sizes that bench.py knows (its --model), the larger two with two layers
WIDTHS = {
    "350m": {},
    "700m": dict(hidden_size=1536, num_attention_heads=24, block_ff_dim=10752, num_hidden_layers=2,
                 layer_types=["conv", "full_attention"]),
    "1.2b": dict(hidden_size=2048, num_attention_heads=32, block_ff_dim=12288, num_hidden_layers=2,
                 layer_types=["full_attention", "conv"]),
}


@pytest.fixture(scope="module")
def full_width_models(tmp_path_factory):
    from zig_ai_b200.config import config_from_dict
    from zig_ai_b200.weights import write_random_model
    made = {}

    def get(width):
        if width not in made:
            d = str(tmp_path_factory.mktemp("full_width_" + width.replace(".", "_")))
            write_random_model(config_from_dict(dict(FULL_WIDTH, **WIDTHS[width])), 41, d, matrix_std="fan_in")
            made[width] = d
        return made[width]
    return get


@pytest.mark.parametrize("width,dtype", [("350m", "bfloat16"), ("350m", "float32"), ("700m", "bfloat16"), ("1.2b", "bfloat16")])
def test_benchmark_layer_sizes_against_plain(full_width_models, width, dtype):
    from zig_ai_b200.engine.runner import load_runner
    d = full_width_models(width)
    c, W = plain_lfm2.read_config(d), plain_lfm2.read_weights(d)
    g = random.Random(43)
    V = c["vocab_size"]
    lengths = {"a": 600, "b": 40, "c": 1, "d": 257, "e": 130}
    toks = {k: [g.randrange(V) for _ in range(n)] for k, n in lengths.items()}
    runner = load_runner(d, dtype, max_tokens=4096, page_size=64, max_requests=8)
    for k in toks:
        runner.add_request(k)
    got, rows = {k: [] for k in toks}, {k: [] for k in toks}

    def run(entries):
        out = runner.step(entries).cpu().numpy()
        at = 0
        for k, new, want in entries:
            base = runner.processed[k] - len(new)
            for w in want:
                assert np.isfinite(out[at]).all(), (k, base + w)
                got[k].append(out[at].copy())
                rows[k].append(base + w)
                at += 1
        assert at == out.shape[0]

    # the prompts in portions: a in three (320, 200, 80), the others whole beside them
    run([("a", toks["a"][:320], [0, 255, 256, 319]), ("b", toks["b"], [39])])
    run([("c", toks["c"], [0]), ("a", toks["a"][320:520], [0, 199]), ("d", toks["d"], [0, 256])])
    run([("a", toks["a"][520:], [79]), ("e", toks["e"], [129])])
    # decode steps of all five (a graph of single tokens), some with a request left out
    for step in range(12):
        live = [k for k in toks if not (step % 5 == 3 and k == "b")]
        entries = []
        for k in live:
            t = g.randrange(V)
            toks[k].append(t)
            entries.append((k, [t], [0]))
        run(entries)
    if dtype == "bfloat16":
        assert runner.graphs.replays >= 10
    for k in toks:
        want = plain_lfm2.forward(c, W, toks[k], rows=rows[k]).numpy()
        traces.check_request(np.stack(got[k]), want, dtype, f"{dtype} request {k}")


@pytest.mark.parametrize("width,page_size", [("350m", 64), ("1.2b", 16)])
def test_serving_at_full_width_leaves_nothing_behind(full_width_models, width, page_size):
    """A hundred and twenty requests of 3 to 4000 prompt tokens, greedy and sampled (top-k, top-p, repetition
    penalty), arriving while others run, through a pool too small for all of them at once: every request ends with the length
    it asked for (or is refused pages it can never have), the kernels' status word stays clear, and no page, state
    slot or row of the sampler's table of counts is held at the end."""
    import torch
    import zig_ai_b200 as z
    from zig_ai_b200.kernels import ops
    from zig_ai_b200.sampling import SamplingParams
    d = full_width_models(width)
    g = random.Random(7)
    eng = z.Engine(d, "bfloat16", max_num_seqs=24, max_batched_tokens=1024, max_model_len=4096, max_tokens=24 * 1024,
                   page_size=page_size)
    V = 65536
    pending = []
    for i in range(120):
        n = g.choice([3, 17, 64, 200, 700, 1500, 3500]) + g.randrange(50)
        sp = dict(max_new_tokens=g.choice([1, 8, 40, 150]), seed=i)
        kind = g.randrange(5)
        if kind == 0:
            sp.update(temperature=0.0)
        elif kind == 1:
            sp.update(temperature=0.9)
        elif kind == 2:
            sp.update(temperature=0.8, top_k=g.choice([1, 40, 5000]), top_p=g.choice([1.0, 0.9]))
        elif kind == 3:
            sp.update(temperature=1.2, top_p=0.95, repetition_penalty=1.2)
        else:
            sp.update(temperature=0.0, repetition_penalty=1.5)
        pending.append(([g.randrange(V) for _ in range(n)], SamplingParams(**sp)))
    done, added, asked = 0, 0, {}
    while done < len(pending):
        while added < len(pending) and (g.random() < 0.3 or not eng.has_work()):
            rid = eng.add_request(*pending[added])
            asked[rid] = pending[added][1].max_new_tokens
            added += 1
        for r in eng.step():
            done += 1
            assert r.finish_reason in ("length", "out_of_pages"), r.finish_reason
            assert r.finish_reason != "length" or len(r.output) == asked[r.request_id]
    eng.flush()
    torch.cuda.synchronize()
    st = eng.stats()
    assert ops.read_status() == 0
    assert not eng.sampler._slots and not eng.requests
    assert all(v == 0 for k, v in st.items() if k.endswith("pages_used"))
