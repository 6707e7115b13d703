"""Each part alone against the plain functions, at sizes and options the LFM2 configurations do not
use (a window, a partial rotation, no q/k norm, a conv width that differs from the model width),
and a toy architecture defined here: a mixer with a state of its own, a layer that runs twice, and
a layer that reads the cache another layer wrote; and a second one with a routed feed-forward and a
position encoding that is no rotation; registered, built, loaded and stepped without a change to the
engine's files."""
import math
import os
import random
from dataclasses import dataclass

import pytest
import torch

import plain_lfm2 as P
from zig_ai_b200.cache import CacheManager
from zig_ai_b200.config import ModelConfig, register_architecture, unregister_architecture
from zig_ai_b200.engine.batch import pack_step
from zig_ai_b200.engine.runner import load_runner
from zig_ai_b200.parts import (FeedForward, LayerCall, LayerSpec, Mixer, ModelSpec, ParamDecl, PartSpec, PositionEncoding,
                               StateNeed, make_part, register_part, unregister_part)
from zig_ai_b200.weights import write_random_model
from zig_ai_b200.weights.random_init import random_tensors

pytestmark = pytest.mark.gpu
F64 = torch.float64


def cuda_ops():
    from zig_ai_b200.kernels import ops
    ops.require()
    return ops


def bind_random(part, dtype, seed):
    decls = part.params()
    t = random_tensors(decls, seed, torch.bfloat16, matrix_std="fan_in")
    dev = {k: v.to("cuda", torch.float32 if (dtype == torch.float32 or decls[k].role == "vector") else dtype)
           for k, v in t.items()}
    part.bind(dev, dtype)
    return {k: v.to(F64) for k, v in t.items()}


def run_in_portions(part, x, cuts, dtype, page_size=8):
    """Run one request's rows through a mixer in the given portions, from its cache."""
    ops = cuda_ops()
    cache = CacheManager([("own", part.cache_need())], page_size, 64, 2, dtype, torch.device("cuda"))
    cache.admit("r")
    outs, at = [], 0
    for n in cuts:
        cache.reserve("r", at + n)
        tables = {g: cache.table_rows(["r"], g, max(len(cache.requests["r"].tables[g]), 1)) for g in cache.paged_groups()}
        step = pack_step(ops, dtype, torch.device("cuda"), [("r", at, [0] * n, [], cache.requests["r"].slot)], tables)
        outs.append(part.forward(x[at:at + n].to(dtype).cuda(), step, cache.view(0, step)))
        at += n
    return torch.cat(outs).double().cpu()


def tol(dtype):
    return 3e-5 if dtype == torch.float32 else 3e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_alone_with_window_and_partial_rotation(dtype):
    H, Hq, Hkv, D, W, rot, theta = 72, 6, 3, 48, 7, 24, 500.0
    part = make_part("mixer", PartSpec("attention", dict(
        hidden=H, heads=Hq, kv_heads=Hkv, head_dim=D, qk_norm=False, eps=1e-5, window=W,
        position=PartSpec("rotary_half_split", dict(head_dim=D, theta=theta, rotary_dim=rot)))))
    Wt = bind_random(part, dtype, 1)
    T = 45
    x = torch.randn(T, H, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).to(F64)
    q = (x @ Wt["attn_q.weight"].T).view(T, Hq, D)
    k = (x @ Wt["attn_k.weight"].T).view(T, Hkv, D)
    v = (x @ Wt["attn_v.weight"].T).view(T, Hkv, D)
    pos = torch.arange(T)
    q, k = P.rotary_half_split(q, pos, theta, rot), P.rotary_half_split(k, pos, theta, rot)
    want = P.causal_attention(q, k, v, 1 / math.sqrt(D), W).reshape(T, Hq * D) @ Wt["attn_output.weight"].T
    for cuts in ([T], [9, 2, 17, 1, 1, 15]):
        got = run_in_portions(part, x, cuts, dtype)
        assert (got - want).abs().max() / want.abs().max() < tol(dtype), cuts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_short_conv_alone_with_its_own_width(dtype):
    H, C, L = 48, 80, 5
    part = make_part("mixer", PartSpec("short_conv", dict(hidden=H, conv_dim=C, taps=L, bias=True)))
    Wt = bind_random(part, dtype, 3)
    T = 23
    x = torch.randn(T, H, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16).to(F64)
    bcx = x @ Wt["shortconv.in_proj.weight"].T
    y = P.causal_depthwise_conv(bcx[:, :C] * bcx[:, 2 * C:], Wt["shortconv.conv.weight"], Wt["shortconv.conv.bias"])
    want = (bcx[:, C:2 * C] * y) @ Wt["shortconv.out_proj.weight"].T
    for cuts in ([T], [1, 3, 1, 1, 6, 4, 5, 2]):
        got = run_in_portions(part, x, cuts, dtype)
        assert (got - want).abs().max() / want.abs().max() < tol(dtype), cuts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_and_norm_alone(dtype):
    ops = cuda_ops()
    H, F = 72, 200
    ff = make_part("feed_forward", PartSpec("swiglu", dict(hidden=H, ff_dim=F)))
    Wt = bind_random(ff, dtype, 5)
    x = torch.randn(11, H, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16)
    step = pack_step(ops, dtype, torch.device("cuda"), [("r", 0, [0] * 11, [], 1)], {})
    got = ff.forward(x.to(dtype).cuda(), step).double().cpu()
    pre = {"ffn_gate.weight": Wt["ffn_gate.weight"], "ffn_up.weight": Wt["ffn_up.weight"],
           "ffn_down.weight": Wt["ffn_down.weight"]}
    want = P.swiglu(x.to(F64), pre, "")
    assert (got - want).abs().max() / want.abs().max() < tol(dtype)
    norm = make_part("norm", PartSpec("rmsnorm", dict(size=H, eps=1e-3, weight="n.weight")))
    Wn = bind_random(norm, dtype, 7)
    h = torch.randn(11, H, generator=torch.Generator().manual_seed(8)) * 4
    delta = torch.randn(11, H, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
    hd = h.clone().cuda()
    got = norm.forward(hd, delta.to(dtype).cuda(), step).double().cpu()
    want = P.rms_norm(h.to(F64) + delta.to(F64), Wn["n.weight"], 1e-3)
    assert (got - want).abs().max() / want.abs().max() < tol(dtype)
    assert torch.allclose(hd.cpu().double(), h.to(F64) + delta.to(F64), atol=1e-6)


# ----------------------------------------------------------------------------- a toy architecture
class ToyEma(Mixer):
    """out_t = (s_t) . W^T with the state s_t = decay * s_{t-1} + (1 - decay) * x_t, one state row
    per request.  Written with torch operations, as a user of the engine might write a first version."""

    def __init__(self, hidden, decay):
        self.hidden, self.decay = hidden, decay

    def params(self):
        return {"ema.proj.weight": ParamDecl((self.hidden, self.hidden))}

    def cache_need(self):
        return StateNeed((1, self.hidden))

    def bind(self, tensors, dtype):
        self.w = tensors["ema.proj.weight"]

    def forward(self, x, step, cache, write_cache=True):
        cu, slots = step.cu_q.tolist(), step.slot_ids.tolist()
        s_all = torch.empty_like(x)
        for s in range(step.n_seqs):
            st = cache.state[slots[s], 0].clone()
            for t in range(cu[s], cu[s + 1]):
                st = self.decay * st + (1 - self.decay) * x[t].float()
                s_all[t] = st.to(x.dtype)
            if write_cache:
                cache.state[slots[s], 0] = st
        return step.ops.linear(s_all, self.w)


@dataclass
class ToyConfig(ModelConfig):
    hidden_size: int = 40
    vocab_size: int = 97
    decay: float = 0.75

    @classmethod
    def from_dict(cls, d):
        return cls("ToyForTests", d["hidden_size"], d["vocab_size"], d["decay"])

    def to_dict(self):
        return {"architectures": ["ToyForTests"], "hidden_size": self.hidden_size, "vocab_size": self.vocab_size,
                "decay": self.decay}


TOY_ATT = dict(heads=4, kv_heads=2, head_dim=16, window=6, theta=100.0, rot=8, eps=1e-4)


def toy_spec(cfg):
    H, a = cfg.hidden_size, TOY_ATT
    norm = lambda name: PartSpec("rmsnorm", dict(size=H, eps=a["eps"], weight=name))
    pos = PartSpec("rotary_half_split", dict(head_dim=a["head_dim"], theta=a["theta"], rotary_dim=a["rot"]))
    att = lambda kv_proj: PartSpec("attention", dict(hidden=H, heads=a["heads"], kv_heads=a["kv_heads"],
                                                     head_dim=a["head_dim"], qk_norm=True, eps=a["eps"],
                                                     position=pos, window=a["window"], kv_proj=kv_proj))
    mixers = [PartSpec("toy_ema", dict(hidden=H, decay=cfg.decay)), att(True), att(False)]
    layers = [LayerSpec(prefix=f"l{i}.", block=PartSpec("prenorm_residual"), mixer=m,
                        feed_forward=PartSpec("swiglu", dict(hidden=H, ff_dim=56)),
                        mixer_norm=norm("a.weight"), ff_norm=norm("b.weight")) for i, m in enumerate(mixers)]
    # layer 0 runs twice (a state of its own each time); the last call reads the cache call 1 wrote
    order = [LayerCall(0), LayerCall(1), LayerCall(0), LayerCall(2, cache_of=1)]
    return ModelSpec("ToyForTests", H, cfg.vocab_size, 512, PartSpec("embedding", dict(weight="emb.weight")),
                     layers, order, norm("final.weight"), PartSpec("linear_head", dict(weight="head.weight", tied=False)))


def toy_plain(cfg, W, tokens):
    a = TOY_ATT
    T = len(tokens)
    pos = torch.arange(T)
    h = W["emb.weight"][torch.tensor(tokens)]
    kv = {}

    def ema(r, pre):
        st, rows = torch.zeros(cfg.hidden_size, dtype=F64), []
        for t in range(T):
            st = cfg.decay * st + (1 - cfg.decay) * r[t]
            rows.append(st)
        return torch.stack(rows) @ W[pre + "ema.proj.weight"].T

    def attention(r, pre, own):
        q = P.rms_norm((r @ W[pre + "attn_q.weight"].T).view(T, a["heads"], a["head_dim"]), W[pre + "attn_q_norm.weight"], a["eps"])
        q = P.rotary_half_split(q, pos, a["theta"], a["rot"])
        if own:
            k = P.rms_norm((r @ W[pre + "attn_k.weight"].T).view(T, a["kv_heads"], a["head_dim"]), W[pre + "attn_k_norm.weight"], a["eps"])
            kv["k"] = P.rotary_half_split(k, pos, a["theta"], a["rot"])
            kv["v"] = (r @ W[pre + "attn_v.weight"].T).view(T, a["kv_heads"], a["head_dim"])
        o = P.causal_attention(q, kv["k"], kv["v"], 1 / math.sqrt(a["head_dim"]), a["window"])
        return o.reshape(T, -1) @ W[pre + "attn_output.weight"].T

    for layer, kind in [(0, "ema"), (1, "own"), (0, "ema"), (2, "shared")]:
        pre = f"l{layer}."
        r = P.rms_norm(h, W[pre + "a.weight"], a["eps"])
        h = h + (ema(r, pre) if kind == "ema" else attention(r, pre, kind == "own"))
        h = h + P.swiglu(P.rms_norm(h, W[pre + "b.weight"], a["eps"]), W, pre)
    return P.rms_norm(h, W["final.weight"], a["eps"]) @ W["head.weight"].T


@pytest.fixture
def toy_registered():
    register_part("mixer", "toy_ema", ToyEma)
    register_architecture("ToyForTests", ToyConfig, toy_spec)
    yield
    unregister_part("mixer", "toy_ema")
    unregister_architecture("ToyForTests")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_is_registered_built_and_stepped(toy_registered, tmp_path, dtype):
    cfg = ToyConfig("ToyForTests")
    d = write_random_model(cfg, 31, str(tmp_path / "toy"), matrix_std="fan_in")
    runner = load_runner(d, dtype, max_tokens=256, max_requests=3, page_size=4)
    assert len(runner.cache.groups) == 2                       # the states, and one paged group with a window
    assert runner.cache.where == [[(0, 0)], [(1, 0)], [(0, 1)], [(1, 0)]]
    W = P.read_weights(d)
    g = random.Random(5)
    reqs = {k: [g.randrange(cfg.vocab_size) for _ in range(n)] for k, n in (("x", 41), ("y", 18))}
    want = {k: toy_plain(cfg, W, t) for k, t in reqs.items()}
    got = {k: [] for k in reqs}
    at = {k: 0 for k in reqs}
    for k in reqs:
        runner.add_request(k)
    while any(at[k] < len(reqs[k]) for k in reqs):
        entries = []
        for k in reqs:
            left = len(reqs[k]) - at[k]
            if left:
                n = min(g.choice([1, 1, 2, 5, 9]), left)
                entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
        out = runner.step(entries)
        row = 0
        for k, t, w in entries:
            got[k].append(out[row:row + len(w)].double().cpu())
            row += len(w)
            at[k] += len(t)
        runner.cache.check()
    held = [p for p in runner.cache.requests["x"].tables[1] if p > 0]
    assert len(held) < len(runner.cache.requests["x"].tables[1])      # the window gave pages back
    for k in reqs:
        err = (torch.cat(got[k]) - want[k]).abs().max() / want[k].abs().max()
        assert err < (5e-5 if dtype == "float32" else 3e-2), (k, float(err))


# ------------------------------------------------- a second toy: routed experts, a position encoding of its own
class ToyRoutedFeedForward(FeedForward):
    """Two experts, the router's softmax in 32-bit, every token through its best expert, the result
    weighted with the router's probability.  Torch operations; a state-free part."""

    def __init__(self, hidden, ff_dim, experts):
        self.hidden, self.ff_dim, self.experts = hidden, ff_dim, experts

    def params(self):
        p = {"router.weight": ParamDecl((self.experts, self.hidden))}
        for e in range(self.experts):
            p[f"expert{e}.up.weight"] = ParamDecl((self.ff_dim, self.hidden))
            p[f"expert{e}.down.weight"] = ParamDecl((self.hidden, self.ff_dim))
        return p

    def bind(self, tensors, dtype):
        self.t = tensors

    def forward(self, x, step):
        probs = torch.softmax(x.float() @ self.t["router.weight"].float().T, dim=-1)
        best = probs.argmax(-1)
        out = torch.zeros_like(x)
        for e in range(self.experts):
            rows = (best == e).nonzero().flatten()
            if rows.numel():
                hid = torch.relu(step.ops.linear(x[rows].contiguous(), self.t[f"expert{e}.up.weight"]))
                y = step.ops.linear(hid, self.t[f"expert{e}.down.weight"])
                out[rows] = (y.float() * probs[rows, e][:, None]).to(x.dtype)
        return out


class ToyScaledPositions(PositionEncoding):
    """Not a rotation: q and k are multiplied by 1 + position / 64 in their first dimensions.  Applied
    by the part itself (`rotary()` stays None), so the attention part runs its unfused path."""

    def __init__(self, dims):
        self.dims = dims

    def apply(self, q, k, positions, step):
        f = (1 + positions.float() / 64)[:, None]
        q, k = q.clone(), (k.clone() if k is not None else None)
        qv = q.view(q.shape[0], -1, TOY2["head_dim"])
        qv[..., :self.dims] = (qv[..., :self.dims].float() * f[..., None]).to(q.dtype)
        if k is not None:
            kv = k.view(k.shape[0], -1, TOY2["head_dim"])
            kv[..., :self.dims] = (kv[..., :self.dims].float() * f[..., None]).to(k.dtype)
        return q, k


TOY2 = dict(hidden=48, heads=3, kv_heads=3, head_dim=16, ff_dim=40, experts=2, eps=1e-5, dims=4, vocab=61)


@dataclass
class Toy2Config(ModelConfig):
    @classmethod
    def from_dict(cls, d):
        return cls("Toy2ForTests")

    def to_dict(self):
        return {"architectures": ["Toy2ForTests"]}


def toy2_spec(cfg):
    a, H = TOY2, TOY2["hidden"]
    norm = lambda name: PartSpec("rmsnorm", dict(size=H, eps=a["eps"], weight=name))
    att = PartSpec("attention", dict(hidden=H, heads=a["heads"], kv_heads=a["kv_heads"], head_dim=a["head_dim"],
                                     qk_norm=False, eps=a["eps"], position=PartSpec("toy_scaled", dict(dims=a["dims"]))))
    ff = PartSpec("toy_routed", dict(hidden=H, ff_dim=a["ff_dim"], experts=a["experts"]))
    layers = [LayerSpec(prefix=f"l{i}.", block=PartSpec("prenorm_residual"), mixer=att, feed_forward=ff,
                        mixer_norm=norm("a.weight"), ff_norm=norm("b.weight")) for i in range(2)]
    return ModelSpec("Toy2ForTests", H, a["vocab"], 256, PartSpec("embedding", dict(weight="emb.weight")),
                     layers, [LayerCall(0), LayerCall(1)], norm("final.weight"),
                     PartSpec("linear_head", dict(weight="emb.weight", tied=True)))


def toy2_plain(W, tokens):
    a = TOY2
    T = len(tokens)
    f = (1 + torch.arange(T, dtype=F64) / 64)[:, None, None]
    h = W["emb.weight"][torch.tensor(tokens)]
    for i in range(2):
        pre = f"l{i}."
        r = P.rms_norm(h, W[pre + "a.weight"], a["eps"])
        q = (r @ W[pre + "attn_q.weight"].T).view(T, a["heads"], a["head_dim"]).clone()
        k = (r @ W[pre + "attn_k.weight"].T).view(T, a["kv_heads"], a["head_dim"]).clone()
        v = (r @ W[pre + "attn_v.weight"].T).view(T, a["kv_heads"], a["head_dim"])
        q[..., :a["dims"]] *= f
        k[..., :a["dims"]] *= f
        o = P.causal_attention(q, k, v, 1 / math.sqrt(a["head_dim"]), None)
        h = h + o.reshape(T, -1) @ W[pre + "attn_output.weight"].T
        r = P.rms_norm(h, W[pre + "b.weight"], a["eps"])
        probs = torch.softmax(r @ W[pre + "router.weight"].T, dim=-1)
        best = probs.argmax(-1)
        y = torch.zeros_like(r)
        for t in range(T):
            e = int(best[t])
            y[t] = (torch.relu(r[t] @ W[pre + f"expert{e}.up.weight"].T) @ W[pre + f"expert{e}.down.weight"].T) * probs[t, e]
        h = h + y
    return P.rms_norm(h, W["final.weight"], a["eps"]) @ W["emb.weight"].T


@pytest.fixture
def toy2_registered():
    register_part("feed_forward", "toy_routed", ToyRoutedFeedForward)
    register_part("position", "toy_scaled", ToyScaledPositions)
    register_architecture("Toy2ForTests", Toy2Config, toy2_spec)
    yield
    unregister_part("feed_forward", "toy_routed")
    unregister_part("position", "toy_scaled")
    unregister_architecture("Toy2ForTests")


def test_toy_routed_feed_forward_and_position_encoding(toy2_registered, tmp_path):
    """A feed-forward with routing and a position encoding that is no rotation, both defined here,
    in a model that is built, loaded and stepped in portions beside another request; 32-bit, so that
    the comparison with the plain formulas is tight (a token near a tie of the router aside)."""
    cfg = Toy2Config("Toy2ForTests")
    d = write_random_model(cfg, 37, str(tmp_path / "toy2"), matrix_std="fan_in")
    runner = load_runner(d, "float32", max_tokens=256, max_requests=3, page_size=4)
    W = P.read_weights(d)
    g = random.Random(6)
    reqs = {k: [g.randrange(TOY2["vocab"]) for _ in range(n)] for k, n in (("x", 33), ("y", 12))}
    want = {k: toy2_plain(W, t) for k, t in reqs.items()}
    got, at = {k: [] for k in reqs}, {k: 0 for k in reqs}
    for k in reqs:
        runner.add_request(k)
    while any(at[k] < len(reqs[k]) for k in reqs):
        entries = []
        for k in reqs:
            left = len(reqs[k]) - at[k]
            if left:
                n = min(g.choice([1, 1, 3, 7]), left)
                entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
        out = runner.step(entries)
        row = 0
        for k, t, w in entries:
            got[k].append(out[row:row + len(w)].double().cpu())
            row += len(w)
            at[k] += len(t)
    for k in reqs:
        err = (torch.cat(got[k]) - want[k]).abs().max() / want[k].abs().max()
        assert err < 5e-5, (k, float(err))
