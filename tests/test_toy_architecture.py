"""A third toy architecture, defined wholly in this file, that differs from LFM2 where the engine
might have wired LFM2 in: an embedding that scales its rows, a head with a bias and a soft cap on
the logits, a layer whose block has two mixers and four norms and no feed-forward, and a mixer that
keeps two things per request (a state matrix and a conv state).  It is registered, written with
random weights, loaded and stepped in mixed batches (prompt portions of some requests beside single
tokens of others, in a pool so small that pages are used again) and compared with its plain
formulas; nothing under the package changes for it.  On the CPU with the plain stand-ins of the
kernels, and on the GPU with the kernels."""
import math
import random
from dataclasses import dataclass

import pytest
import torch

import plain_lfm2 as P
import ref_ops
from zig_ai_b200.config import ModelConfig, register_architecture, unregister_architecture
from zig_ai_b200.engine.runner import load_runner
from zig_ai_b200.parts import (Block, Embedding, Head, LayerCall, LayerSpec, Mixer, ModelSpec, ParamDecl, PartSpec,
                               StateNeed, register_part, unregister_part)
from zig_ai_b200.weights import write_random_model

F64 = torch.float64
T3 = dict(hidden=40, vocab=83, heads=2, kv_heads=1, head_dim=16, theta=50.0, eps=1e-5, d=8, taps=3, decay=0.9,
          ff_dim=56, cap=3.0)


class ScaledEmbedding(Embedding):
    def __init__(self, weight, vocab, hidden, scale):
        self.weight_name, self.vocab, self.hidden, self.scale = weight, vocab, hidden, scale

    def params(self):
        return {self.weight_name: ParamDecl((self.vocab, self.hidden), "table")}

    def bind(self, tensors, dtype):
        self.table = tensors[self.weight_name]

    def forward(self, token_ids, step):
        return step.ops.embed(token_ids, self.table) * self.scale


class SoftCapHead(Head):
    """logits = cap * tanh((x . W^T + b) / cap)"""

    def __init__(self, weight, bias, cap, vocab, hidden):
        self.weight_name, self.bias_name, self.cap, self.vocab, self.hidden = weight, bias, cap, vocab, hidden

    def params(self):
        return {self.weight_name: ParamDecl((self.vocab, self.hidden)), self.bias_name: ParamDecl((self.vocab,), "vector")}

    def bind(self, tensors, dtype):
        self.w, self.b = tensors[self.weight_name], tensors[self.bias_name]

    def forward(self, x, step):
        y = step.ops.linear(x, self.w, out_dtype=torch.float32) + self.b
        return self.cap * torch.tanh(y / self.cap)


class MatrixAndConvMixer(Mixer):
    """u = causal depthwise conv of x over (conv state ++ x);  q, k, v = u Wq, u Wk, u Wv (width d);
    S_t = decay S_{t-1} + k_t^T v_t;  out_t = (q_t S_t) Wo.  Two things are kept per request: the
    matrix S [d, d] and the last taps-1 rows of x."""

    def __init__(self, hidden, d, taps, decay):
        self.hidden, self.d, self.taps, self.decay = hidden, d, taps, decay

    def params(self):
        return {"mc.conv.weight": ParamDecl((self.hidden, self.taps), "vector", init="conv"),
                "mc.q.weight": ParamDecl((self.d, self.hidden)), "mc.k.weight": ParamDecl((self.d, self.hidden)),
                "mc.v.weight": ParamDecl((self.d, self.hidden)), "mc.o.weight": ParamDecl((self.hidden, self.d))}

    def cache_need(self):
        return (StateNeed((self.d, self.d)), StateNeed((self.taps - 1, self.hidden), "model"))

    def bind(self, tensors, dtype):
        self.t = tensors

    def forward(self, x, step, cache, write_cache=True):
        matrix, conv = cache                                   # one view per need, in the order declared
        ops, L = step.ops, self.taps
        cu, slots = step.cu_q.tolist(), step.slot_ids.tolist()
        u = torch.empty_like(x)
        for s in range(step.n_seqs):
            a, b = cu[s], cu[s + 1]
            full = torch.cat([conv.state[slots[s]].to(x.dtype), x[a:b]], dim=0).float()
            acc = torch.zeros((b - a, self.hidden), dtype=torch.float32, device=x.device)
            for j in range(L):
                acc += full[j:j + (b - a)] * self.t["mc.conv.weight"][:, j][None, :]
            u[a:b] = acc.to(x.dtype)
            if write_cache:
                conv.state[slots[s]] = full[full.shape[0] - (L - 1):].to(conv.state.dtype)
        q, k, v = (ops.linear(u, self.t[n]).float() for n in ("mc.q.weight", "mc.k.weight", "mc.v.weight"))
        out = torch.empty((x.shape[0], self.d), dtype=torch.float32, device=x.device)
        for s in range(step.n_seqs):
            S = matrix.state[slots[s]].clone()
            for t in range(cu[s], cu[s + 1]):
                S = self.decay * S + k[t][:, None] * v[t][None, :]
                out[t] = q[t] @ S
            if write_cache:
                matrix.state[slots[s]] = S
        return ops.linear(out.to(x.dtype), self.t["mc.o.weight"])


class SandwichBlock(Block):
    """Two mixers, each between a norm before and a norm after it, and no feed-forward:
        h += post_a(mixer_a(pre_a(h)));   h += post_b(mixer_b(pre_b(h)))"""

    def __init__(self, mixer_a, mixer_b, norms):
        super().__init__()
        self.pre_a, self.post_a, self.pre_b, self.post_b = (self.sub(f"norm{i}", "norm", n) for i, n in enumerate(norms))
        self.mixer_a = self.sub("mixer_a", "mixer", mixer_a)
        self.mixer_b = self.sub("mixer_b", "mixer", mixer_b)

    def forward(self, h, pending, step, cache, write_cache=True):
        r = self.pre_a.forward(h, pending, step)
        m = self.mixer_a.forward(r, step, self.cache_for(self.mixer_a, cache), write_cache)
        m = self.post_a.forward(m.float(), None, step)
        r = self.pre_b.forward(h, m, step)
        m = self.mixer_b.forward(r, step, self.cache_for(self.mixer_b, cache), write_cache)
        return h, self.post_b.forward(m.float(), None, step)


@dataclass
class Toy3Config(ModelConfig):
    @classmethod
    def from_dict(cls, d):
        return cls("Toy3ForTests")

    def to_dict(self):
        return {"architectures": ["Toy3ForTests"]}


def toy3_spec(cfg):
    a, H = T3, T3["hidden"]
    norm = lambda name: PartSpec("rmsnorm", dict(size=H, eps=a["eps"], weight=name))
    att = PartSpec("attention", dict(hidden=H, heads=a["heads"], kv_heads=a["kv_heads"], head_dim=a["head_dim"], qk_norm=False,
                                     eps=a["eps"], position=PartSpec("rotary_half_split", dict(head_dim=a["head_dim"], theta=a["theta"]))))
    mc = PartSpec("toy_matrix_conv", dict(hidden=H, d=a["d"], taps=a["taps"], decay=a["decay"]))
    layers = [
        LayerSpec("l0.", PartSpec("toy_sandwich", dict(mixer_a=att, mixer_b=mc, norms=[norm(f"n{i}.weight") for i in range(4)]))),
        LayerSpec("l1.", PartSpec("prenorm_residual", dict(mixer=mc, feed_forward=PartSpec("swiglu", dict(hidden=H, ff_dim=a["ff_dim"])),
                                                           mixer_norm=norm("a.weight"), ff_norm=norm("b.weight")))),
    ]
    return ModelSpec("Toy3ForTests", H, a["vocab"], 256,
                     PartSpec("toy_scaled_embedding", dict(weight="emb.weight", scale=math.sqrt(H))),
                     layers, [LayerCall(0), LayerCall(1), LayerCall(0)], norm("final.weight"),
                     PartSpec("toy_softcap_head", dict(weight="head.weight", bias="head.bias", cap=a["cap"])))


def toy3_plain(W, tokens):
    a, T = T3, len(tokens)
    pos = torch.arange(T)

    def matrix_conv(r, pre):
        u = P.causal_depthwise_conv(r, W[pre + "mc.conv.weight"], None)
        q, k, v = (u @ W[pre + f"mc.{n}.weight"].T for n in "qkv")
        S, rows = torch.zeros((a["d"], a["d"]), dtype=F64), []
        for t in range(T):
            S = a["decay"] * S + k[t][:, None] * v[t][None, :]
            rows.append(q[t] @ S)
        return torch.stack(rows) @ W[pre + "mc.o.weight"].T

    def attention(r, pre):
        q = P.rotary_half_split((r @ W[pre + "attn_q.weight"].T).view(T, a["heads"], a["head_dim"]), pos, a["theta"])
        k = P.rotary_half_split((r @ W[pre + "attn_k.weight"].T).view(T, a["kv_heads"], a["head_dim"]), pos, a["theta"])
        v = (r @ W[pre + "attn_v.weight"].T).view(T, a["kv_heads"], a["head_dim"])
        return P.causal_attention(q, k, v, 1 / math.sqrt(a["head_dim"]), None).reshape(T, -1) @ W[pre + "attn_output.weight"].T

    def sandwich(h):
        n = lambda x, i: P.rms_norm(x, W[f"l0.n{i}.weight"], a["eps"])
        h = h + n(attention(n(h, 0), "l0."), 1)
        return h + n(matrix_conv(n(h, 2), "l0."), 3)

    h = W["emb.weight"][torch.tensor(tokens)] * math.sqrt(a["hidden"])
    h = sandwich(h)
    h = h + matrix_conv(P.rms_norm(h, W["l1.a.weight"], a["eps"]), "l1.")
    h = h + P.swiglu(P.rms_norm(h, W["l1.b.weight"], a["eps"]), W, "l1.")
    h = sandwich(h)                                            # layer 0 again, with caches of its own
    y = P.rms_norm(h, W["final.weight"], a["eps"]) @ W["head.weight"].T + W["head.bias"]
    return a["cap"] * torch.tanh(y / a["cap"])


@pytest.fixture
def toy3_registered():
    register_part("embedding", "toy_scaled_embedding", ScaledEmbedding)
    register_part("head", "toy_softcap_head", SoftCapHead)
    register_part("mixer", "toy_matrix_conv", MatrixAndConvMixer)
    register_part("block", "toy_sandwich", SandwichBlock)
    register_architecture("Toy3ForTests", Toy3Config, toy3_spec)
    yield
    for family, kind in (("embedding", "toy_scaled_embedding"), ("head", "toy_softcap_head"), ("mixer", "toy_matrix_conv"),
                         ("block", "toy_sandwich")):
        unregister_part(family, kind)
    unregister_architecture("Toy3ForTests")


def run_toy3(tmp_path, device):
    cfg = Toy3Config("Toy3ForTests")
    d = write_random_model(cfg, 53, str(tmp_path / "toy3"), matrix_std="fan_in")
    kw = dict(device="cpu", ops=ref_ops) if device == "cpu" else {}
    runner = load_runner(d, "float32", max_tokens=96, max_requests=3, page_size=4, **kw)
    # layer call 0 and 2: pages + matrix + conv state; call 1: matrix + conv state: three groups, planes counted per group
    kinds = [type(g.need).__name__ for g in runner.cache.groups]
    assert kinds == ["PagedKVNeed", "StateNeed", "StateNeed"]
    assert runner.cache.where == [[(0, 0), (1, 0), (2, 0)], [(1, 1), (2, 1)], [(0, 1), (1, 2), (2, 2)]]
    W = P.read_weights(d)
    g = random.Random(7)
    lengths = {"x": 37, "y": 14, "z": 29, "w": 22}
    reqs = {k: [g.randrange(T3["vocab"]) for _ in range(n)] for k, n in lengths.items()}
    want = {k: toy3_plain(W, t) for k, t in reqs.items()}
    got, at = {k: [] for k in reqs}, {}
    waiting, live = list(reqs), []
    while waiting or live:
        while waiting and len(live) < 3 and sum(-(-lengths[k] // 4) * 4 for k in live + waiting[:1]) <= 96:
            k = waiting.pop(0)
            runner.add_request(k)
            live.append(k)
            at[k] = 0
        entries = []
        for k in live:
            left = len(reqs[k]) - at[k]
            n = 1 if left <= len(reqs[k]) // 3 else min(g.choice([2, 3, 5, 8]), left)
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
        out = runner.step(entries)
        row = 0
        for k, t, w in entries:
            got[k].append(out[row:row + len(w)].double().cpu())
            row += len(w)
            at[k] += len(t)
        for k in [k for k in live if at[k] == len(reqs[k])]:
            runner.end_request(k)
            live.remove(k)
        runner.cache.check()
    assert runner.cache.pages_reused > 0
    for k in reqs:
        err = (torch.cat(got[k]) - want[k]).abs().max() / want[k].abs().max()
        assert err < 5e-5, (k, float(err))


def test_third_toy_architecture_on_the_cpu_stand_ins(toy3_registered, tmp_path):
    run_toy3(tmp_path, "cpu")


@pytest.mark.gpu
def test_third_toy_architecture_on_the_gpu(toy3_registered, tmp_path):
    run_toy3(tmp_path, "cuda")
