"""A plain, slow implementation of the LFM2 ShortConv hybrid: whole sequences, no cache, one
function for each part, float64 on the CPU.  It shares no code with the engine: it reads
config.json as a dict and the tensors with the `safetensors` package.

It rests on formulas, not on running the reference: the reference is Zig 0.16 (README.md:124-127,
build.zig.zon:4) and no Zig compiler exists on the machines this suite runs on, so its model
code can neither be imported nor compiled here; besides, its ShortConv path computes a different
operator (it convolves the normed input and applies SiLU, src/transformer/short_conv.zig:184-271)
and has no test of its own.  Each function cites the lines of the reference whose formula it
restates, and says where the LFM2 operator departs from them.
"""
from __future__ import annotations

import json
import math
import os

import torch

F64 = torch.float64


# ----------------------------------------------------------------------------- configuration
def read_config(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def feed_forward_width(c):
    """Two thirds of block_ff_dim, times the multiplier, rounded up to a multiple, when
    auto-adjust is on; else block_ff_dim.  (The reference reads the width directly from
    `feed_forward_length`, src/loader/model_config.zig:58.)"""
    if "block_ff_dim" not in c and "intermediate_size" in c:
        return c["intermediate_size"]
    f = c["block_ff_dim"]
    if not c.get("block_auto_adjust_ff_dim", False):
        return f
    f = int(2 * f / 3)
    m = c.get("block_ffn_dim_multiplier")
    if m is not None:
        f = int(m * f)
    k = c.get("block_multiple_of", 256)
    return k * ((f + k - 1) // k)


def layer_kinds(c):
    """'conv' or 'full_attention' for every layer (the reference marks attention layers by a
    non-zero entry of `attention.head_count_kv`, src/loader/model_config.zig:101-124,137-149)."""
    if c.get("layer_types") is not None:
        return list(c["layer_types"])
    idx = set(c["full_attn_idxs"])
    return ["full_attention" if i in idx else "conv" for i in range(c["num_hidden_layers"])]


def read_weights(model_dir):
    from safetensors import safe_open
    out = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k).to(F64)
    return out


# ----------------------------------------------------------------------------- parts
def rms_norm(x, gamma, eps):
    """x * rsqrt(mean(x^2) + eps) * gamma over the last dimension (src/transformer/norm.zig:14-32;
    device kernel src/cuda/layer_kernels.cu:17-43)."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x / torch.sqrt(ms + eps) * gamma


def rotary_half_split(x, positions, theta, rotary_dim=None):
    """x [T, heads, D].  For i < n/2 the pair (x[i], x[i+n/2]) turns by pos * theta^(-2i/n)
    (src/cuda/layer_kernels.cu:353-365, with the position taken as the token's own absolute
    position instead of that kernel's `row % N`, :351)."""
    T, Hh, D = x.shape
    n = D if rotary_dim is None else rotary_dim
    half = n // 2
    i = torch.arange(half, dtype=F64)
    freq = theta ** (-2.0 * i / n)
    ang = positions.to(F64)[:, None] * freq[None, :]            # [T, half]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:n]
    out = x.clone()
    out[..., :half] = a * cos - b * sin
    out[..., half:n] = a * sin + b * cos
    return out


def causal_attention(q, k, v, scale, window=None):
    """q [T,Hq,D], k,v [T,Hkv,D] of one request.  Scores q.k * scale (src/transformer/hybrid_attn.zig:571),
    keys after the query masked (:587), max-subtracted softmax (:578-600), query head hq reads
    key/value head hq // (Hq/Hkv) (:553-569, src/transformer/gqa.zig:28-30).  With a window a
    query at position p sees keys p-window+1 .. p."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    group = Hq // Hkv
    out = torch.zeros_like(q)
    pos = torch.arange(T)
    mask = pos[None, :] > pos[:, None]
    if window is not None:
        mask = mask | (pos[None, :] <= pos[:, None] - window)
    for h in range(Hq):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = s.masked_fill(mask, float("-inf"))
        s = s - s.max(dim=-1, keepdim=True).values
        p = torch.exp(s)
        p = p / p.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, kh, :]
    return out


def attention_mixer(r, W, pre, c, positions=None, window=None):
    """Projections without bias (src/transformer/hybrid_attn.zig:285-354), per-head RMSNorm of q
    and k over D with the block's eps (:371-382, device :719,723), rotation of q and k but not v,
    attention, output projection (:622-640).  Tensor names: :250-267."""
    T = r.shape[0]
    Hq, Hkv = c["num_attention_heads"], c.get("num_key_value_heads", c["num_attention_heads"])
    D = c.get("head_dim", c["hidden_size"] // Hq)
    eps = c.get("norm_eps", 1e-5)
    q = (r @ W[pre + "attn_q.weight"].T).view(T, Hq, D)
    k = (r @ W[pre + "attn_k.weight"].T).view(T, Hkv, D)
    v = (r @ W[pre + "attn_v.weight"].T).view(T, Hkv, D)
    if c.get("use_qk_norm", True):
        q = rms_norm(q, W[pre + "attn_q_norm.weight"], eps)
        k = rms_norm(k, W[pre + "attn_k_norm.weight"], eps)
    if positions is None:
        positions = torch.arange(T)
    theta = c.get("rope_theta", 1000000.0)
    q = rotary_half_split(q, positions, theta)
    k = rotary_half_split(k, positions, theta)
    o = causal_attention(q, k, v, 1.0 / math.sqrt(D), window)
    return o.reshape(T, Hq * D) @ W[pre + "attn_output.weight"].T


def causal_depthwise_conv(u, w, bias):
    """y[t,c] = sum_j w[c,j] * u_[t+j, c] with u_ = (L-1 zero rows) ++ u, so tap L-1 multiplies the
    current token (the indexing of src/cuda/layer_kernels.cu:206-213 and
    src/transformer/short_conv.zig:209-225, without their SiLU)."""
    T, C = u.shape
    L = w.shape[1]
    padded = torch.cat([torch.zeros(L - 1, C, dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(L):
        y = y + padded[j:j + T, :] * w[:, j][None, :]
    if bias is not None:
        y = y + bias[None, :]
    return y


def short_conv_mixer(r, W, pre, c):
    """in_proj -> (B, C, x) as thirds of the last dimension of each token; u = B*x; causal
    depthwise convolution of u; C * y; out_proj.  Tensor names src/transformer/short_conv.zig:155-163.
    This is the LFM2 operator; the reference runs convolution and projections in another order
    with SiLU (short_conv.zig:184-271) and splits [n,3H] into planes (:481-488)."""
    Hc = W[pre + "shortconv.out_proj.weight"].shape[1]
    bcx = r @ W[pre + "shortconv.in_proj.weight"].T
    B, C, x = bcx[:, :Hc], bcx[:, Hc:2 * Hc], bcx[:, 2 * Hc:]
    w = W[pre + "shortconv.conv.weight"].reshape(Hc, -1)
    y = causal_depthwise_conv(B * x, w, W.get(pre + "shortconv.conv.bias"))
    return (C * y) @ W[pre + "shortconv.out_proj.weight"].T


def swiglu(r, W, pre):
    """down( silu(gate(x)) * up(x) ), silu(g) = g * sigmoid(g) (src/transformer/ffn.zig:19-33,
    src/cuda/layer_kernels.cu:62-70)."""
    g = r @ W[pre + "ffn_gate.weight"].T
    u = r @ W[pre + "ffn_up.weight"].T
    return (g * torch.sigmoid(g) * u) @ W[pre + "ffn_down.weight"].T


def block(h, W, i, kind, c):
    """r = rms(h, attn_norm); h += mixer(r); r2 = rms(h, ffn_norm); h += ffn(r2)
    (src/transformer/hybrid_layer.zig:364-365, 370-377, 409-422, 488-491)."""
    pre = f"blk.{i}."
    eps = c.get("norm_eps", 1e-5)
    r = rms_norm(h, W[pre + "attn_norm.weight"], eps)
    if kind == "full_attention":
        h = h + attention_mixer(r, W, pre, c)
    else:
        h = h + short_conv_mixer(r, W, pre, c)
    r2 = rms_norm(h, W[pre + "ffn_norm.weight"], eps)
    return h + swiglu(r2, W, pre)


def forward(c, W, tokens, rows=None):
    """Logits [T, vocab] for one whole sequence (only at the positions `rows` if given): embedding
    row lookup without scaling (src/transformer/embedding.zig:6-31), the blocks, the final norm
    `token_embd_norm` and the head, which is the embedding table when tied
    (src/loader/gguf_model.zig:47-54,68-78; src/main.zig:867-878)."""
    ids = torch.as_tensor(tokens, dtype=torch.long)
    h = W["token_embd.weight"][ids]
    for i, kind in enumerate(layer_kinds(c)):
        h = block(h, W, i, kind, c)
    if rows is not None:
        h = h[torch.as_tensor(list(rows), dtype=torch.long)]
    n = rms_norm(h, W["token_embd_norm.weight"], c.get("norm_eps", 1e-5))
    tied = c.get("tie_embedding", c.get("tie_word_embeddings", True))
    head = W["token_embd.weight"] if tied else W["output.weight"]
    return n @ head.T


# ----------------------------------------------------------------------------- sampling
def greedy(logits):
    """Index of the first occurrence of the maximum (src/transformer/pipeline.zig:153-181)."""
    best, idx = -float("inf"), 0
    for i, v in enumerate(logits.tolist()):
        if v > best:
            best, idx = v, i
    return idx


def sample(logits, u, temperature=1.0, top_k=0, top_p=1.0, repetition_penalty=1.0, history=()):
    """The reference's sampler with the uniform number `u` in [0,1) given from outside
    (src/transformer/pipeline.zig:25-151): repetition penalty on tokens of the history (positive
    logits divided, negative multiplied, :60-67), greedy if temperature <= 0 (:70-72), division by
    the temperature (:75-76), top-k keeps values >= the k-th largest (:79-99), top-p keeps the
    shortest prefix of the descending order whose probability reaches p (:102-138), then the first
    index, in that order, whose cumulative probability reaches u times the kept mass (:141-149).
    Without top-k, top-p and penalty the scan runs in index order (:39-52)."""
    work = [float(x) for x in logits.tolist()]
    V = len(work)
    if repetition_penalty != 1.0:
        for t in history:
            if t < V:
                if work[t] > 0:
                    work[t] /= repetition_penalty
                elif work[t] < 0:
                    work[t] *= repetition_penalty
    if temperature <= 0:
        return greedy(torch.tensor(work, dtype=F64))
    if top_k == 0 and top_p >= 1.0 and repetition_penalty == 1.0:
        m = max(work)
        e = [math.exp((v - m) / temperature) for v in work]
        r = u * sum(e)
        acc = 0.0
        for i, x in enumerate(e):
            acc += x
            if r <= acc:
                return i
        return V - 1
    work = [v / temperature for v in work]
    if 0 < top_k < V:
        kth = sorted(work, reverse=True)[top_k - 1]
        work = [v if v >= kth else -float("inf") for v in work]
    cand = [i for i in range(V) if work[i] != -float("inf")]
    cand.sort(key=lambda i: -work[i])       # stable: ties keep index order
    m = max(work[i] for i in cand)
    probs = [math.exp(work[i] - m) for i in cand]
    s = sum(probs)
    probs = [p / s for p in probs]
    cutoff, cum = len(cand), 0.0
    for j, p in enumerate(probs):
        cum += p
        if cum >= top_p:
            cutoff = j + 1
            break
    r = u * sum(probs[:cutoff])
    cum = 0.0
    for j in range(cutoff):
        cum += probs[j]
        if r <= cum:
            return cand[j]
    return cand[cutoff - 1]
