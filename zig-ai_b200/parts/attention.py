"""Grouped-query attention over the paged cache.

    q = x.Wq^T [N,Hq,D]   k = x.Wk^T, v = x.Wv^T [N,Hkv,D]       (no biases)
    q, k = rms(q, q_norm), rms(k, k_norm)  per head over D           (if qk_norm)
    q, k = position(q, k)                                           (v is neither normed nor rotated)
    k, v of the new positions are written into the request's pages
    s = q.k^T * scale over the request's cached positions <= the query's (and inside the window)
    out = softmax(s).v  -> [N, Hq*D] . Wo^T

Reference: projections src/transformer/hybrid_attn.zig:285-354, per-head norm :371-382 (device
:719,723), scale 1/sqrt(D) :571, causal mask :587, softmax :578-600, query head hq reads kv head
hq // (Hq/Hkv) :553-569 and src/cuda/paged_attention.cu:142, output projection :622-640; tensor
names :250-267.  Softmax and the norms are 32-bit.
"""
from __future__ import annotations

import math

import torch

from .base import Mixer, PagedKVNeed, ParamDecl, make_part, register_part, PartSpec


class Attention(Mixer):
    accepts_lazy_input = True     # x goes straight into a product
    graph_safe = True      # forward launches kernels only; nothing is read back to the host

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, qk_norm: bool, eps: float,
                 position: PartSpec, window=None, scale=None, kv_proj: bool = True):
        self.hidden, self.heads, self.kv_heads, self.head_dim = int(hidden), int(heads), int(kv_heads), int(head_dim)
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads cannot share {self.kv_heads} key/value heads evenly")
        self.qk_norm, self.eps = bool(qk_norm), float(eps)
        self.window = None if window is None else int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.kv_proj = bool(kv_proj)
        self.position = make_part("position", position)

    def params(self):
        q_dim, kv_dim = self.heads * self.head_dim, self.kv_heads * self.head_dim
        p = {"attn_q.weight": ParamDecl((q_dim, self.hidden)),
             "attn_output.weight": ParamDecl((self.hidden, q_dim))}
        if self.kv_proj:
            p["attn_k.weight"] = ParamDecl((kv_dim, self.hidden))
            p["attn_v.weight"] = ParamDecl((kv_dim, self.hidden))
        if self.qk_norm:
            p["attn_q_norm.weight"] = ParamDecl((self.head_dim,), "vector", init="norm_weight")
            if self.kv_proj:
                p["attn_k_norm.weight"] = ParamDecl((self.head_dim,), "vector", init="norm_weight")
        return p

    def cache_need(self):
        return PagedKVNeed(self.kv_heads, self.head_dim, self.window)

    def bind(self, tensors, dtype):
        mats = [tensors["attn_q.weight"]]
        if self.kv_proj:
            mats += [tensors["attn_k.weight"], tensors["attn_v.weight"]]
        self.w_qkv = torch.cat(mats, dim=0).contiguous()
        self.w_o = tensors["attn_output.weight"]
        self.q_norm = tensors.get("attn_q_norm.weight")
        self.k_norm = tensors.get("attn_k_norm.weight")
        self.dtype = dtype

    def forward(self, x, step, cache, write_cache=True):
        ops = step.ops
        write = write_cache and self.kv_proj
        qkv = ops.linear(x, self.w_qkv)
        rot = self.position.rotary()
        fused = getattr(ops, "fused_decode_attention_available", None)
        if (rot is not None and step.decode_only and self.kv_proj and fused is not None
                and fused(qkv.dtype, self.heads, self.kv_heads, self.head_dim)):
            # every row is one token: norm, rotation, page write, attention and the combination of
            # the key chunks run as one kernel
            o = ops.decode_attention_fused(qkv, self.q_norm, self.k_norm, self.eps, rot[0], rot[1], step, cache,
                                           self.heads, self.kv_heads, self.head_dim, self.scale, self.window, write)
            return ops.linear(o, self.w_o)
        if rot is not None:
            q, _ = ops.qk_norm_rope(qkv, self.q_norm, self.k_norm, self.eps, rot[0], rot[1], step, cache,
                                    self.heads, self.kv_heads, self.head_dim, self.kv_proj, write, False)
        else:
            q, k = ops.qk_norm_rope(qkv, self.q_norm, self.k_norm, self.eps, 0, 1.0, step, cache,
                                    self.heads, self.kv_heads, self.head_dim, self.kv_proj, False, self.kv_proj)
            q, k = self.position.apply(q, k, step.positions, step)
            if write:
                v = qkv[:, (self.heads + self.kv_heads) * self.head_dim:]
                ops.kv_write(k, v, step, cache, self.kv_heads, self.head_dim)
        o = ops.paged_attention(q, step, cache, self.heads, self.kv_heads, self.head_dim, self.scale, self.window)
        return ops.linear(o, self.w_o)


register_part("mixer", "attention", Attention)
