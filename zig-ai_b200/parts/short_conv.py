"""ShortConv mixer: a gated short causal depthwise convolution.

    bcx = x . W_in^T          -> B, C, x~ (thirds of the last dimension, per token)
    u   = B * x~
    y[t, c] = sum_j w[c, j] * u_[t - (L-1) + j, c]  (+ b[c])     u_ = conv state ++ u
    out = (C * y) . W_out^T

Tap j = L-1 multiplies the current token, the indexing of the reference's device kernel
(src/cuda/layer_kernels.cu:206-213); the state is the last L-1 rows of u_ (ibid. :216-221,
src/transformer/short_conv.zig:228-233) and is kept in 32-bit, one slot per request
(the reference keeps one inside the layer object, short_conv.zig:63-64).  Tensor names:
short_conv.zig:155-163.  The operator order (projection, gate, convolution, gate, projection,
no activation) is the LFM2 operator; the reference convolves the normed input and applies SiLU
(short_conv.zig:184-271).
"""
from __future__ import annotations

from .base import Mixer, ParamDecl, StateNeed, register_part


MAX_TAPS = 16      # ZAI_MAX_TAPS of csrc/shortconv.cu


class ShortConv(Mixer):
    accepts_lazy_input = True     # x goes straight into a product
    graph_safe = True      # forward launches kernels only; nothing is read back to the host

    def __init__(self, hidden: int, conv_dim: int, taps: int, bias: bool):
        self.hidden, self.conv_dim, self.taps, self.bias = int(hidden), int(conv_dim), int(taps), bool(bias)
        if self.taps < 1:
            raise ValueError("a convolution needs at least one tap")
        if self.taps > MAX_TAPS:
            raise ValueError(f"{self.taps} taps are more than the {MAX_TAPS} the convolution kernels take")

    def params(self):
        p = {
            "shortconv.in_proj.weight": ParamDecl((3 * self.conv_dim, self.hidden)),
            "shortconv.conv.weight": ParamDecl((self.conv_dim, self.taps), "vector",
                                               alt_shapes=((self.conv_dim, 1, self.taps),), init="conv"),
            "shortconv.out_proj.weight": ParamDecl((self.hidden, self.conv_dim)),
        }
        if self.bias:
            p["shortconv.conv.bias"] = ParamDecl((self.conv_dim,), "vector", init="conv")
        return p

    def cache_need(self):
        # a convolution with one tap needs no history; keep one row so that the slot exists
        return StateNeed((max(self.taps - 1, 1), self.conv_dim))

    def bind(self, tensors, dtype):
        self.w_in = tensors["shortconv.in_proj.weight"]
        self.w_out = tensors["shortconv.out_proj.weight"]
        self.conv_w = tensors["shortconv.conv.weight"].reshape(self.conv_dim, self.taps).contiguous()
        self.conv_b = tensors.get("shortconv.conv.bias")
        self.dtype = dtype

    def forward(self, x, step, cache, write_cache=True):
        ops = step.ops
        z = ops.linear_short_conv(x, self.w_in, self.conv_w, self.conv_b, cache.state, step, self.taps, write_cache)
        return ops.linear(z, self.w_out)


register_part("mixer", "short_conv", ShortConv)
