"""SwiGLU feed-forward: `down( silu(gate(x)) * up(x) )`, no biases
(src/transformer/ffn.zig:7-34; device activation src/cuda/layer_kernels.cu:62-70; tensor names
src/transformer/hybrid_layer.zig:313-321).  The gate and up matrices are stacked into one
[2F, hidden] matrix at load so that one product feeds the activation.
"""
from __future__ import annotations

import torch

from .base import FeedForward, ParamDecl, register_part


class SwiGlu(FeedForward):
    accepts_lazy_input = True     # x goes straight into a product
    graph_safe = True      # forward launches kernels only; nothing is read back to the host

    def __init__(self, hidden: int, ff_dim: int):
        self.hidden, self.ff_dim = int(hidden), int(ff_dim)

    def params(self):
        return {
            "ffn_gate.weight": ParamDecl((self.ff_dim, self.hidden)),
            "ffn_up.weight": ParamDecl((self.ff_dim, self.hidden)),
            "ffn_down.weight": ParamDecl((self.hidden, self.ff_dim)),
        }

    def bind(self, tensors, dtype):
        self.w_gate_up = torch.cat([tensors["ffn_gate.weight"], tensors["ffn_up.weight"]], dim=0).contiguous()
        self.w_down = tensors["ffn_down.weight"]
        self.dtype = dtype

    def forward(self, x, step):
        ops = step.ops
        a = ops.linear_swiglu(x, self.w_gate_up, self.ff_dim)
        return ops.linear(a, self.w_down)


register_part("feed_forward", "swiglu", SwiGlu)
