"""RMSNorm, fused with the residual addition that precedes it.

`out = x * rsqrt(mean(x^2) + eps) * gamma`, all in 32-bit (src/transformer/norm.zig:6-33; device
version src/cuda/layer_kernels.cu:17-43).  The reference adds residuals with separate kernels
(`addKernel`, layer_kernels.cu:46-59); here the pending term is added into the 32-bit residual
stream by the same kernel that normalises it.
"""
from __future__ import annotations

from .base import LazyNorm, Norm, ParamDecl, Residual, register_part


class RmsNorm(Norm):
    graph_safe = True      # forward launches kernels only; nothing is read back to the host

    def __init__(self, size: int, eps: float, weight: str):
        self.size, self.eps, self.weight_name = int(size), float(eps), weight
        self.weight = None

    def params(self):
        return {self.weight_name: ParamDecl((self.size,), "vector", init="norm_weight")}

    def bind(self, tensors, dtype):
        self.weight = tensors[self.weight_name]
        self.dtype = dtype

    def forward(self, h, delta, step, lazy=False, rows=None):
        res = h if isinstance(h, Residual) else Residual(h)
        x = LazyNorm(res, delta, self.weight, self.eps, self.dtype, rows)
        if lazy and getattr(step.ops, "fuses_norm", False):
            return x
        return x.materialize(step.ops)


register_part("norm", "rmsnorm", RmsNorm)
