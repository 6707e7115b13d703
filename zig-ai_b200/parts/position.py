"""Position encodings.

Rotary embedding in the half-split pairing: for i < rotary_dim/2 the pair (x[i], x[i + rotary_dim/2])
is rotated by the angle pos * theta^(-2i/rotary_dim) (the reference's device kernel,
src/cuda/layer_kernels.cu:343-366; its host version pairs (2i, 2i+1), src/transformer/rope.zig:41-53).
The position is the token's absolute position in its request.  Angles are computed in 32-bit.
"""
from __future__ import annotations

from .base import PositionEncoding, register_part


class RotaryHalfSplit(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, rotary_dim: int = None):
        self.head_dim = int(head_dim)
        self.rotary_dim = int(head_dim if rotary_dim is None else rotary_dim)
        self.theta = float(theta)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} should be even and at most head_dim {self.head_dim}")

    def rotary(self):
        return self.rotary_dim, self.theta


class NoPosition(PositionEncoding):
    def __init__(self, head_dim: int = 0):
        self.head_dim = head_dim

    def rotary(self):
        return 0, 1.0


register_part("position", "rotary_half_split", RotaryHalfSplit)
register_part("position", "none", NoPosition)
