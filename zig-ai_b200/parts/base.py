"""What a model is made of: descriptions (data) and the interfaces of the parts.

A model is a `ModelSpec`: a list of `LayerSpec`s, each naming its parts by kind with their sizes
and constants as parameters, and an `order`, the list of layer calls that one forward pass makes.
The reference builds its layers by switching on `is_lfm2` / `is_attention`
(src/transformer/hybrid_layer.zig:186-221) and runs them in index order (src/main.zig:846-861);
here both the choice of parts and the order are data, so that one model can mix parts layer by
layer, run a layer twice, or let a layer read the cache another layer wrote.

No part knows which model it is in: a part sees its own parameters, its own tensors, the
step's batch description and its own piece of the cache.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple


# --------------------------------------------------------------------------- descriptions
@dataclass
class PartSpec:
    """A part by kind, with its sizes and constants."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass
class LayerSpec:
    prefix: str                 # prefix of this layer's tensor names, e.g. "blk.3."
    block: PartSpec             # arrangement of the parts below (which norm where, which sums)
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    ff_norm: PartSpec


@dataclass
class LayerCall:
    """One entry of the running order.  `cache_of` names an earlier entry of the order whose cache
    this call reads instead of owning one (it then writes nothing into it)."""
    layer: int
    cache_of: Optional[int] = None


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: List[LayerSpec]
    order: List[LayerCall]
    final_norm: PartSpec
    head: PartSpec


# --------------------------------------------------------------------------- tensors a part owns
@dataclass
class ParamDecl:
    """A tensor a part expects: its shape and what it is ('matrix' follows the model's dtype,
    'vector' (norm weights, conv taps, biases) is kept in 32-bit, 'table' is the embedding)."""
    shape: Tuple[int, ...]
    role: str = "matrix"
    alt_shapes: Tuple[Tuple[int, ...], ...] = ()   # other stored layouts accepted and reshaped
    init: str = "normal"    # random-weights mode: "normal" N(0, 0.02^2), "norm_weight" 1 + U(-0.1, 0.1),
                            # "conv" N(0, 0.1^2)


# --------------------------------------------------------------------------- cache needs
@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every position (window None) or of the last `window` positions."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size state per request, zero for a new request, kept in 32-bit."""
    shape: Tuple[int, ...]


# --------------------------------------------------------------------------- the residual stream
class Residual:
    """The 32-bit residual stream of a step.  A holder, because a fused kernel writes the updated
    stream into a fresh buffer (other blocks of that kernel still read the old one)."""

    def __init__(self, data):
        self.data = data


class LazyNorm:
    """A norm that has not run yet: `norm(residual + delta) * gamma`, optionally on gathered rows.
    A product kernel that can apply it on the fly takes it as its input (`ops.linear`,
    `ops.linear_swiglu`); anything else calls `materialize`."""

    def __init__(self, residual: Residual, delta, gamma, eps: float, dtype, rows=None):
        self.residual, self.delta, self.gamma, self.eps, self.dtype, self.rows = residual, delta, gamma, eps, dtype, rows

    @property
    def shape(self):
        n = self.rows.numel() if self.rows is not None else self.residual.data.shape[0]
        return (n, self.residual.data.shape[1])

    def materialize(self, ops):
        if self.rows is not None:
            h = ops.gather_add(self.residual.data, self.delta, self.rows)
            return ops.add_rmsnorm(h, None, self.gamma, self.eps, self.dtype)
        return ops.add_rmsnorm(self.residual.data, self.delta, self.gamma, self.eps, self.dtype)


# --------------------------------------------------------------------------- interfaces
class Part:
    """Base of every part.  `params()` declares tensors by local name (the layer's prefix is put
    in front by the model); `bind()` receives them on the device."""

    def params(self) -> Dict[str, ParamDecl]:
        return {}

    def bind(self, tensors: Dict[str, Any], dtype) -> None:
        for k, v in tensors.items():
            setattr(self, "w_" + k.replace(".", "_"), v)


class Mixer(Part):
    """Mixes information between positions of a request.
    forward(x [N, hidden] in the model's dtype, step, cache, write_cache) -> [N, hidden].
    A mixer (or feed-forward) whose first operation on x is `ops.linear` / `ops.linear_swiglu` may
    set `accepts_lazy_input = True`; it is then given a `LazyNorm` where a kernel can fuse the norm."""

    accepts_lazy_input = False

    def cache_need(self):
        return None

    def forward(self, x, step, cache, write_cache: bool = True):
        raise NotImplementedError


class FeedForward(Part):
    """forward(x [N, hidden], step) -> [N, hidden]"""

    accepts_lazy_input = False

    def forward(self, x, step):
        raise NotImplementedError


class Norm(Part):
    """forward(h, delta or None, step) -> normed [N, hidden] in the model's dtype.  `h` is the
    32-bit residual stream, a `Residual` (or a plain tensor); `delta` is added into it first (the
    residual sum is 32-bit).  With `lazy=True` the norm may return a `LazyNorm` for a product
    kernel to apply; with `rows` only those rows are normed (the stream is left as it is)."""

    def forward(self, h, delta, step, lazy=False, rows=None):
        raise NotImplementedError


class PositionEncoding(Part):
    """Either describes itself as a rotation the fused kernel can apply (`rotary()` returns
    (rotary_dim, theta)), or transforms q and k itself in `apply`."""

    def rotary(self) -> Optional[Tuple[int, float]]:
        return None

    def apply(self, q, k, positions, step):
        raise NotImplementedError


class Block(Part):
    """Arrangement of a layer's parts.  forward(h, pending, step, cache, write_cache) ->
    (h, pending): `h` is the 32-bit residual stream (a `Residual`) and `pending` a term not yet
    added to it, so that the addition can be fused with the next norm."""

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, ff_norm: Norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.ff_norm = mixer_norm, ff_norm

    def forward(self, h, pending, step, cache, write_cache: bool = True):
        raise NotImplementedError


# --------------------------------------------------------------------------- registries of parts
_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {},
}


def register_part(family: str, kind: str, factory: Callable, replace: bool = False) -> None:
    """Make a part available under `kind` in one of the families mixer, feed_forward, norm,
    position, block.  `factory(**params)` returns the part (a block's factory also gets its
    four parts)."""
    reg = _REGISTRIES[family]
    if kind in reg and not replace:
        raise ValueError(f"{family} '{kind}' is already registered")
    reg[kind] = factory


def unregister_part(family: str, kind: str) -> None:
    _REGISTRIES[family].pop(kind, None)


def make_part(family: str, spec: PartSpec, *args):
    reg = _REGISTRIES[family]
    if spec.kind not in reg:
        raise ValueError(f"unknown {family} '{spec.kind}'; registered: {', '.join(sorted(reg)) or '(none)'}")
    return reg[spec.kind](*args, **spec.params)
