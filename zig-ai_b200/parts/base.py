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
    """A layer: the prefix of its tensor names and its block.  What the layer consists of is the
    block's business: its `params` name the sub-parts as `PartSpec`s (a pre-norm residual block: a
    mixer, a feed-forward and two norms; another block may have two mixers, four norms, or no
    feed-forward).  The four optional fields are a shorthand for exactly that common set and are
    handed to the block beside its own parameters."""
    prefix: str                 # prefix of this layer's tensor names, e.g. "blk.3."
    block: PartSpec             # arrangement of the layer's parts (which norm where, which sums) and the parts themselves
    mixer: Optional[PartSpec] = None
    feed_forward: Optional[PartSpec] = None
    mixer_norm: Optional[PartSpec] = None
    ff_norm: Optional[PartSpec] = None

    def block_params(self) -> Dict[str, Any]:
        extra = {k: getattr(self, k) for k in ("mixer", "feed_forward", "mixer_norm", "ff_norm") if getattr(self, k) is not None}
        return {**extra, **self.block.params}


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
# A part that keeps something between steps says so with one need, or with a tuple of needs (keys and
# values in pages beside a state, a state matrix beside a conv state); it then gets one `CacheView`
# per need, in that order.  A paged need describes what a page holds through `page_shape`; the cache
# manager asks for nothing else, so a cache of one latent vector per position is a need like any other.
@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every position (window None) or of the last `window` positions; a page is
    [2, kv_heads, page_size, head_dim] in the model's dtype."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def page_shape(self, page_size: int) -> Tuple[int, ...]:
        return (2, self.kv_heads, page_size, self.head_dim)

    def elements_per_token(self) -> int:
        return 2 * self.kv_heads * self.head_dim


@dataclass(frozen=True)
class PagedRowsNeed:
    """One vector of `width` elements per position (all positions, or the last `window`); a page is
    [page_size, width] in the model's dtype."""
    width: int
    window: Optional[int] = None

    def page_shape(self, page_size: int) -> Tuple[int, ...]:
        return (page_size, self.width)

    def elements_per_token(self) -> int:
        return self.width


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size state per request, zero for a new request, kept in `dtype` (32-bit by default;
    "model" stands for the model's dtype)."""
    shape: Tuple[int, ...]
    dtype: Any = "float32"


def needs_of(part) -> Tuple:
    """A part's cache needs as a tuple (empty if it keeps nothing)."""
    need = part.cache_need() if hasattr(part, "cache_need") else None
    if need is None:
        return ()
    return tuple(need) if isinstance(need, (tuple, list)) else (need,)


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
        """None, one need, or a tuple of needs; `forward` gets an empty `CacheView`, one `CacheView`, or a
        tuple of them accordingly."""
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
    added to it, so that the addition can be fused with the next norm.

    A block builds its own sub-parts from the `PartSpec`s among its parameters with `sub(name, family,
    spec)`; the model learns of them through `parts()` (tensors, graph safety) and `cache_needs()` (the
    needs of all sub-parts, in the order of `parts()`).  `cache` is the list of this layer call's
    `CacheView`s in that same order; `cache_for(part, cache)` picks a sub-part's share."""

    def __init__(self):
        self._subparts: Dict[str, Part] = {}

    def sub(self, name: str, family: str, spec):
        """Build (or take, if it is built already) the sub-part `name` and remember it."""
        if not hasattr(self, "_subparts"):
            self._subparts = {}
        part = make_part(family, spec) if isinstance(spec, PartSpec) else spec
        self._subparts[name] = part
        return part

    def parts(self) -> Dict[str, Part]:
        return dict(getattr(self, "_subparts", {}))

    def cache_needs(self) -> Tuple:
        out = ()
        for part in self.parts().values():
            out += needs_of(part)
        return out

    def cache_for(self, part, cache):
        """The share of this layer call's cache views that belongs to `part`: an empty view, one view, or
        a tuple of views, as `part.cache_need()` declared."""
        from ..cache.manager import CacheView
        views = cache if isinstance(cache, (list, tuple)) else [cache]
        at = 0
        for other in self.parts().values():
            n = len(needs_of(other))
            if other is part:
                need = part.cache_need()
                if n == 0:
                    return CacheView()
                mine = tuple(views[at:at + n])
                return mine if isinstance(need, (tuple, list)) else mine[0]
            at += n
        raise ValueError("the part does not belong to this block")

    def forward(self, h, pending, step, cache, write_cache: bool = True):
        raise NotImplementedError


class Embedding(Part):
    """Token ids to the first residual stream: forward(token_ids int32 [N], step) -> 32-bit [N, hidden].
    Built with the model's `vocab` and `hidden` beside its own parameters."""

    def forward(self, token_ids, step):
        raise NotImplementedError


class Head(Part):
    """The last step: forward(x, step) -> 32-bit logits [rows, vocab].  `x` is the output of the final
    norm at the wanted rows: a tensor in the model's dtype, or a `LazyNorm` if `accepts_lazy_input`.
    A head that shares the embedding's table sets `tied = True`, declares no tensor of its own and is
    given the embedding part through `tie(embedding)` after both are bound."""

    accepts_lazy_input = False
    tied = False

    def tie(self, embedding) -> None:
        raise NotImplementedError

    def forward(self, x, step):
        raise NotImplementedError


# --------------------------------------------------------------------------- registries of parts
_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {}, "embedding": {}, "head": {},
}


def register_part(family: str, kind: str, factory: Callable, replace: bool = False) -> None:
    """Make a part available under `kind` in one of the families mixer, feed_forward, norm,
    position, block, embedding, head.  `factory(**params)` returns the part."""
    reg = _REGISTRIES[family]
    if kind in reg and not replace:
        raise ValueError(f"{family} '{kind}' is already registered")
    reg[kind] = factory


def unregister_part(family: str, kind: str) -> None:
    _REGISTRIES[family].pop(kind, None)


def make_part(family: str, spec: PartSpec, *args, **defaults):
    """The part that `spec` describes.  `defaults` are parameters the caller supplies unless the spec
    names them itself (the model's vocabulary and width for an embedding or a head)."""
    reg = _REGISTRIES[family]
    if spec.kind not in reg:
        raise ValueError(f"unknown {family} '{spec.kind}'; registered: {', '.join(sorted(reg)) or '(none)'}")
    return reg[spec.kind](*args, **{**defaults, **spec.params})


def make_block(layer: LayerSpec):
    """The block of a layer, with the layer's sub-part specs among its parameters."""
    return make_part("block", PartSpec(layer.block.kind, layer.block_params()))
