"""Configuration of the LFM2 ShortConv hybrid, read from its own config.json keys.

The reference reads the same facts from GGUF metadata (src/loader/model_config.zig:96-128):
`lfm2.embedding_length`, `lfm2.block_count`, `attention.head_count`, the per-layer
`attention.head_count_kv` array whose non-zero entries mark the attention layers (:101-124),
`attention.layer_norm_rms_epsilon` (:61), `rope.freq_base` (:63), `shortconv.l_cache` (:127) and
`feed_forward_length` (:58).  Here `conv_L_cache` is the number of taps of the depthwise
convolution (its state holds one row less), and the feed-forward width may be derived from
`block_ff_dim` by the auto-adjust rule.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, ModelConfig, read_key

ARCHITECTURE = "Lfm2ForCausalLM"
CONV = "conv"
ATTENTION = "full_attention"


def adjusted_ff_dim(block_ff_dim: int, auto_adjust: bool, multiplier: Optional[float], multiple_of: int) -> int:
    """Width of the SwiGLU feed-forward.  With auto-adjust: two thirds of `block_ff_dim`
    (rounded down), times `multiplier` if given (rounded down), rounded up to a multiple of
    `multiple_of`; otherwise `block_ff_dim` itself."""
    if not auto_adjust:
        return block_ff_dim
    f = (2 * block_ff_dim) // 3
    if multiplier is not None:
        f = int(math.floor(multiplier * f))
    return multiple_of * ((f + multiple_of - 1) // multiple_of)


MAX_CONV_TAPS = 16      # ZAI_MAX_TAPS of csrc/shortconv.cu


@dataclass
class Lfm2Config(ModelConfig):
    hidden_size: int = 0
    num_hidden_layers: int = 0
    layer_types: List[str] = field(default_factory=list)
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    vocab_size: int = 0
    norm_eps: float = 1e-5
    rope_theta: float = 1000000.0
    conv_L_cache: int = 3
    conv_bias: bool = False
    block_ff_dim: int = 0
    block_auto_adjust_ff_dim: bool = False
    block_ffn_dim_multiplier: Optional[float] = None
    block_multiple_of: int = 256
    use_qk_norm: bool = True
    tie_embedding: bool = True
    max_position_embeddings: int = 128000

    @property
    def ff_dim(self) -> int:
        return adjusted_ff_dim(self.block_ff_dim, self.block_auto_adjust_ff_dim,
                               self.block_ffn_dim_multiplier, self.block_multiple_of)

    @property
    def attention_layers(self) -> List[int]:
        return [i for i, t in enumerate(self.layer_types) if t == ATTENTION]

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Lfm2Config":
        n_layers = read_key(d, "num_hidden_layers", int)
        if n_layers < 1:
            raise ConfigError("num_hidden_layers should be at least 1")
        has_types = d.get("layer_types") is not None
        has_idxs = d.get("full_attn_idxs") is not None
        if has_types == has_idxs:
            raise ConfigError("give exactly one of 'layer_types' and 'full_attn_idxs'")
        if has_types:
            layer_types = read_key(d, "layer_types", list)
            if len(layer_types) != n_layers:
                raise ConfigError(
                    f"layer_types has {len(layer_types)} entries but num_hidden_layers is {n_layers}")
            for t in layer_types:
                if t not in (CONV, ATTENTION):
                    raise ConfigError(f"unknown layer type {t!r}; known: '{CONV}', '{ATTENTION}'")
        else:
            idxs = read_key(d, "full_attn_idxs", list)
            for i in idxs:
                if not isinstance(i, int) or isinstance(i, bool) or not 0 <= i < n_layers:
                    raise ConfigError(f"full_attn_idxs entry {i!r} is not a layer index below {n_layers}")
            if len(set(idxs)) != len(idxs):
                raise ConfigError("full_attn_idxs names a layer twice")
            layer_types = [ATTENTION if i in set(idxs) else CONV for i in range(n_layers)]

        hidden = read_key(d, "hidden_size", int)
        heads = read_key(d, "num_attention_heads", int)
        kv_heads = read_key(d, "num_key_value_heads", int, heads)
        if hidden < 1 or heads < 1 or kv_heads < 1:
            raise ConfigError("hidden_size, num_attention_heads and num_key_value_heads should be positive")
        if heads % kv_heads != 0:
            raise ConfigError(f"num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}")
        if d.get("head_dim") is None and hidden % heads != 0:
            raise ConfigError(f"hidden_size {hidden} is not a multiple of num_attention_heads {heads}; give head_dim")
        head_dim = read_key(d, "head_dim", int, hidden // heads)
        if head_dim < 2 or head_dim % 2 != 0:
            raise ConfigError(f"head_dim {head_dim} should be even (rotary pairs)")

        if d.get("block_ff_dim") is None and d.get("intermediate_size") is not None:
            block_ff, auto = read_key(d, "intermediate_size", int), False
        else:
            block_ff = read_key(d, "block_ff_dim", int)
            auto = read_key(d, "block_auto_adjust_ff_dim", bool, False)
        multiple_of = read_key(d, "block_multiple_of", int, 256)
        mult = read_key(d, "block_ffn_dim_multiplier", float, None)
        if block_ff < 1 or multiple_of < 1 or (mult is not None and mult <= 0):
            raise ConfigError("block_ff_dim, block_multiple_of and block_ffn_dim_multiplier should be positive")

        taps = read_key(d, "conv_L_cache", int, 3)
        if taps < 1:
            raise ConfigError(f"conv_L_cache {taps} should be at least 1")
        if taps > MAX_CONV_TAPS:
            raise ConfigError(f"conv_L_cache {taps} is more than the {MAX_CONV_TAPS} taps the convolution kernels take")
        vocab = read_key(d, "vocab_size", int)
        if vocab < 1:
            raise ConfigError("vocab_size should be positive")
        eps = read_key(d, "norm_eps", float, 1e-5)
        theta = read_key(d, "rope_theta", float, 1000000.0)
        if eps <= 0 or theta <= 0:
            raise ConfigError("norm_eps and rope_theta should be positive")
        max_pos = read_key(d, "max_position_embeddings", int, 128000)
        if max_pos < 1:
            raise ConfigError("max_position_embeddings should be positive")
        tie = read_key(d, "tie_embedding", bool, None)
        if tie is None:
            tie = read_key(d, "tie_word_embeddings", bool, True)
        return cls(
            architecture=ARCHITECTURE, hidden_size=hidden, num_hidden_layers=n_layers,
            layer_types=layer_types, num_attention_heads=heads, num_key_value_heads=kv_heads,
            head_dim=head_dim, vocab_size=vocab, norm_eps=eps, rope_theta=theta,
            conv_L_cache=taps, conv_bias=read_key(d, "conv_bias", bool, False),
            block_ff_dim=block_ff, block_auto_adjust_ff_dim=auto, block_ffn_dim_multiplier=mult,
            block_multiple_of=multiple_of, use_qk_norm=read_key(d, "use_qk_norm", bool, True),
            tie_embedding=tie, max_position_embeddings=max_pos)

    def to_dict(self) -> Dict[str, Any]:
        d = {k: v for k, v in self.field_dict().items() if k != "architecture"}
        if d["block_ffn_dim_multiplier"] is None:
            del d["block_ffn_dim_multiplier"]
        return {"architectures": [self.architecture], "model_type": "lfm2", **d}
