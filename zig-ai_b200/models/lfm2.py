"""The LFM2 ShortConv hybrid as a list of layers made from parts.

Every layer is a pre-norm residual block with a SwiGLU feed-forward; its mixer is the ShortConv
or grouped-query attention according to `layer_types` (the reference decides per layer from the
`attention.head_count_kv` array, src/loader/model_config.zig:101-124 and
src/transformer/hybrid_layer.zig:186-221).  Tensor names are the reference's: `token_embd.weight`,
`token_embd_norm.weight`, `output.weight` (src/loader/gguf_model.zig:36-78) and `blk.{i}.…`
(src/transformer/hybrid_layer.zig:295).  When the embedding is tied the head uses the embedding
table (gguf_model.zig:47-54).
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.lfm2 import ARCHITECTURE, ATTENTION, Lfm2Config
from ..parts.base import LayerCall, LayerSpec, ModelSpec, PartSpec


def build_spec(cfg: Lfm2Config) -> ModelSpec:
    layers = []
    for i, kind in enumerate(cfg.layer_types):
        if kind == ATTENTION:
            mixer = PartSpec("attention", dict(
                hidden=cfg.hidden_size, heads=cfg.num_attention_heads, kv_heads=cfg.num_key_value_heads,
                head_dim=cfg.head_dim, qk_norm=cfg.use_qk_norm, eps=cfg.norm_eps,
                position=PartSpec("rotary_half_split", dict(head_dim=cfg.head_dim, theta=cfg.rope_theta))))
        else:
            mixer = PartSpec("short_conv", dict(
                hidden=cfg.hidden_size, conv_dim=cfg.hidden_size, taps=cfg.conv_L_cache, bias=cfg.conv_bias))
        layers.append(LayerSpec(prefix=f"blk.{i}.", block=PartSpec("prenorm_residual", dict(
            mixer=mixer,
            feed_forward=PartSpec("swiglu", dict(hidden=cfg.hidden_size, ff_dim=cfg.ff_dim)),
            mixer_norm=PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.norm_eps, weight="attn_norm.weight")),
            ff_norm=PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.norm_eps, weight="ffn_norm.weight"))))))
    return ModelSpec(
        architecture=ARCHITECTURE,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("embedding", dict(weight="token_embd.weight")),
        layers=layers,
        order=[LayerCall(i) for i in range(len(layers))],
        final_norm=PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.norm_eps, weight="token_embd_norm.weight")),
        head=PartSpec("linear_head", dict(weight="output.weight", tied=cfg.tie_embedding)),
    )


register_architecture(ARCHITECTURE, Lfm2Config, build_spec, replace=True)
