"""The one place where tensor names of other naming schemes are mapped onto the canonical names.

The canonical names are the GGUF ones the reference loads LFM2 by: `token_embd.weight`,
`token_embd_norm.weight`, `output.weight` (src/loader/gguf_model.zig:36-78) and `blk.{i}.<part>`
(src/transformer/hybrid_layer.zig:295, short_conv.zig:155-163, hybrid_attn.zig:250-267).  The
reference accepts further spellings in several places, each next to the code that loads the tensor;
here they are one table:

* per-layer aliases of the projections, the feed-forward and the two norms
  (src/transformer/layer.zig:244-253; src/loader/gguf.zig:470-533),
* `output_norm.weight` for the final norm (src/loader/gguf_model.zig:66-70),
* the per-layer prefix `model.layers.{i}.` with `self_attn.*_proj`, `mlp.*_proj`, `input_layernorm`,
  `post_attention_layernorm` (src/transformer/layer.zig:216-226, src/loader/safetensors.zig:9).

A scheme is added by adding rows; nothing else in the loader knows a name.  `rope_freqs.weight`
(src/loader/gguf.zig:487) carries nothing this engine reads and is passed over with a note.
"""
from __future__ import annotations

import re
from typing import Dict, Iterable, List, Tuple

# prefix of a layer's tensors in another scheme -> the canonical prefix
LAYER_PREFIXES: List[Tuple[str, str]] = [
    (r"^model\.layers\.(\d+)\.", r"blk.\1."),
    (r"^layers\.(\d+)\.", r"blk.\1."),
]

# name of a tensor inside a layer (after the prefix) in another scheme -> the canonical one
LAYER_ALIASES: Dict[str, str] = {
    "wq.weight": "attn_q.weight", "wk.weight": "attn_k.weight", "wv.weight": "attn_v.weight",
    "wo.weight": "attn_output.weight", "attn_o.weight": "attn_output.weight",
    "self_attn.q_proj.weight": "attn_q.weight", "self_attn.k_proj.weight": "attn_k.weight",
    "self_attn.v_proj.weight": "attn_v.weight", "self_attn.o_proj.weight": "attn_output.weight",
    "mlp.gate_proj.weight": "ffn_gate.weight", "mlp.up_proj.weight": "ffn_up.weight",
    "mlp.down_proj.weight": "ffn_down.weight",
    "feed_forward.w1.weight": "ffn_gate.weight", "feed_forward.w3.weight": "ffn_up.weight",
    "feed_forward.w2.weight": "ffn_down.weight",
    "input_layernorm.weight": "attn_norm.weight", "post_attention_layernorm.weight": "ffn_norm.weight",
}

# names outside the layers
GLOBAL_ALIASES: Dict[str, str] = {
    "output_norm.weight": "token_embd_norm.weight",
}

# tensors that a file may carry and this engine never reads
PASSED_OVER = ("rope_freqs.weight",)

_LAYER = re.compile(r"^(blk\.\d+\.)(.+)$")


def canonical_name(stored: str) -> str:
    """The canonical name of a tensor stored under `stored` (itself, if no row of the table applies)."""
    name = GLOBAL_ALIASES.get(stored, stored)
    for pattern, prefix in LAYER_PREFIXES:
        renamed, n = re.subn(pattern, prefix, name)
        if n:
            name = renamed
            break
    m = _LAYER.match(name)
    if m:
        name = m.group(1) + LAYER_ALIASES.get(m.group(2), m.group(2))
    return name


def resolve(stored_names: Iterable[str]):
    """canonical name -> stored name for every stored tensor, the canonical names stored more than once
    (under one spelling in two files, or under two spellings), and the names passed over."""
    by_canonical, twice, passed = {}, [], []
    for stored in stored_names:
        if stored in PASSED_OVER:
            passed.append(stored)
            continue
        c = canonical_name(stored)
        if c in by_canonical:
            twice.append(c if by_canonical[c] == stored else f"{c} (as {by_canonical[c]} and as {stored})")
            continue
        by_canonical[c] = stored
    return by_canonical, twice, passed
