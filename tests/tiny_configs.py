"""Two tiny configurations of the LFM2 ShortConv hybrid that differ in every size and option:
layer order and count, width, head counts and grouping, head size, feed-forward rule, vocabulary,
rotary base, number of conv taps, conv bias, the norms' eps, tied or untied head, page size."""

TINY_A = {
    "architectures": ["Lfm2ForCausalLM"],
    "hidden_size": 64, "num_hidden_layers": 4,
    "layer_types": ["conv", "full_attention", "conv", "full_attention"],
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "block_ff_dim": 192, "block_auto_adjust_ff_dim": False,
    "vocab_size": 256, "rope_theta": 10000.0, "conv_L_cache": 3, "conv_bias": False,
    "use_qk_norm": True, "norm_eps": 1e-5, "tie_embedding": True, "max_position_embeddings": 128,
}

TINY_B = {
    "architectures": ["Lfm2ForCausalLM"],
    "hidden_size": 96, "num_hidden_layers": 6,
    "full_attn_idxs": [0, 3],
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
    "block_ff_dim": 320, "block_auto_adjust_ff_dim": True, "block_ffn_dim_multiplier": 1.0,
    "block_multiple_of": 64,
    "vocab_size": 517, "rope_theta": 1000000.0, "conv_L_cache": 4, "conv_bias": True,
    "use_qk_norm": True, "norm_eps": 1e-6, "tie_embedding": False, "max_position_embeddings": 4096,
}

# A third one with the head size of the LFM2 checkpoints (64), two query heads per key/value head and
# a feed-forward wide enough for the long-row product: the whole-model tests reach through it the
# kernels that only that head size has (keys and values by TMA in decoding, the tcgen05 span
# attention) and the product that splits K across a cluster.
SMALL_C = {
    "architectures": ["Lfm2ForCausalLM"],
    "hidden_size": 256, "num_hidden_layers": 4,
    "layer_types": ["conv", "full_attention", "full_attention", "conv"],
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
    "block_ff_dim": 2304, "block_auto_adjust_ff_dim": True, "block_multiple_of": 256,
    "vocab_size": 1000, "rope_theta": 1000000.0, "conv_L_cache": 3, "conv_bias": False,
    "use_qk_norm": True, "norm_eps": 1e-5, "tie_embedding": True, "max_position_embeddings": 4096,
}

# name -> (config, seed of the random weights)
TINY = {"A": (TINY_A, 11), "B": (TINY_B, 23), "C": (SMALL_C, 29)}
PAGE_SIZE = {"A": 16, "B": 8, "C": 64}
