"""Configuration, registry and weight loading (no GPU)."""
import json
import os

import pytest
import torch

from tiny_configs import TINY_A, TINY_B
from zig_ai_b200.config import (ConfigError, Lfm2Config, adjusted_ff_dim, config_from_dict, known_architectures,
                                load_config)
from zig_ai_b200.models import build_model
from zig_ai_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_tensors, random_tensors,
                                 write_random_model, write_safetensors)


def test_feed_forward_rule():
    # the widths the published LFM2 shapes give: 6656 -> 4608, 10752 -> 7168, 12288 -> 8192; tiny B: 320 -> 256
    assert adjusted_ff_dim(6656, True, None, 256) == 4608
    assert adjusted_ff_dim(10752, True, None, 256) == 7168
    assert adjusted_ff_dim(12288, True, None, 256) == 8192
    assert adjusted_ff_dim(320, True, 1.0, 64) == 256
    assert adjusted_ff_dim(192, False, None, 256) == 192


def test_tiny_configs_parse_and_differ():
    a, b = config_from_dict(TINY_A), config_from_dict(TINY_B)
    assert isinstance(a, Lfm2Config) and a.ff_dim == 192 and b.ff_dim == 256
    assert b.layer_types == ["full_attention", "conv", "conv", "full_attention", "conv", "conv"]
    for f in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
              "vocab_size", "rope_theta", "conv_L_cache", "conv_bias", "norm_eps", "tie_embedding", "ff_dim"):
        assert getattr(a, f) != getattr(b, f), f
    assert config_from_dict(a.to_dict()) == a and config_from_dict(b.to_dict()) == b


@pytest.mark.parametrize("change,fragment", [
    ({"hidden_size": None}, "hidden_size"),
    ({"layer_types": ["conv"]}, "num_hidden_layers"),
    ({"layer_types": ["conv", "attn", "conv", "conv"]}, "unknown layer type"),
    ({"full_attn_idxs": [1]}, "exactly one"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"conv_L_cache": 0}, "conv_L_cache"),
    ({"conv_L_cache": 17}, "more than the 16 taps"),
    ({"norm_eps": "small"}, "norm_eps"),
    ({"architectures": ["NoSuchModel"]}, "unknown architecture"),
    ({"vocab_size": 0}, "vocab_size"),
])
def test_bad_configs_are_refused(change, fragment):
    d = dict(TINY_A)
    for k, v in change.items():
        if v is None:
            d.pop(k)
        else:
            d[k] = v
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert fragment in str(e.value)


def test_registry_lists_and_builds():
    assert "Lfm2ForCausalLM" in known_architectures()
    m = build_model(config_from_dict(TINY_B))
    kinds = [type(b.mixer).__name__ for b in m.blocks]
    assert kinds == ["Attention", "ShortConv", "ShortConv", "Attention", "ShortConv", "ShortConv"]
    decls = m.param_decls()
    assert decls["blk.1.shortconv.conv.weight"].shape == (96, 4) and "blk.1.shortconv.conv.bias" in decls
    assert "output.weight" in decls and decls["blk.0.attn_k.weight"].shape == (32, 96)
    assert "output.weight" not in build_model(config_from_dict(TINY_A)).param_decls()


def test_safetensors_roundtrip_against_the_package(tmp_path):
    from safetensors.torch import load_file, save_file
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int64), "c": torch.randn(2, 2)}
    write_safetensors(str(tmp_path / "mine.safetensors"), t)
    theirs = load_file(str(tmp_path / "mine.safetensors"))
    assert all(torch.equal(theirs[k], v) for k, v in t.items())
    save_file(t, str(tmp_path / "theirs.safetensors"))
    f = SafetensorsFile(str(tmp_path / "theirs.safetensors"))
    assert sorted(f.names()) == ["a", "b", "c"] and all(torch.equal(f.read(k), v) for k, v in t.items())


def test_truncated_and_malformed_files(tmp_path):
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, {"a": torch.randn(8, 8)})
    blob = open(p, "rb").read()
    open(p, "wb").write(blob[:-10])
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)
    open(p, "wb").write(b"\x05\x00\x00")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)


def test_load_keeps_dtypes_and_reports_all_faults(tmp_path):
    cfg = config_from_dict(TINY_B)
    d = str(tmp_path / "m")
    write_random_model(cfg, 3, d)
    assert load_config(d) == cfg
    model = build_model(cfg)
    decls = model.param_decls()
    t = load_tensors(d, decls, torch.bfloat16, "cpu")
    assert t["blk.0.attn_q.weight"].dtype == torch.bfloat16 and t["token_embd.weight"].dtype == torch.bfloat16
    assert t["blk.0.attn_norm.weight"].dtype == torch.float32 and t["blk.1.shortconv.conv.weight"].dtype == torch.float32
    t32 = load_tensors(d, decls, torch.float32, "cpu")
    assert all(v.dtype == torch.float32 for v in t32.values())
    assert torch.equal(t32["blk.0.attn_q.weight"], t["blk.0.attn_q.weight"].float())

    # a matrix stored in 32-bit stays 32-bit, an integer table becomes int32, [C,1,L] conv taps are accepted
    tensors = random_tensors(decls, 3)
    tensors["blk.0.ffn_up.weight"] = tensors["blk.0.ffn_up.weight"].float()
    tensors["blk.1.shortconv.conv.weight"] = tensors["blk.1.shortconv.conv.weight"].reshape(96, 1, 4)
    d2 = str(tmp_path / "m2")
    os.makedirs(d2)
    write_safetensors(os.path.join(d2, "model.safetensors"), tensors)
    t2 = load_tensors(d2, decls, torch.bfloat16, "cpu")
    assert t2["blk.0.ffn_up.weight"].dtype == torch.float32 and t2["blk.1.shortconv.conv.weight"].shape == (96, 4)

    # one error that lists the missing, the unexpected and the misshapen
    del tensors["blk.2.ffn_down.weight"], tensors["token_embd_norm.weight"]
    tensors["blk.9.extra.weight"] = torch.zeros(2)
    tensors["blk.0.attn_q.weight"] = torch.zeros(5, 5, dtype=torch.bfloat16)
    tensors["blk.0.attn_k.weight"] = torch.zeros(32, 96, dtype=torch.bool)
    d3 = str(tmp_path / "m3")
    os.makedirs(d3)
    write_safetensors(os.path.join(d3, "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        load_tensors(d3, decls, torch.bfloat16, "cpu")
    err = e.value
    assert sorted(err.missing) == ["blk.2.ffn_down.weight", "token_embd_norm.weight"]
    assert err.unexpected == ["blk.9.extra.weight"]
    assert [w[0] for w in err.wrong_shape] == ["blk.0.attn_q.weight"]
    assert [w[0] for w in err.wrong_dtype] == ["blk.0.attn_k.weight"]
    for word in ("missing", "unexpected", "wrong shape", "blk.9.extra.weight", "[96, 96]"):
        assert word in str(err)


def test_other_naming_schemes_load_through_the_rename_table(tmp_path):
    """A folder that spells its tensors in the other ways the reference accepts (layer.zig:244-253,
    gguf_model.zig:66-70, `model.layers.{i}.self_attn.*`) gives the same tensors; a tensor stored under
    two spellings is an error; tensors nobody asks for are an error or, if the caller says so, a list."""
    from zig_ai_b200.weights.names import canonical_name
    assert canonical_name("model.layers.3.self_attn.o_proj.weight") == "blk.3.attn_output.weight"
    assert canonical_name("blk.12.feed_forward.w3.weight") == "blk.12.ffn_up.weight"
    assert canonical_name("output_norm.weight") == "token_embd_norm.weight"
    assert canonical_name("blk.1.shortconv.conv.weight") == "blk.1.shortconv.conv.weight"
    cfg = config_from_dict(TINY_B)
    decls = build_model(cfg).param_decls()
    tensors = random_tensors(decls, 3)
    other = {"self_attn.q_proj.weight": "attn_q.weight", "wk.weight": "attn_k.weight", "self_attn.v_proj.weight": "attn_v.weight",
             "attn_o.weight": "attn_output.weight", "mlp.gate_proj.weight": "ffn_gate.weight",
             "feed_forward.w3.weight": "ffn_up.weight", "mlp.down_proj.weight": "ffn_down.weight",
             "input_layernorm.weight": "attn_norm.weight", "post_attention_layernorm.weight": "ffn_norm.weight"}
    back = {v: k for k, v in other.items()}
    renamed = {}
    for name, t in tensors.items():
        if name.startswith("blk."):
            _, i, rest = name.split(".", 2)
            name = f"model.layers.{i}." + back.get(rest, rest)
        renamed["output_norm.weight" if name == "token_embd_norm.weight" else name] = t
    assert set(renamed) != set(tensors)
    d = str(tmp_path / "renamed")
    os.makedirs(d)
    write_safetensors(os.path.join(d, "model.safetensors"), renamed)
    got = load_tensors(d, decls, torch.bfloat16, "cpu")
    assert set(got) == set(decls) and all(torch.equal(got[k].float(), tensors[k].float().reshape(got[k].shape)) for k in decls)
    assert got.renamed["blk.0.attn_q.weight"] == "model.layers.0.self_attn.q_proj.weight" and got.unused == []
    # the same tensor under two spellings
    renamed["blk.0.attn_q.weight"] = tensors["blk.0.attn_q.weight"]
    renamed["rope_freqs.weight"] = torch.zeros(4)
    renamed["model.layers.0.rotary.inv_freq"] = torch.zeros(4)
    write_safetensors(os.path.join(d, "model.safetensors"), renamed)
    with pytest.raises(WeightError) as e:
        load_tensors(d, decls, torch.bfloat16, "cpu")
    assert any("stored twice" in u and "attn_q" in u for u in e.value.unexpected)
    assert any("rotary.inv_freq" in u for u in e.value.unexpected) and not any("rope_freqs" in u for u in e.value.unexpected)
    del renamed["blk.0.attn_q.weight"]
    write_safetensors(os.path.join(d, "model.safetensors"), renamed)
    with pytest.raises(WeightError):
        load_tensors(d, decls, torch.bfloat16, "cpu")
    got = load_tensors(d, decls, torch.bfloat16, "cpu", unexpected="warn")
    assert len(got.unused) == 2 and set(got) == set(decls)


def test_random_weights_are_reproducible(tmp_path):
    cfg = config_from_dict(TINY_A)
    a, b, c = (str(tmp_path / x) for x in "abc")
    write_random_model(cfg, 5, a)
    write_random_model(cfg, 5, b)
    write_random_model(cfg, 6, c)
    fa, fb, fc = (SafetensorsFile(os.path.join(x, "model.safetensors")) for x in (a, b, c))
    for n in fa.names():
        assert torch.equal(fa.read(n), fb.read(n))
    assert not torch.equal(fa.read("token_embd.weight"), fc.read("token_embd.weight"))
    w = fa.read("blk.0.attn_norm.weight").float()
    assert 0.89 < float(w.min()) and float(w.max()) < 1.11
    assert json.load(open(os.path.join(a, "config.json")))["architectures"] == ["Lfm2ForCausalLM"]
