"""Configuration, registry, safetensors reading and writing, and the weight errors (no GPU)."""
import json
import os

import pytest
import torch

import tiny
from hipinfer_b200.config import (ConfigError, LlamaConfig, config_from_dict, get_architecture, load_config,
                                  registered_architectures)
from hipinfer_b200.parts.spec import spec_param_specs
from hipinfer_b200.weights import (ModelFiles, ParamSpec, WeightError, load_weights, random_weights, save_safetensors,
                                   write_random_model)


def test_llama_config_reads_every_key():
    c = config_from_dict(tiny.TINY_B)
    assert isinstance(c, LlamaConfig)
    assert (c.vocab_size, c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (384, 96, 320, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (3, 1, 32)
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 500000.0 and not c.tie_word_embeddings
    assert c.rope_scaling.factor == 32.0 and c.rope_scaling.original_max_position_embeddings == 64
    again = config_from_dict(c.to_dict())
    assert again == c


def test_llama_config_defaults():
    d = dict(tiny.TINY_A)
    for k in ("head_dim", "num_key_value_heads", "rope_theta", "rms_norm_eps", "tie_word_embeddings", "rope_scaling"):
        d.pop(k)
    c = config_from_dict(d)
    assert c.head_dim == 16 and c.num_key_value_heads == 4 and c.rope_theta == 10000.0
    assert c.rms_norm_eps == 1e-6 and c.tie_word_embeddings is False and c.rope_scaling is None


@pytest.mark.parametrize("change,match", [
    (dict(architectures=["NoSuchModel"]), "not registered"),
    (dict(architectures=[]), "architectures"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(attention_bias=True), "attention_bias"),
    (dict(mlp_bias=True), "mlp_bias"),
    (dict(num_key_value_heads=3), "multiple"),
    (dict(head_dim=15), "even"),
    (dict(vocab_size="256"), "vocab_size"),
    (dict(vocab_size=0), "positive"),
    (dict(rope_scaling=dict(rope_type="yarn", factor=2.0)), "rope_type"),
    (dict(rope_scaling=dict(rope_type="llama3", factor=2.0)), "low_freq_factor"),
    (dict(rms_norm_eps=True), "rms_norm_eps"),
])
def test_config_errors(change, match):
    d = dict(tiny.TINY_A)
    d.update(change)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(d)


def test_config_missing_key_and_file(tmp_path):
    d = dict(tiny.TINY_A)
    d.pop("intermediate_size")
    with pytest.raises(ConfigError, match="intermediate_size"):
        config_from_dict(d)
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(str(tmp_path))


def test_registry_lists_llama():
    assert "LlamaForCausalLM" in registered_architectures()
    arch = get_architecture("LlamaForCausalLM")
    spec = arch.build_spec(config_from_dict(tiny.TINY_A))
    assert len(spec.layers) == 2 and [s.layer for s in spec.order] == [0, 1]
    assert spec.head.params.get("tied_to") == "model.embed_tokens.weight"


def test_safetensors_roundtrip_matches_the_library(tmp_path):
    from safetensors.torch import load_file, save_file

    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int64),
         "c": torch.randn(2, 2, 2), "d": torch.randn(4).to(torch.float16), "e": torch.empty(0, 3)}
    p = str(tmp_path / "model.safetensors")
    save_safetensors(t, p, {"k": "v"})
    theirs = load_file(p)
    for k in t:
        assert torch.equal(theirs[k], t[k]) and theirs[k].dtype == t[k].dtype
    save_file(t, str(tmp_path / "x.safetensors"))
    os.replace(str(tmp_path / "x.safetensors"), p)
    mf = ModelFiles(str(tmp_path))
    for k in t:
        assert torch.equal(mf.get(k), t[k])
    mf.close()


def test_storage_policy(tmp_path):
    """16-bit floats are kept in bfloat16, integer tables become int32, 32-bit stays 32-bit."""
    t = {"h": torch.randn(4).to(torch.float16), "b": torch.randn(4).to(torch.bfloat16), "f": torch.randn(4),
         "i": torch.arange(4, dtype=torch.int64)}
    save_safetensors(t, str(tmp_path / "model.safetensors"))
    specs = [ParamSpec(k, (4,), numbers="int" if k == "i" else "float") for k in t]
    w = load_weights(str(tmp_path), specs)
    assert w["h"].dtype == torch.bfloat16 and w["b"].dtype == torch.bfloat16
    assert w["f"].dtype == torch.float32 and torch.equal(w["f"], t["f"])
    assert w["i"].dtype == torch.int32 and w["i"].tolist() == [0, 1, 2, 3]
    exact = load_weights(str(tmp_path), specs, half_as=torch.float32)   # the 32-bit engine
    assert exact["h"].dtype == torch.float32 and torch.equal(exact["h"], t["h"].float()) and exact["b"].dtype == torch.bfloat16


def test_random_model_folder_and_seed(tmp_path):
    cfg = config_from_dict(tiny.TINY_B)
    a = write_random_model(cfg, str(tmp_path / "a"), seed=2, std=0.05, norm_std=0.1)
    b = write_random_model(cfg, str(tmp_path / "b"), seed=2, std=0.05, norm_std=0.1)
    c = write_random_model(cfg, str(tmp_path / "c"), seed=3, std=0.05, norm_std=0.1)
    assert load_config(a) == cfg
    spec = get_architecture(cfg.architecture).build_spec(cfg)
    specs = spec_param_specs(spec)
    wa, wb, wc = (load_weights(p, specs) for p in (a, b, c))
    assert set(wa) == {s.name for s in specs} and "lm_head.weight" in wa
    for k in wa:
        assert torch.equal(wa[k], wb[k]) and wa[k].dtype == torch.bfloat16
    assert not torch.equal(wa["model.embed_tokens.weight"], wc["model.embed_tokens.weight"])
    e = wa["model.embed_tokens.weight"].float()
    assert abs(float(e.std()) - 0.05) < 0.005
    n = wa["model.norm.weight"].float()
    assert abs(float(n.mean()) - 1.0) < 0.05 and 0.05 < float(n.std()) < 0.15


def test_a_table_of_integers_must_be_stored_as_integers(tmp_path):
    """The other direction: a spec that asks for integers refuses floats, and keeps integers as int32."""
    specs = [ParamSpec("table", (4,), "zeros", numbers="int"), ParamSpec("w", (2, 2))]
    save_safetensors({"table": torch.zeros(4), "w": torch.zeros(2, 2)}, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightError) as ei:
        load_weights(str(tmp_path), specs)
    assert ei.value.wrong_dtype == [("table", "float32", "an integer type")]
    save_safetensors({"table": torch.arange(4, dtype=torch.int64), "w": torch.zeros(2, 2, dtype=torch.float16)},
                     str(tmp_path / "model.safetensors"))
    got = load_weights(str(tmp_path), specs)
    assert got["table"].dtype == torch.int32 and got["table"].tolist() == [0, 1, 2, 3] and got["w"].dtype == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = config_from_dict(tiny.TINY_A)
    spec = get_architecture(cfg.architecture).build_spec(cfg)
    specs = spec_param_specs(spec)
    t = random_weights(specs, 0)
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    t["lm_head.weight"] = torch.zeros(256, 64)                # tied model with a head of its own
    t["model.layers.0.mlp.down_proj.weight"] = torch.zeros(64, 127)
    t["model.layers.0.self_attn.o_proj.weight"] = torch.zeros(64, 64, dtype=torch.int32)   # integers under a weight's name
    save_safetensors(t, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightError) as ei:
        load_weights(str(tmp_path), specs)
    e = ei.value
    assert e.wrong_dtype == [("model.layers.0.self_attn.o_proj.weight", "int32", "a float type")]
    assert "wrong element type (1)" in str(e) and "o_proj.weight is int32" in str(e)
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["lm_head.weight", "model.layers.0.self_attn.q_proj.bias"]
    assert e.wrong_shape == [("model.layers.0.mlp.down_proj.weight", (64, 127), (64, 128))]
    msg = str(e)
    for frag in ("missing (2)", "unexpected (2)", "wrong shape (1)", "q_proj.bias", "[64, 127]", "expected [64, 128]"):
        assert frag in msg


def test_weight_errors_for_broken_files(tmp_path):
    specs = [ParamSpec("a", (2,))]
    with pytest.raises(WeightError, match="no model.safetensors"):
        load_weights(str(tmp_path), specs)
    (tmp_path / "model.safetensors").write_bytes(b"\x10\0\0\0\0\0\0\0{not json........")
    with pytest.raises(WeightError, match="JSON"):
        load_weights(str(tmp_path), specs)
    (tmp_path / "model.safetensors").write_bytes(b"\xff\xff\xff\xff\0\0\0\0{}")
    with pytest.raises(WeightError, match="header length"):
        load_weights(str(tmp_path), specs)


def test_sharded_folder(tmp_path):
    save_safetensors({"a": torch.ones(2)}, str(tmp_path / "m-1.safetensors"))
    save_safetensors({"b": torch.zeros(3)}, str(tmp_path / "m-2.safetensors"))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "m-1.safetensors", "b": "m-2.safetensors"}}))
    w = load_weights(str(tmp_path), [ParamSpec("a", (2,)), ParamSpec("b", (3,))])
    assert w["a"].tolist() == [1, 1] and w["b"].tolist() == [0, 0, 0]
