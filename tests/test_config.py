import json

import pytest

import tiny_models
from ayaka_py_b200.config import ConfigError, EngineConfig, GPT2Config
from ayaka_py_b200.registry import architecture_for, read_config, registered_architectures


def test_defaults_are_gpt2_small():
    c = GPT2Config()
    assert (c.vocab_size, c.n_embd, c.n_layer, c.n_head, c.n_positions) == (50257, 768, 12, 12, 1024)
    assert c.inner_size == 3072 and c.head_dim == 64 and c.activation_function == "gelu_new"
    assert c.attention_scale(0) == 64 ** -0.5 == c.attention_scale(7)


def test_short_and_long_spellings():
    a = GPT2Config.from_dict({"n_embd": 96, "n_head": 2, "n_layer": 3, "n_inner": 320, "layer_norm_epsilon": 1e-6})
    b = GPT2Config.from_dict({"hidden_size": 96, "num_attention_heads": 2, "num_hidden_layers": 3,
                              "intermediate_size": 320, "layer_norm_eps": 1e-6, "unknown_key": 1})
    assert a == b and a.inner_size == 320
    with pytest.raises(ConfigError):
        GPT2Config.from_dict({"n_embd": 96, "hidden_size": 64})


def test_inverse_layer_scaling_and_unscaled():
    c = GPT2Config.from_dict(tiny_models.TINY_B)
    assert c.attention_scale(2) == pytest.approx(48 ** -0.5 / 3)
    assert GPT2Config(scale_attn_weights=False).attention_scale(5) == 1.0


@pytest.mark.parametrize("bad", [
    {"n_embd": 100, "n_head": 3}, {"n_layer": 0}, {"vocab_size": -1}, {"n_head": 2.5},
    {"activation_function": "relu"}, {"layer_norm_epsilon": 0.0}, {"layer_norm_epsilon": float("nan")},
    {"n_inner": 0}, {"tie_word_embeddings": "yes"}, {"n_embd": True},
])
def test_rejections(bad):
    with pytest.raises(ConfigError):
        GPT2Config.from_dict(bad)


def test_registry(tmp_path):
    assert "GPT2LMHeadModel" in registered_architectures()
    assert architecture_for({"architectures": ["GPT2LMHeadModel"]}).model_type == "gpt2"
    assert architecture_for({"model_type": "gpt2"}).name == "GPT2LMHeadModel"
    with pytest.raises(ConfigError, match="GPT2LMHeadModel"):
        architecture_for({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError):
        read_config(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(tiny_models.TINY_A))
    arch, cfg = read_config(tmp_path)
    assert cfg.n_embd == 64 and cfg.to_dict()["architectures"] == ["GPT2LMHeadModel"]


def test_spec_has_no_size_of_its_own():
    cfg = GPT2Config.from_dict(tiny_models.TINY_B)
    spec = architecture_for(cfg.to_dict()).build_spec(cfg)
    assert len(spec.layers) == 3 and [s.layer for s in spec.order] == [0, 1, 2]
    m = spec.layers[2].part("mixer")
    assert m.params["head_dim"] == 48 and m.params["num_heads"] == 2
    assert m.params["scale"] == pytest.approx(48 ** -0.5 / 3)
    assert spec.layers[0].part("ffn").params == {"width": 96, "inner": 320, "activation": "gelu_erf", "bias": True}
    assert spec.layers[0].part("norm1").params["eps"] == 1e-6
    assert spec.head.sources["weight"].name == "transformer.wte.weight"
    untied = GPT2Config.from_dict({**tiny_models.TINY_B, "tie_word_embeddings": False})
    assert architecture_for(untied.to_dict()).build_spec(untied).head.sources["weight"].name == "lm_head.weight"


def test_engine_config():
    e = EngineConfig(dtype="bf16")
    assert e.dtype == "bfloat16" and e.page_size == 16 and e.kv_pages == 1024 and e.batch_tokens == 256
    for bad in ({"page_size": 12}, {"kv_pages": 1}, {"dtype": "fp8"}, {"batch_tokens": 0}):
        with pytest.raises(ConfigError):
            EngineConfig(**bad)


def test_command_line_says_what_is_wrong_in_one_line(tmp_path, capsys):
    """A folder without config.json, an architecture nobody registered, a configuration that
    contradicts itself: status 1 or 2 and one line on standard error, no traceback."""
    import json

    from ayaka_py_b200.commands.cli import main

    assert main(["generate", str(tmp_path / "nowhere"), "--prompt-ids", "5"]) != 0
    said = capsys.readouterr()
    assert "config.json" in said.err + said.out
    other = tmp_path / "other"
    other.mkdir()
    (other / "config.json").write_text(json.dumps({"architectures": ["SomethingElseLM"], "model_type": "else"}))
    assert main(["generate", str(other), "--prompt-ids", "5"]) == 1
    err = capsys.readouterr().err
    assert "unknown architecture 'SomethingElseLM'" in err and "GPT2LMHeadModel" in err and "Traceback" not in err
    odd = tmp_path / "odd"
    odd.mkdir()
    (odd / "config.json").write_text(json.dumps({"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
                                                 "n_embd": 65, "n_head": 4}))
    assert main(["generate", str(odd), "--prompt-ids", "5"]) == 1
    err = capsys.readouterr().err
    assert "n_embd (65) must be divisible by n_head (4)" in err and len(err.strip().splitlines()) == 1
