"""Typed configuration and the architecture registry."""
import copy
import json

import pytest

from neurogrid_b200.config import (ConfigError, Lfm2Config, config_from_dict, load_config,
                                   register_architecture, registered_architectures)
from tiny_configs import TINY_A, TINY_B, TINY_C


def test_tiny_a_and_b_differ_in_every_size_and_option():
    a, b = config_from_dict(TINY_A), config_from_dict(TINY_B)
    for f in ("vocab_size", "hidden_size", "num_hidden_layers", "layer_types", "num_attention_heads",
              "num_key_value_heads", "head_dim", "intermediate_size", "block_auto_adjust_ff_dim", "conv_L_cache",
              "conv_bias", "tie_embedding", "rope_theta", "norm_eps", "max_position_embeddings"):
        assert getattr(a, f) != getattr(b, f), f


def test_derived_sizes():
    a = config_from_dict(TINY_A)
    assert a.head_dim == 16 and a.intermediate_size == 192
    assert config_from_dict(TINY_B).intermediate_size == 256
    assert config_from_dict(TINY_C).intermediate_size == 192          # int(1.3 * 133) = 172 -> 8 * 24
    # the published shapes: block_ff_dim -> SwiGLU width
    for ff, want in ((12288, 8192), (6656, 4608), (10240, 6912)):
        assert Lfm2Config.ffn_width(ff, True, 256, 1.0) == want


def test_round_trip_and_spec():
    for d in (TINY_A, TINY_B, TINY_C):
        c = config_from_dict(d)
        assert config_from_dict(c.to_dict()) == c
        spec = c.model_spec()
        assert len(spec.layers) == c.num_hidden_layers == len(spec.schedule)
        kinds = [l.mixer.kind for l in spec.layers]
        assert kinds == ["short_conv" if t == "conv" else "attention" for t in c.layer_types]
        assert spec.tie_head == c.tie_embedding


def test_fallback_keys():
    d = copy.deepcopy(TINY_A)
    d["rms_norm_eps"] = d.pop("norm_eps")
    d["intermediate_size"] = d.pop("block_ff_dim")
    d["tie_word_embeddings"] = d.pop("tie_embedding")
    del d["architectures"]                                  # model_type "lfm2" still finds the class
    assert config_from_dict(d) == config_from_dict(TINY_A)
    d["rope_parameters"] = {"rope_theta": d.pop("rope_theta"), "rope_type": "default"}
    assert config_from_dict(d) == config_from_dict(TINY_A)


def test_no_position_limit_in_the_config():
    d = copy.deepcopy(TINY_B)
    del d["max_position_embeddings"]
    c = config_from_dict(d)
    assert c.max_position_embeddings == 0 and c.model_spec().max_positions == 0
    assert config_from_dict(c.to_dict()) == c


@pytest.mark.parametrize("mutate,needle", [
    (lambda d: d.pop("hidden_size"), "hidden_size"),
    (lambda d: d.pop("rope_theta"), "rope_theta"),
    (lambda d: d.pop("norm_eps"), "norm_eps"),
    (lambda d: d.pop("block_multiple_of"), "block_multiple_of"),
    (lambda d: d.update(layer_types=["conv", "mamba", "conv", "conv"]), "layer_types[1]"),
    (lambda d: d.update(num_hidden_layers=5), "layer_types has 4"),
    (lambda d: d.update(num_key_value_heads=3), "multiple"),
    (lambda d: d.update(conv_L_cache=1), "conv_L_cache"),
    (lambda d: d.update(conv_dim=32), "conv_dim"),
    (lambda d: d.update(vocab_size="many"), "vocab_size"),
    (lambda d: d.update(architectures=["LlamaForCausalLM"]), "unknown architecture"),
])
def test_errors_name_the_key(mutate, needle):
    d = copy.deepcopy(TINY_A)
    mutate(d)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert needle in str(e.value)


def test_unknown_architecture_lists_registered():
    with pytest.raises(ConfigError) as e:
        config_from_dict({"architectures": ["Nope"]})
    assert "Lfm2ForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        config_from_dict({"model_type": "nope"})


def test_load_config_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert load_config(str(tmp_path)) == config_from_dict(TINY_B)
    with pytest.raises(ConfigError):
        load_config(str(tmp_path / "missing"))


def test_registry_takes_another_architecture():
    class Toy:
        @classmethod
        def from_dict(cls, d):
            return cls()
    register_architecture("ToyForTests", Toy, model_type="toy")
    assert "ToyForTests" in registered_architectures()
    assert isinstance(config_from_dict({"model_type": "toy"}), Toy)
