"""Typed configuration from config.json keys, and the architecture registry."""
import json

import pytest

from helpers import TINY
from iian_b200.config.registry import (Architecture, architecture_names, get_architecture, load_model_config,
                                       register_architecture, unregister_architecture)
from iian_b200.models.qwen3 import ConfigError, qwen3_config_from_dict


def test_every_size_comes_from_the_file():
    c = qwen3_config_from_dict(TINY["B"])
    assert (c.vocab_size, c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (503, 96, 160, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (8, 2, 32)     # head_dim != hidden / heads
    assert c.q_size == 256 and c.kv_size == 64 and c.gqa == 4
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 1e6 and not c.tie_word_embeddings


def test_defaults_are_the_references():
    raw = dict(TINY["A"])
    for k in ("num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "tie_word_embeddings"):
        raw.pop(k)
    c = qwen3_config_from_dict(raw)
    assert c.num_key_value_heads == c.num_attention_heads        # default = heads
    assert c.head_dim == raw["hidden_size"] // raw["num_attention_heads"]
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0 and c.tie_word_embeddings is False


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "max_position_embeddings"])
def test_missing_key_is_named(key):
    raw = dict(TINY["A"])
    raw.pop(key)
    with pytest.raises(ConfigError, match=key):
        qwen3_config_from_dict(raw)


def test_bad_values_are_refused():
    with pytest.raises(ConfigError, match="multiple"):
        qwen3_config_from_dict(dict(TINY["A"], num_key_value_heads=3))
    with pytest.raises(ConfigError, match="hidden_act"):
        qwen3_config_from_dict(dict(TINY["A"], hidden_act="gelu"))
    with pytest.raises(ConfigError, match="rope_scaling"):
        qwen3_config_from_dict(dict(TINY["A"], rope_scaling={"rope_type": "yarn", "factor": 4.0}))
    with pytest.raises(ConfigError, match="integer"):
        qwen3_config_from_dict(dict(TINY["A"], hidden_size="64"))
    with pytest.raises(ConfigError, match="head_dim"):
        qwen3_config_from_dict(dict(TINY["A"], head_dim=15))
    assert qwen3_config_from_dict(dict(TINY["A"], rope_scaling=None)).rope_theta == 10000.0


def test_windows_per_layer():
    c = qwen3_config_from_dict(TINY["C"])
    assert c.layer_types == ("full_attention", "sliding_attention", "sliding_attention", "sliding_attention")
    assert [c.window_of_layer(i) for i in range(4)] == [None, 20, 20, 20]
    c = qwen3_config_from_dict(dict(TINY["C"], use_sliding_window=False))
    assert c.sliding_window is None and set(c.layer_types) == {"full_attention"}
    c = qwen3_config_from_dict(dict(TINY["A"], sliding_window=8, layer_types=["sliding_attention", "full_attention"]))
    assert [c.window_of_layer(i) for i in range(2)] == [8, None]
    with pytest.raises(ConfigError, match="sliding_window"):
        qwen3_config_from_dict(dict(TINY["A"], layer_types=["sliding_attention", "full_attention"]))


def test_eos_ids():
    assert qwen3_config_from_dict(dict(TINY["A"], eos_token_id=7)).eos_token_ids == (7,)
    assert qwen3_config_from_dict(dict(TINY["A"], eos_token_id=[7, 9])).eos_token_ids == (7, 9)


def test_spec_carries_every_constant_to_its_part():
    arch = get_architecture("Qwen3ForCausalLM")
    c = qwen3_config_from_dict(TINY["C"])
    spec = arch.build_spec(c)
    spec.validate()
    assert len(spec.layers) == 4 and [call.layer for call in spec.order] == [0, 1, 2, 3]
    m = spec.layers[2].mixer
    assert m.kind == "attention" and m["num_heads"] == 6 and m["num_kv_heads"] == 3 and m["head_dim"] == 48
    assert m["window"] == 20 and spec.layers[0].mixer["window"] is None
    assert m["position"].kind == "rotary" and m["position"]["base"] == 500000.0 and m["position"]["dim"] == 48
    assert abs(m["scale"] - 48 ** -0.5) < 1e-12 and m["qk_norm_eps"] == 3e-6
    assert spec.layers[0].feed_forward["intermediate_size"] == 112
    assert spec.final_norm["eps"] == 3e-6 and spec.head["tied"] is False


def test_config_round_trips_through_config_json():
    arch = get_architecture("Qwen3ForCausalLM")
    for name in TINY:
        c = qwen3_config_from_dict(TINY[name])
        again = arch.load_config(json.loads(json.dumps(arch.config_to_dict(c))))
        assert again == c


def test_registry(tmp_path):
    assert "Qwen3ForCausalLM" in architecture_names()
    with pytest.raises(KeyError, match="supported: .*Qwen3ForCausalLM"):
        get_architecture("NoSuchModel")

    @register_architecture
    class Toy(Architecture):
        name = "ToyForTests"

        def load_config(self, raw):
            return dict(raw)

    try:
        (tmp_path / "config.json").write_text(json.dumps({"architectures": ["ToyForTests"], "x": 1}))
        arch, cfg = load_model_config(str(tmp_path))
        assert arch.name == "ToyForTests" and cfg["x"] == 1
    finally:
        unregister_architecture("ToyForTests")
    (tmp_path / "config.json").write_text(json.dumps({"architectures": []}))
    with pytest.raises(ValueError, match="architectures"):
        load_model_config(str(tmp_path))


def test_run_order_is_checked():
    from iian_b200.config.spec import LayerCall, ModelSpec
    arch = get_architecture("Qwen3ForCausalLM")
    spec = arch.build_spec(qwen3_config_from_dict(TINY["A"]))

    def with_order(order):
        return ModelSpec(spec.hidden_size, spec.vocab_size, spec.max_position, spec.embedding, spec.layers, order,
                         spec.final_norm, spec.head)
    with_order((LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2), LayerCall(1, 0, writes_cache=False))).validate()
    with pytest.raises(ValueError, match="names layer 5"):
        with_order((LayerCall(5, 0),)).validate()
    with pytest.raises(ValueError, match="written by"):
        with_order((LayerCall(0, 0), LayerCall(1, 0))).validate()
    with pytest.raises(ValueError, match="no entry writes"):
        with_order((LayerCall(0, 0), LayerCall(1, 3, writes_cache=False))).validate()
    with pytest.raises(ValueError, match="before entry"):
        with_order((LayerCall(0, 1, writes_cache=False), LayerCall(1, 1))).validate()
