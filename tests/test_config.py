"""Configuration parsing and the architecture registry (no GPU)."""
import json

import pytest

import tiny
from prelude_b200.config import (ConfigError, Qwen3Config, load_model_config, load_model_spec, register_architecture,
                                 registered_architectures, unregister_architecture)
from prelude_b200.config.registry import extract_eos_token_ids, normalize_identifier, resolve_architecture


def test_qwen3_fields_come_from_config_json():
    cfg = load_model_config(tiny.TINY_B)
    assert isinstance(cfg, Qwen3Config)
    for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                "num_key_value_heads", "head_dim", "max_position_embeddings", "rope_theta", "rms_norm_eps",
                "tie_word_embeddings"):
        assert getattr(cfg, key) == tiny.TINY_B[key]
    assert cfg.eos_token_ids == (7, 9)
    spec = cfg.to_model_spec()
    assert len(spec.blocks) == 3 and [c.block for c in spec.order] == [0, 1, 2]
    attn = spec.blocks[0].mixer
    assert (attn.num_heads, attn.num_kv_heads, attn.head_dim) == (6, 2, 32)
    assert attn.head_dim * attn.num_heads != spec.hidden_size          # inner width is its own number
    assert attn.softmax_scale == pytest.approx(32 ** -0.5)
    assert attn.qk_norm_eps == 1e-5 and spec.final_norm.eps == 1e-5
    assert attn.position.theta == 1000000.0 and attn.position.max_positions == 256
    assert not spec.tie_embeddings


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "num_key_value_heads", "head_dim",
                                 "max_position_embeddings", "rope_theta", "rms_norm_eps", "tie_word_embeddings"])
def test_missing_required_key_is_named(key):
    raw = dict(tiny.TINY_A)
    del raw[key]
    with pytest.raises(ConfigError, match=f"failed to parse Qwen3 config.*{key}"):
        load_model_config(raw)


def test_all_problems_in_one_error():
    raw = dict(tiny.TINY_A, head_dim="16", num_key_value_heads=0)
    del raw["rope_theta"]
    with pytest.raises(ConfigError) as e:
        load_model_config(raw)
    for word in ("head_dim", "num_key_value_heads", "rope_theta"):
        assert word in str(e.value)


def test_optional_switches_default_and_extra_keys_ignored():
    raw = {k: v for k, v in tiny.TINY_A.items() if k not in ("attention_bias", "use_sliding_window", "sliding_window",
                                                            "max_window_layers", "hidden_act")}
    raw.update(torch_dtype="bfloat16", bos_token_id=1, rope_scaling=None, transformers_version="4.51.0")
    cfg = load_model_config(raw)
    assert (cfg.attention_bias, cfg.use_sliding_window, cfg.sliding_window, cfg.hidden_act) == (False, False, None, "silu")


def test_refusals():
    with pytest.raises(ConfigError, match="sliding window is not supported"):
        load_model_config(dict(tiny.TINY_A, use_sliding_window=True, sliding_window=64))
    with pytest.raises(ConfigError, match="not a multiple"):
        load_model_config(dict(tiny.TINY_A, num_attention_heads=5))
    with pytest.raises(ConfigError, match="hidden_act"):
        load_model_config(dict(tiny.TINY_A, hidden_act="gelu"))
    with pytest.raises(ConfigError, match="head_dim"):
        load_model_config(dict(tiny.TINY_A, head_dim=15))


def test_registry_resolution_rules():
    assert normalize_identifier("Qwen-3_Model") == "qwen3model"
    base = {k: v for k, v in tiny.TINY_A.items() if k not in ("architectures", "model_type")}
    assert resolve_architecture(dict(base, architectures=["Qwen3ForCausalLM"])).name == "Qwen3"
    assert resolve_architecture(dict(base, architectures=["qwen_3ForConditionalGeneration"])).name == "Qwen3"
    assert resolve_architecture(dict(base, architectures=["Qwen3ModelForTextGeneration"])).name == "Qwen3"
    assert resolve_architecture(dict(base, architectures=["SomethingElse"], model_type="qwen3")).name == "Qwen3"
    assert resolve_architecture(dict(base, model_type="QWEN3")).name == "Qwen3"
    with pytest.raises(ConfigError, match="unable to resolve model architecture"):
        resolve_architecture(dict(base, architectures=["LlamaForCausalLM"], model_type="llama"))
    with pytest.raises(ConfigError, match="not supported"):
        resolve_architecture(dict(base, architectures=["Qwen3ForSequenceClassification"]))


def test_eos_forms():
    assert extract_eos_token_ids({"eos_token_id": 5}) == (5,)
    assert extract_eos_token_ids({"eos_token_id": [5, 6]}) == (5, 6)
    assert extract_eos_token_ids({"text_config": {"eos_token_id": 3}}) == (3,)
    assert extract_eos_token_ids({}) == ()
    with pytest.raises(ConfigError, match="missing required field"):
        extract_eos_token_ids({}, required=True)
    for bad in ("5", [1, "2"], [], 1.5, True):
        with pytest.raises(ConfigError):
            extract_eos_token_ids({"eos_token_id": bad})


def test_config_from_folder_and_errors(tmp_path):
    with pytest.raises(ConfigError, match="no config.json"):
        load_model_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_model_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(tiny.TINY_A))
    assert load_model_spec(str(tmp_path)).vocab_size == 256


def test_another_architecture_registers_without_touching_the_framework():
    from prelude_b200.config.spec import ModelSpec

    @register_architecture("Toy", aliases=("Toy", "ToyLM"), model_types=("toy",))
    class ToyConfig:
        def __init__(self, raw):
            self.raw = raw

        @classmethod
        def from_dict(cls, raw):
            return cls(raw)

        def to_model_spec(self):
            spec = Qwen3Config.from_dict(dict(tiny.TINY_A, **self.raw.get("inner", {}))).to_model_spec()
            return ModelSpec(**{**spec.__dict__, "architecture": "ToyForCausalLM"})

    try:
        assert "Toy" in registered_architectures()
        spec = load_model_spec({"architectures": ["ToyLMForCausalLM"], "inner": {"vocab_size": 99}})
        assert spec.architecture == "ToyForCausalLM" and spec.vocab_size == 99
    finally:
        unregister_architecture("Toy")
    assert "Toy" not in registered_architectures()


def test_order_list_is_checked():
    from prelude_b200.config.spec import LayerCall, ModelSpec
    spec = load_model_spec(tiny.TINY_A)

    def with_order(order):
        return ModelSpec(**{**spec.__dict__, "order": tuple(order)})

    ok = with_order([LayerCall(0), LayerCall(1), LayerCall(0), LayerCall(1, cache=1, writes_cache=False)])
    assert [c.cache for c in ok.resolved_order()] == [0, 1, 2, 1]
    with pytest.raises(ValueError, match="names block 5"):
        with_order([LayerCall(5)]).resolved_order()
    with pytest.raises(ValueError, match="no earlier call owns"):
        with_order([LayerCall(0, cache=0, writes_cache=False)]).resolved_order()
    with pytest.raises(ValueError, match="must own it"):
        with_order([LayerCall(0), LayerCall(1, cache=0)]).resolved_order()
