import json

import pytest

from coheryn_ai_studio_b200.config import (ConfigError, ModelSpec, PartSpec, Qwen2Config, ScheduleEntry,
                                           architecture_for, load_config, register_architecture,
                                           registered_architectures, unregister_architecture)
import tiny


def base():
    d = tiny.TINY_B.to_dict()
    return d


def test_round_trip_keeps_every_field():
    for cfg in (tiny.TINY_A, tiny.TINY_B):
        assert Qwen2Config.from_dict(cfg.to_dict()) == cfg


def test_sizes_come_from_config_json(tmp_path):
    d = base()
    d.update(hidden_size=80, num_attention_heads=5, num_key_value_heads=5, head_dim=16,
             intermediate_size=100, num_hidden_layers=1, vocab_size=77)
    (tmp_path / "config.json").write_text(json.dumps(d))
    cfg, spec = load_config(str(tmp_path))
    assert (cfg.hidden_size, cfg.head_dim, cfg.vocab_size) == (80, 16, 77)
    assert len(spec.layers) == 1 and spec.layers[0].mixer.params["num_heads"] == 5
    assert spec.layers[0].feed_forward.params["intermediate_size"] == 100
    assert spec.head_name == "lm_head" and spec.vocab_size == 77


def test_head_dim_defaults_to_hidden_over_heads():
    d = base(); del d["head_dim"]
    assert Qwen2Config.from_dict(d).head_dim == 32
    d["hidden_size"] = 100
    with pytest.raises(ConfigError, match="multiple"):
        Qwen2Config.from_dict(d)


def test_rope_theta_defaults_and_eps_is_required():
    d = base(); del d["rope_theta"]
    assert Qwen2Config.from_dict(d).rope_theta == 10000.0      # compat.rs:102-105
    del d["rms_norm_eps"]
    with pytest.raises(ConfigError, match="rms_norm_eps"):      # compat.rs:106-109
        Qwen2Config.from_dict(d)


@pytest.mark.parametrize("patch,match", [
    ({"rope_scaling": {"type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"use_sliding_window": True}, "sliding"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"num_key_value_heads": 2}, "multiple"),
    ({"head_dim": 31}, "even"),
    ({"vocab_size": 0}, "vocab_size"),
    ({"num_hidden_layers": 1000}, "num_hidden_layers"),
    ({"rms_norm_eps": -1}, "rms_norm_eps"),
    ({"mystery_option": 3}, "mystery_option"),
    ({"model_type": "llama"}, "model_type"),
])
def test_unimplemented_values_are_refused(patch, match):
    d = base(); d.update(patch)
    with pytest.raises(ConfigError, match=match):
        Qwen2Config.from_dict(d)


def test_duplicate_keys_and_garbage_are_refused(tmp_path):
    (tmp_path / "config.json").write_text('{"architectures": ["Qwen2ForCausalLM"], "vocab_size": 1, "vocab_size": 2}')
    with pytest.raises(ConfigError, match="duplicate"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("[1, 2]")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{" * 40)
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))


def test_registry_semantics():
    assert "Qwen2ForCausalLM" in registered_architectures()
    with pytest.raises(ConfigError, match="not registered"):
        architecture_for({"architectures": ["NoSuchModel"]})
    with pytest.raises(ConfigError, match="exactly one"):
        architecture_for({"architectures": ["A", "B"]})
    with pytest.raises(ValueError, match="already registered"):
        register_architecture("Qwen2ForCausalLM", dict, lambda c: None)
    with pytest.raises(ValueError, match="non-empty"):
        register_architecture("", dict, lambda c: None)
    register_architecture("ToyForTest", dict, lambda c: None)
    assert architecture_for({"architectures": ["ToyForTest"]}).name == "ToyForTest"
    unregister_architecture("ToyForTest")


def test_schedule_is_validated():
    norm = PartSpec("rmsnorm", {"size": 8, "eps": 1e-6})
    from coheryn_ai_studio_b200.config import LayerSpec
    layer = LayerSpec("model.layers.0", "prenorm_residual", PartSpec("attention"), PartSpec("gated_mlp"), norm, norm)
    def spec(schedule):
        return ModelSpec("T", 8, 10, 16, "model.embed_tokens", [layer], schedule, norm, "model.norm", None)
    spec([ScheduleEntry(0), ScheduleEntry(0), ScheduleEntry(0, cache_from=1)]).validate()
    with pytest.raises(ValueError, match="names layer"):
        spec([ScheduleEntry(1)]).validate()
    with pytest.raises(ValueError, match="earlier"):
        spec([ScheduleEntry(0, cache_from=0)]).validate()
    with pytest.raises(ValueError, match="owns no cache"):
        spec([ScheduleEntry(0), ScheduleEntry(0, cache_from=0), ScheduleEntry(0, cache_from=1)]).validate()
