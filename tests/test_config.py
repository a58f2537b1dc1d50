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
    assert len(spec.layers) == 1 and spec.layers[0].parts["mixer"].params["num_heads"] == 5
    assert spec.layers[0].parts["feed_forward"].params["intermediate_size"] == 100
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
    from coheryn_ai_studio_b200.config import prenorm_layer
    layer = prenorm_layer("model.layers.0", PartSpec("attention"), PartSpec("gated_mlp"), norm, norm)
    def spec(schedule):
        return ModelSpec("T", 8, 10, 16, "model.embed_tokens", [layer], schedule, norm, "model.norm", None)
    spec([ScheduleEntry(0), ScheduleEntry(0), ScheduleEntry(0, cache_from=1)]).validate()
    with pytest.raises(ValueError, match="names layer"):
        spec([ScheduleEntry(1)]).validate()
    with pytest.raises(ValueError, match="earlier"):
        spec([ScheduleEntry(0, cache_from=0)]).validate()
    with pytest.raises(ValueError, match="owns no cache"):
        spec([ScheduleEntry(0), ScheduleEntry(0, cache_from=0), ScheduleEntry(0, cache_from=1)]).validate()


def test_describe_is_metadata_only():
    """Capabilities and cache cost from the configuration alone
    (crates/coheryn-engine/src/adapters.rs:11-21, 39-58)."""
    import tiny
    arch = architecture_for(tiny.TINY_B.to_dict())
    d = arch.describe(tiny.TINY_B)
    caps = d["capabilities"]
    assert caps["adapter"] == "qwen2-b200-v1" and caps["architecture"] == "Qwen2ForCausalLM"
    assert caps["formats"] == ("safetensors", "gguf") and caps["dtypes"] == ("bfloat16", "float32")
    assert caps["paged_kv"] and caps["fixed_state_bytes_per_request"] == 0 and caps["continuous_batching"]
    # 3 layers x (keys + values) x 1 kv head x 32
    assert caps["kv_bytes_per_token"] == {"bfloat16": 3 * 2 * 32 * 2, "float32": 3 * 2 * 32 * 4}
    assert d["layers"] == 3 and d["context"] == 512 and d["vocabulary"] == 1000
    c = tiny.TINY_B
    per_layer = ((c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim * (c.hidden_size + 1)
                 + c.hidden_size * c.num_attention_heads * c.head_dim + 3 * c.hidden_size * c.intermediate_size + 2 * c.hidden_size)
    assert d["parameters"] == 3 * per_layer + 2 * c.vocab_size * c.hidden_size + c.hidden_size
    assert d["config"]["rms_norm_eps"] == 1e-5


def test_unknown_slot_of_an_arrangement_is_refused():
    import torch
    from coheryn_ai_studio_b200.config import LayerSpec
    from coheryn_ai_studio_b200.parts import DecoderModel, Runtime
    norm = PartSpec("rmsnorm", {"size": 8, "eps": 1e-6})
    layer = LayerSpec("model.layers.0", "prenorm_residual", {"mixer_norm": norm, "third_norm": norm})
    spec = ModelSpec("T", 8, 10, 16, "model.embed_tokens", [layer], [ScheduleEntry(0)], norm, "model.norm", None)
    with pytest.raises(ValueError, match="third_norm"):
        DecoderModel(spec, Runtime(torch.float32, torch.device("cpu")))
    layer = LayerSpec("model.layers.0", "prenorm_residual", {"mixer_norm": norm})
    spec = ModelSpec("T", 8, 10, 16, "model.embed_tokens", [layer], [ScheduleEntry(0)], norm, "model.norm", None)
    with pytest.raises(ValueError, match="missing slots"):
        DecoderModel(spec, Runtime(torch.float32, torch.device("cpu")))
