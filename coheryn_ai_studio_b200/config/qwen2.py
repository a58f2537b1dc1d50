"""Typed configuration of the Qwen2 dense decoder, read from ``config.json`` keys.

What the reference takes from GGUF metadata (crates/coheryn-engine/src/compat.rs:54-159:
bounded positive integers, ``hidden % heads == 0``, ``heads % kv_heads == 0``, an even
head size, ``rope_base`` defaulting to 10000, a REQUIRED norm epsilon, rejection of
RoPE scaling and of sliding windows and of every key it does not implement) is taken
here from the same quantities under their ``config.json`` names, in the manner of the
reference's one ``config.json`` parser (crates/coheryn-engine/src/qwen35/config.rs:30-110:
an allow-list of keys, hard rejection of unimplemented values).  JSON limits (at most
1 MiB, depth at most 32, duplicate keys rejected) follow
crates/coheryn-engine/src/safetensors.rs:191-230.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import asdict, dataclass
from typing import Any, Dict, List

from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, prenorm_layer

MAX_CONFIG_BYTES = 1 << 20
MAX_CONFIG_DEPTH = 32


class ConfigError(ValueError):
    """config.json is malformed, or asks for something that is not implemented."""


def _reject_duplicates(pairs):
    out = {}
    for k, v in pairs:
        if k in out:
            raise ConfigError(f"duplicate key {k!r} in config.json")
        out[k] = v
    return out


def _depth(value, level=1):
    if level > MAX_CONFIG_DEPTH:
        raise ConfigError(f"config.json is nested deeper than {MAX_CONFIG_DEPTH}")
    if isinstance(value, dict):
        for v in value.values():
            _depth(v, level + 1)
    elif isinstance(value, list):
        for v in value:
            _depth(v, level + 1)


def read_config_json(path: str) -> Dict[str, Any]:
    """Parse a config.json with the limits above; returns the top-level object."""
    size = os.path.getsize(path)
    if size > MAX_CONFIG_BYTES:
        raise ConfigError(f"{path} is {size} bytes; at most {MAX_CONFIG_BYTES} are read")
    with open(path, "rb") as f:
        raw = f.read()
    try:
        root = json.loads(raw.decode("utf-8"), object_pairs_hook=_reject_duplicates)
    except (UnicodeDecodeError, json.JSONDecodeError, RecursionError) as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from None
    if not isinstance(root, dict):
        raise ConfigError(f"{path} does not hold a JSON object")
    _depth(root)
    return root


def _positive(d: Dict[str, Any], key: str, maximum: int) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0 or v > maximum:
        raise ConfigError(f"{key} must be an integer in 1..={maximum}, got {v!r}")
    return v


def _number(d: Dict[str, Any], key: str, default=None) -> float:
    v = d.get(key, default)
    if v is None:
        raise ConfigError(f"{key} is required")
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or v <= 0:
        raise ConfigError(f"{key} must be a finite positive number, got {v!r}")
    return float(v)


# Keys that carry no information the engine uses (checked for type only where cheap).
_INFORMATIONAL = {
    "architectures", "model_type", "torch_dtype", "dtype", "transformers_version",
    "use_cache", "initializer_range", "bos_token_id", "eos_token_id", "pad_token_id",
    "attention_dropout", "max_window_layers", "sliding_window", "layer_types",
    "_name_or_path",
}
_IMPLEMENTED = {
    "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
    "num_attention_heads", "num_key_value_heads", "head_dim", "hidden_act",
    "max_position_embeddings", "rms_norm_eps", "rope_theta", "rope_scaling",
    "tie_word_embeddings", "use_sliding_window", "attention_bias",
}


@dataclass(frozen=True)
class Qwen2Config:
    """Every size and constant of the model; nothing of this stands in code elsewhere."""

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    attention_bias: bool = True  # q/k/v carry a bias, o does not (compat.rs:187-194)
    hidden_act: str = "silu"
    eos_token_ids: tuple = ()

    architecture = "Qwen2ForCausalLM"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen2Config":
        unknown = sorted(k for k in d if k not in _IMPLEMENTED and k not in _INFORMATIONAL)
        if unknown:
            raise ConfigError("unimplemented configuration key(s): " + ", ".join(unknown))
        if d.get("model_type", "qwen2") != "qwen2":
            raise ConfigError(f"model_type {d.get('model_type')!r} is not qwen2")
        if d.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act {d.get('hidden_act')!r} is not implemented (silu only)")
        if d.get("rope_scaling") is not None:
            raise ConfigError("rope_scaling is not implemented (compat.rs:138-146 rejects it)")
        if d.get("use_sliding_window", False) not in (False,):
            raise ConfigError("use_sliding_window=true is not implemented "
                              "(compat.rs:138-146 rejects sliding-window variants)")
        if d.get("attention_dropout", 0.0) not in (0, 0.0):
            raise ConfigError("attention_dropout must be 0 for inference")
        hidden = _positive(d, "hidden_size", 32768)
        heads = _positive(d, "num_attention_heads", 512)
        kv_heads = _positive(d, "num_key_value_heads", 512)
        if heads % kv_heads != 0:
            raise ConfigError(f"num_attention_heads {heads} is not a multiple of "
                              f"num_key_value_heads {kv_heads}")
        if "head_dim" in d and d["head_dim"] is not None:
            head_dim = _positive(d, "head_dim", 1024)
        else:
            if hidden % heads != 0:
                raise ConfigError(f"hidden_size {hidden} is not a multiple of "
                                  f"num_attention_heads {heads} and no head_dim is given")
            head_dim = hidden // heads
        if head_dim % 2 != 0:
            raise ConfigError(f"head_dim {head_dim} must be even for rotate-half RoPE")
        tie = d.get("tie_word_embeddings", False)
        bias = d.get("attention_bias", True)
        if not isinstance(tie, bool) or not isinstance(bias, bool):
            raise ConfigError("tie_word_embeddings and attention_bias must be booleans")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: tuple = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError("eos_token_id must be an integer or a list of integers")
        return cls(
            vocab_size=_positive(d, "vocab_size", 1_000_000),
            hidden_size=hidden,
            intermediate_size=_positive(d, "intermediate_size", 131072),
            num_hidden_layers=_positive(d, "num_hidden_layers", 256),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            max_position_embeddings=_positive(d, "max_position_embeddings", 1_048_576),
            rms_norm_eps=_number(d, "rms_norm_eps"),
            rope_theta=_number(d, "rope_theta", 10000.0),
            tie_word_embeddings=tie,
            attention_bias=bias,
            eos_token_ids=eos_ids,
        )

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        eos = d.pop("eos_token_ids")
        if eos:
            d["eos_token_id"] = list(eos) if len(eos) > 1 else eos[0]
        d["architectures"] = [self.architecture]
        d["model_type"] = "qwen2"
        d["use_sliding_window"] = False
        return d


# GGUF: metadata keys of general.architecture = "qwen2" and the tensor names
# (crates/coheryn-engine/src/compat.rs:54-159 for the keys, 161-221 for the tensors).
_GGUF_KEYS = {
    "qwen2.block_count": "num_hidden_layers", "qwen2.embedding_length": "hidden_size",
    "qwen2.feed_forward_length": "intermediate_size", "qwen2.attention.head_count": "num_attention_heads",
    "qwen2.attention.head_count_kv": "num_key_value_heads", "qwen2.context_length": "max_position_embeddings",
    "qwen2.rope.freq_base": "rope_theta", "qwen2.attention.layer_norm_rms_epsilon": "rms_norm_eps",
}
_GGUF_HEAD_DIM_KEYS = ("qwen2.attention.key_length", "qwen2.attention.value_length", "qwen2.rope.dimension_count")
_GGUF_LAYER_NAMES = {
    "attn_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm",
    "attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj",
    "attn_output": "self_attn.o_proj", "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj",
    "ffn_down": "mlp.down_proj",
}
_GGUF_TOP_NAMES = {"token_embd": "model.embed_tokens", "output_norm": "model.norm", "output": "lm_head"}


def qwen2_config_from_gguf(meta: Dict[str, Any], tensor_names) -> Qwen2Config:
    """The typed configuration from GGUF metadata.  Keys of the architecture that are not
    implemented are refused (rope scaling, sliding window, anything else under "qwen2."), as
    compat.rs:66-89 and 132-146 do; the vocabulary is the tokenizer's token count
    (compat.rs:96-101), the output is tied when the file holds no "output.weight"."""
    if meta.get("split.count", 1) not in (0, 1):
        raise ConfigError("split GGUF files are not read")
    known = set(_GGUF_KEYS) | set(_GGUF_HEAD_DIM_KEYS)
    unknown = sorted(k for k in meta if k.startswith("qwen2.") and k not in known)
    if unknown:
        raise ConfigError("unimplemented GGUF key(s): " + ", ".join(unknown))
    d: Dict[str, Any] = {"architectures": [Qwen2Config.architecture], "model_type": "qwen2"}
    for key, name in _GGUF_KEYS.items():
        if key in meta:
            d[name] = meta[key]
    tokens = meta.get("tokenizer.ggml.tokens")
    if not isinstance(tokens, list) or not tokens:
        raise ConfigError("tokenizer.ggml.tokens is required: its length is the vocabulary")
    d["vocab_size"] = len(tokens)
    d["tie_word_embeddings"] = "output.weight" not in set(tensor_names)
    if "tokenizer.ggml.eos_token_id" in meta:
        d["eos_token_id"] = meta["tokenizer.ggml.eos_token_id"]
    config = Qwen2Config.from_dict(d)
    for key in _GGUF_HEAD_DIM_KEYS:
        if key in meta and meta[key] != config.head_dim:
            raise ConfigError(f"{key} = {meta[key]!r} differs from the head size {config.head_dim} "
                              "(partial rotation and separate key/value sizes are not implemented)")
    return config


def qwen2_gguf_tensor_name(name: str) -> str:
    """GGUF tensor name -> checkpoint (HF) name; names outside the table come back unchanged
    and are then reported as unexpected."""
    stem, dot, kind = name.rpartition(".")
    if not dot or kind not in ("weight", "bias"):
        return name
    if stem in _GGUF_TOP_NAMES:
        return f"{_GGUF_TOP_NAMES[stem]}.{kind}"
    parts = stem.split(".")
    if len(parts) == 3 and parts[0] == "blk" and parts[1].isdigit() and parts[2] in _GGUF_LAYER_NAMES:
        return f"model.layers.{int(parts[1])}.{_GGUF_LAYER_NAMES[parts[2]]}.{kind}"
    return name


def qwen2_gguf_metadata(c: Qwen2Config) -> Dict[str, Any]:
    """GGUF metadata for a configuration (the random-weights mode): the inverse of
    ``qwen2_config_from_gguf``, with a placeholder token table of the vocabulary's length."""
    meta: Dict[str, Any] = {"general.architecture": "qwen2", "general.alignment": 32}
    for key, name in _GGUF_KEYS.items():
        meta[key] = getattr(c, name)
    for key in _GGUF_HEAD_DIM_KEYS:
        meta[key] = c.head_dim
    meta["tokenizer.ggml.tokens"] = [f"<{i}>" for i in range(c.vocab_size)]
    if c.eos_token_ids:
        meta["tokenizer.ggml.eos_token_id"] = c.eos_token_ids[0]
    return meta


def qwen2_gguf_name_of(hf_name: str) -> str:
    """Checkpoint (HF) name -> GGUF tensor name (for writing)."""
    stem, _, kind = hf_name.rpartition(".")
    for g, h in _GGUF_TOP_NAMES.items():
        if stem == h:
            return f"{g}.{kind}"
    parts = stem.split(".", 3)       # model, layers, i, rest
    if len(parts) == 4 and parts[:2] == ["model", "layers"]:
        for g, h in _GGUF_LAYER_NAMES.items():
            if parts[3] == h:
                return f"blk.{parts[2]}.{g}.{kind}"
    raise ConfigError(f"tensor {hf_name} has no GGUF name")


def qwen2_model_spec(c: Qwen2Config) -> ModelSpec:
    """Qwen2: every layer is pre-norm residual over GQA attention (q/k/v bias, no o
    bias, rotate-half RoPE over the whole head) and a SwiGLU feed-forward
    (crates/coheryn-engine/src/inference.rs:440-540)."""
    norm = PartSpec("rmsnorm", {"size": c.hidden_size, "eps": c.rms_norm_eps})
    rope = PartSpec("rope_rotate_half", {
        "head_dim": c.head_dim, "rotary_dim": c.head_dim, "theta": c.rope_theta,
        "max_positions": c.max_position_embeddings})
    layers: List[LayerSpec] = []
    for i in range(c.num_hidden_layers):
        layers.append(prenorm_layer(
            prefix=f"model.layers.{i}",
            mixer=PartSpec("attention", {
                "hidden_size": c.hidden_size, "num_heads": c.num_attention_heads,
                "num_kv_heads": c.num_key_value_heads, "head_dim": c.head_dim,
                "qkv_bias": c.attention_bias, "o_bias": False, "window": None,
                "scale": 1.0 / math.sqrt(c.head_dim)}),
            feed_forward=PartSpec("gated_mlp", {
                "hidden_size": c.hidden_size, "intermediate_size": c.intermediate_size,
                "activation": c.hidden_act}),
            mixer_norm=norm, feed_forward_norm=norm, position=rope))
    return ModelSpec(
        architecture=c.architecture,
        hidden_size=c.hidden_size,
        vocab_size=c.vocab_size,
        max_positions=c.max_position_embeddings,
        embedding_name="model.embed_tokens",
        layers=layers,
        schedule=[ScheduleEntry(i) for i in range(c.num_hidden_layers)],
        final_norm=norm,
        final_norm_name="model.norm",
        head_name=None if c.tie_word_embeddings else "lm_head",
    )
