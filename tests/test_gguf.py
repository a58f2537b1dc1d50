"""GGUF files with unquantized tensors: the container, the configuration from its metadata,
the tensor names, and that a model loaded from one equals the model loaded from safetensors."""
import dataclasses
import os
import struct

import numpy as np
import pytest
import torch

import tiny
from coheryn_ai_studio_b200.config import ConfigError, load_config
from coheryn_ai_studio_b200.config.qwen2 import qwen2_gguf_name_of, qwen2_gguf_tensor_name
from coheryn_ai_studio_b200.engine import write_random_gguf
from coheryn_ai_studio_b200.engine.loading import gguf_rename
from coheryn_ai_studio_b200.parts import DecoderModel, Runtime
from coheryn_ai_studio_b200.weights import (GgufError, WeightError, index_model, load_tensors, read_gguf,
                                            write_gguf)


def make_gguf(tmp_path, name, store=torch.bfloat16):
    cfg, pol, seed = tiny.CONFIGS[name]
    path = str(tmp_path / f"tiny_{name}.gguf")
    write_random_gguf(path, cfg, seed, pol, store=store)
    return path


@pytest.mark.parametrize("name", ["A", "B"])
def test_configuration_comes_from_the_metadata(tmp_path, name):
    path = make_gguf(tmp_path, name)
    config, spec = load_config(path)
    want = tiny.CONFIGS[name][0]
    # the metadata holds eps and theta as 32-bit floats, as the reference reads them
    assert config == dataclasses.replace(want, rms_norm_eps=float(np.float32(want.rms_norm_eps)),
                                         rope_theta=float(np.float32(want.rope_theta)))
    meta, entries = read_gguf(path)
    assert meta["general.architecture"] == "qwen2" and len(meta["tokenizer.ggml.tokens"]) == config.vocab_size
    assert ("output.weight" in entries) == (not config.tie_word_embeddings)
    # GGML lists a matrix as [in, out]; the index gives it row-major [out, in]
    assert entries["blk.0.attn_k.weight"].shape == (config.num_key_value_heads * config.head_dim, config.hidden_size)


@pytest.mark.parametrize("store", [torch.bfloat16, torch.float32, torch.float16])
def test_same_tensors_as_the_folder(tmp_path, store):
    folder = tiny.make_folder(tmp_path, "B", store=store if store != torch.float16 else torch.float32)
    path = make_gguf(tmp_path, "B", store=store)
    _, spec = load_config(path)
    specs = DecoderModel(spec, Runtime(torch.float32, torch.device("cpu"))).tensor_specs()
    a = load_tensors(folder, specs, torch.float32, "cpu")
    b = load_tensors(path, specs, torch.float32, "cpu", rename=gguf_rename(path))
    assert set(a) == set(b)
    for n in a:
        if store == torch.float16:      # the same draws rounded to binary16 instead of kept in float32
            assert torch.allclose(a[n], b[n], atol=1e-3, rtol=2 ** -10), n
        else:
            assert torch.equal(a[n], b[n]), n


def test_names_map_both_ways():
    for hf in ["model.embed_tokens.weight", "model.norm.weight", "lm_head.weight", "model.layers.11.self_attn.q_proj.bias",
               "model.layers.0.mlp.down_proj.weight", "model.layers.3.post_attention_layernorm.weight"]:
        assert qwen2_gguf_tensor_name(qwen2_gguf_name_of(hf)) == hf
    assert qwen2_gguf_tensor_name("blk.2.attn_output.weight") == "model.layers.2.self_attn.o_proj.weight"
    assert qwen2_gguf_tensor_name("blk.2.attn_qkv.weight") == "blk.2.attn_qkv.weight"     # unknown: left alone


def test_one_error_lists_missing_and_unexpected(tmp_path):
    path = make_gguf(tmp_path, "A")
    meta, entries = read_gguf(path)
    from coheryn_ai_studio_b200.weights.safetensors_io import TensorReader
    reader = TensorReader(entries)
    tensors = {n: reader.read(n) for n in entries}
    reader.close()
    del tensors["blk.1.ffn_up.weight"]
    tensors["blk.0.attn_output.bias"] = torch.zeros(64)
    tensors["blk.0.attn_v.weight"] = torch.zeros(8, 64, dtype=torch.bfloat16)
    write_gguf(path, meta, sorted(tensors.items()))
    _, spec = load_config(path)
    specs = DecoderModel(spec, Runtime(torch.bfloat16, torch.device("cpu"))).tensor_specs()
    with pytest.raises(WeightError) as e:
        load_tensors(path, specs, torch.bfloat16, "cpu", rename=gguf_rename(path))
    assert e.value.missing == ["model.layers.1.mlp.up_proj.weight"]
    assert e.value.unexpected == ["model.layers.0.self_attn.o_proj.bias"]
    assert e.value.wrong_shape[0][0] == "model.layers.0.self_attn.v_proj.weight"


def test_unimplemented_metadata_and_types_are_refused(tmp_path):
    path = make_gguf(tmp_path, "A")
    meta, entries = read_gguf(path)
    from coheryn_ai_studio_b200.weights.safetensors_io import TensorReader
    reader = TensorReader(entries)
    tensors = sorted((n, reader.read(n)) for n in entries)
    reader.close()
    for extra, match in [({"qwen2.rope.scaling.type": "yarn"}, "rope.scaling"), ({"qwen2.attention.sliding_window": 64}, "sliding_window"),
                         ({"qwen2.rope.dimension_count": 8}, "rope.dimension_count"), ({"general.architecture": "llama"}, "not registered"),
                         ({"split.count": 2}, "split")]:
        write_gguf(path, dict(meta, **extra), tensors)
        with pytest.raises(ConfigError, match=match):
            load_config(path)
    no_eps = {k: v for k, v in meta.items() if k != "qwen2.attention.layer_norm_rms_epsilon"}
    write_gguf(path, no_eps, tensors)
    with pytest.raises(ConfigError, match="rms_norm_eps"):
        load_config(path)
    # a packed tensor type: the error names the tensor
    write_gguf(path, meta, tensors)
    raw = bytearray(open(path, "rb").read())
    key = b"blk.0.ffn_down.weight"
    at = raw.index(key) + len(key)
    nd = struct.unpack_from("<I", raw, at)[0]
    struct.pack_into("<I", raw, at + 4 + 8 * nd, 12)       # GGML type 12 (a packed type)
    open(path, "wb").write(bytes(raw))
    with pytest.raises(GgufError, match="blk.0.ffn_down.weight"):
        read_gguf(path)


def test_container_checks(tmp_path):
    path = str(tmp_path / "x.gguf")
    open(path, "wb").write(b"GGML" + b"\0" * 64)
    with pytest.raises(GgufError, match="not a GGUF"):
        read_gguf(path)
    open(path, "wb").write(b"GGUF" + struct.pack("<IQQ", 2, 0, 0))
    with pytest.raises(GgufError, match="version"):
        read_gguf(path)
    write_gguf(path, {"general.architecture": "qwen2"}, [("a.weight", torch.ones(4, 8))])
    meta, entries = read_gguf(path)
    assert entries["a.weight"].shape == (4, 8) and entries["a.weight"].begin % 32 == 0
    raw = open(path, "rb").read()
    open(path, "wb").write(raw[:-16])                        # the last tensor runs past the end
    with pytest.raises(GgufError, match="outside the file"):
        read_gguf(path)


@pytest.mark.gpu
def test_generation_from_gguf_equals_generation_from_the_folder(tmp_path):
    from coheryn_ai_studio_b200.engine import Engine
    folder = tiny.make_folder(tmp_path, "B", policy=tiny.POLICY_LOUD)
    cfg, _, seed = tiny.CONFIGS["B"]
    path = str(tmp_path / "b.gguf")
    write_random_gguf(path, cfg, seed, tiny.POLICY_LOUD)
    prompts = [tiny.prompt(3, 40, cfg.vocab_size), tiny.prompt(4, 7, cfg.vocab_size)]
    outs = []
    for source in (folder, path):
        eng = Engine.from_folder(source, "bfloat16", context=256, page_size=16)
        outs.append([r.token_ids for r in eng.generate(prompts, max_tokens=12)])
    assert outs[0] == outs[1]
