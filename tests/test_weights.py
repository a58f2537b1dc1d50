import json
import os
import struct

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
import tiny
from coheryn_ai_studio_b200.config import load_config
from coheryn_ai_studio_b200.parts import DecoderModel, Runtime
from coheryn_ai_studio_b200.weights import (SafetensorsError, WeightError, index_model_dir, load_tensors,
                                            read_header, write_file)
from coheryn_ai_studio_b200.weights.safetensors_io import TensorReader


def specs_for(folder, dtype=torch.bfloat16):
    _, spec = load_config(folder)
    return DecoderModel(spec, Runtime(dtype, torch.device("cpu"))).tensor_specs()


def rewrite(folder, change):
    path = os.path.join(folder, "model.safetensors")
    entries = read_header(path)
    reader = TensorReader(entries)
    tensors = {n: reader.read(n) for n in entries}
    reader.close()
    change(tensors)
    write_file(path, sorted(tensors.items()))


def test_random_folder_is_reproducible_and_complete(tmp_path):
    a = tiny.make_folder(tmp_path / "x", "A")
    b = tiny.make_folder(tmp_path / "y", "A")
    assert open(os.path.join(a, "model.safetensors"), "rb").read() == open(os.path.join(b, "model.safetensors"), "rb").read()
    names = set(index_model_dir(a))
    assert "lm_head.weight" not in names and "model.embed_tokens.weight" in names      # tied
    assert len(names) == 2 + 12 * tiny.TINY_A.num_hidden_layers                        # 3 + 12 L, tied: 2 + 12 L
    assert "lm_head.weight" in set(index_model_dir(tiny.make_folder(tmp_path, "B")))
    cfg, w = plain.read_model(a)
    assert abs(w["model.layers.0.mlp.up_proj.weight"].std() - 0.02) < 0.002
    assert abs(w["model.norm.weight"].mean() - 1) < 0.01


def test_dtype_policy(tmp_path):
    d = tiny.make_folder(tmp_path, "B")
    specs = specs_for(d)
    t = load_tensors(d, specs, torch.bfloat16, "cpu")
    assert t["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16
    assert t["model.layers.0.self_attn.q_proj.bias"].dtype == torch.bfloat16
    assert t["model.norm.weight"].dtype == torch.float32           # stored in 32-bit: stays so
    t32 = load_tensors(d, specs, torch.float32, "cpu")
    assert all(x.dtype == torch.float32 for x in t32.values())
    assert torch.equal(t32["lm_head.weight"], t["lm_head.weight"].float())


def test_one_error_lists_everything(tmp_path):
    d = tiny.make_folder(tmp_path, "B")
    def change(t):
        del t["model.layers.1.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.0.self_attn.o_proj.bias"] = torch.zeros(96)
        t["extra.thing"] = torch.zeros(2, 2)
        t["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(64, 96, dtype=torch.bfloat16)
        t["model.embed_tokens.weight"] = torch.zeros(1000, 96, dtype=torch.int32)
    rewrite(d, change)
    with pytest.raises(WeightError) as e:
        load_tensors(d, specs_for(d), torch.bfloat16, "cpu")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["extra.thing", "model.layers.0.self_attn.o_proj.bias"]
    assert err.wrong_shape == [("model.layers.2.self_attn.k_proj.weight", (64, 96), (32, 96))]
    assert err.wrong_dtype and err.wrong_dtype[0][0] == "model.embed_tokens.weight"
    text = str(err)
    for needle in ("missing (2)", "unexpected (2)", "extra.thing", "[64, 96]", "[32, 96]"):
        assert needle in text


def test_tied_model_refuses_a_separate_head(tmp_path):
    d = tiny.make_folder(tmp_path, "A")
    rewrite(d, lambda t: t.__setitem__("lm_head.weight", torch.zeros(512, 64, dtype=torch.bfloat16)))
    with pytest.raises(WeightError) as e:
        load_tensors(d, specs_for(d), torch.bfloat16, "cpu")
    assert e.value.unexpected == ["lm_head.weight"]


def test_non_finite_weight_is_refused(tmp_path):
    d = tiny.make_folder(tmp_path, "A")
    def change(t):
        t["model.norm.weight"][3] = float("inf")
    rewrite(d, change)
    with pytest.raises(ValueError, match="non-finite"):
        load_tensors(d, specs_for(d), torch.float32, "cpu")


def test_container_checks(tmp_path):
    p = str(tmp_path / "m.safetensors")
    write_file(p, [("a", torch.arange(6, dtype=torch.float32).reshape(2, 3)), ("b", torch.ones(4, dtype=torch.bfloat16))])
    h = read_header(p)
    assert h["a"].shape == (2, 3) and h["b"].dtype == torch.bfloat16
    raw = open(p, "rb").read()
    # every truncation is refused
    for cut in (0, 4, 8, 20, len(raw) - 1):
        open(p, "wb").write(raw[:cut])
        with pytest.raises(SafetensorsError):
            read_header(p)
    def with_header(obj, payload=b"\0" * 32):
        text = json.dumps(obj).encode()
        open(p, "wb").write(struct.pack("<Q", len(text)) + text + payload)
    with_header({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]},
                 "b": {"dtype": "F32", "shape": [4], "data_offsets": [8, 24]}})
    with pytest.raises(SafetensorsError, match="hole or an overlap"):
        read_header(p)
    with_header({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}})
    with pytest.raises(SafetensorsError, match="belong to no tensor"):
        read_header(p)
    with_header({"a": {"dtype": "F64", "shape": [4], "data_offsets": [0, 32]}})
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        read_header(p)
    with_header({"a": {"dtype": "F32", "shape": [5], "data_offsets": [0, 16]}})
    with pytest.raises(SafetensorsError, match="does not match"):
        read_header(p)
    open(p, "wb").write(struct.pack("<Q", 40) + b'{"a":{"dtype":"F32"},"a":{"dtype":"F32"}}')
    with pytest.raises(SafetensorsError):
        read_header(p)


def test_sharded_folder(tmp_path):
    d = tiny.make_folder(tmp_path, "A")
    entries = read_header(os.path.join(d, "model.safetensors"))
    reader = TensorReader(entries)
    names = sorted(entries)
    half = len(names) // 2
    write_file(os.path.join(d, "s1.safetensors"), [(n, reader.read(n)) for n in names[:half]])
    write_file(os.path.join(d, "s2.safetensors"), [(n, reader.read(n)) for n in names[half:]])
    reader.close()
    os.unlink(os.path.join(d, "model.safetensors"))
    wm = {n: ("s1.safetensors" if i < half else "s2.safetensors") for i, n in enumerate(names)}
    json.dump({"weight_map": wm}, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    t = load_tensors(d, specs_for(d), torch.float32, "cpu")
    assert len(t) == len(names)
    wm[names[0]] = "../s1.safetensors"
    json.dump({"weight_map": wm}, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    with pytest.raises(SafetensorsError, match="plain file name"):
        index_model_dir(d)


# ------------------------------------------------------------------ seeded values
def test_splitmix64_known_answers():
    """The first outputs of SplitMix64 from state 0, as published with the generator, and the
    sampler's stream of the reference's fixture use the same constants
    (crates/coheryn-engine/src/sampling.rs:123-130)."""
    import plain_random as pr
    got = [int(v) for v in pr._draw(0, np.array([1, 2, 3], dtype=np.uint64))]
    assert got == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]
    assert plain.PlainSampler(seed=0).random() == (0xE220A8397B1DCDAF >> 11) / 2.0 ** 53


def test_seeded_values_host_equals_numpy_bit_for_bit():
    """The host runtime's generator (C++) and the numpy restatement of the plain implementation
    give the same float32 and bfloat16 bits, for any stretch of a tensor."""
    import plain_random as pr
    from coheryn_ai_studio_b200.weights.seeded import seeded_tensor, tensor_key
    name = "model.layers.3.self_attn.q_proj.weight"
    assert tensor_key(7, name) == pr.tensor_key(7, name)
    assert tensor_key(2 ** 64 - 1, "") == (2 ** 64 - 1) ^ 0xCBF29CE484222325
    for seed, first, n, mean, dev in [(7, 0, 70001, 0.0, 0.02), (0, 2 ** 33 + 5, 4099, 1.0, 0.01), (2 ** 63 + 11, 3, 1000, 0.0, 0.1)]:
        ref = pr.values(pr.tensor_key(seed, name), np.arange(first, first + n, dtype=np.uint64), mean, dev)
        got = seeded_tensor(seed, name, (n,), mean, dev, first=first).numpy()
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
        got16 = seeded_tensor(seed, name, (n,), mean, dev, dtype=torch.bfloat16, first=first)
        assert np.array_equal(got16.float().numpy().view(np.uint32), pr.round_bf16(ref).view(np.uint32))
    # whole-tensor helper of the plain side: rows picked out equal the rows of the whole
    whole = pr.tensor(5, "model.embed_tokens.weight", (40, 24), 0.0, 0.02)
    some = pr.tensor(5, "model.embed_tokens.weight", (40, 24), 0.0, 0.02, rows=[39, 0, 7])
    assert np.array_equal(whole[[39, 0, 7]], some)
    assert np.array_equal(seeded_tensor(5, "model.embed_tokens.weight", (40, 24), 0.0, 0.02).numpy(), whole)


def test_seeded_values_are_standard_normal():
    import plain_random as pr
    from coheryn_ai_studio_b200.weights.seeded import seeded_tensor
    z = seeded_tensor(3, "t", (2_000_000,), 0.0, 1.0).double().numpy()
    assert abs(z.mean()) < 4e-3 and abs(z.std() - 1) < 4e-3
    assert abs((z ** 3).mean()) < 2e-2 and abs((z ** 4).mean() - 3) < 5e-2
    assert np.isfinite(z).all() and np.abs(z).max() < 8.6            # sqrt(-2 ln 2^-53) = 8.57
    # the spelled-out logarithm and cosine agree with the maths library to 1e-14
    k = np.random.default_rng(0).integers(1, 2 ** 53, size=50000, dtype=np.uint64)
    assert np.abs(pr._ln_unit(k) - np.log(k.astype(np.float64) / 2.0 ** 53)).max() < 1e-14
    assert np.abs(pr._cos_turn(k) - np.cos(2 * np.pi * (k.astype(np.float64) / 2.0 ** 53))).max() < 1e-14
    edge = np.array([1, 2 ** 53, 2 ** 52, 2 ** 52 + 1, 3], dtype=np.uint64)
    assert np.abs(pr._ln_unit(edge) - np.log(edge.astype(np.float64) / 2.0 ** 53)).max() < 1e-13
    assert pr._ln_unit(np.array([2 ** 53], dtype=np.uint64))[0] == 0.0


def test_a_tensor_does_not_depend_on_the_others(tmp_path):
    """value(seed, name, index): the same tensor comes out whatever else the model holds."""
    from coheryn_ai_studio_b200.weights import InitPolicy, random_tensors
    from coheryn_ai_studio_b200.weights.spec import TensorSpec
    a = random_tensors({"w": TensorSpec((8, 16)), "n": TensorSpec((16,), role="vector", init="norm")}, 4, InitPolicy())
    b = random_tensors({"w": TensorSpec((8, 16)), "aa": TensorSpec((3, 3))}, 4, InitPolicy())
    assert torch.equal(a["w"], b["w"]) and a["n"].dtype == torch.float32 and a["w"].dtype == torch.bfloat16
    assert not torch.equal(a["w"], random_tensors({"w": TensorSpec((8, 16))}, 5, InitPolicy())["w"])
