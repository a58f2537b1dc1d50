"""The plain implementation against what the reference publishes without weights: its
RoPE and sampler fixtures (copied under tests/golden/ from fixtures/quantized/rope.json
and fixtures/constraints/sampling-v2.json) and the literal values of its unit tests."""
import json
import os

import numpy as np

import plain_qwen2 as plain

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_rope_matches_reference_fixture():
    fx = json.load(open(os.path.join(GOLDEN, "reference_rope.json")))
    tol_a, tol_r = fx["tolerances"]["absolute"], fx["tolerances"]["relative"]
    assert len(fx["cases"]) == 12
    for case in fx["cases"]:
        x = np.asarray(case["input"], dtype=np.float32)[None, :]
        y = plain.rope(x, [case["position"]], case["head_dim"], float(case["base"]))[0]
        ref = np.asarray(case["output"], dtype=np.float64)
        assert np.all(np.abs(y - ref) <= tol_a + tol_r * np.abs(ref)), case["position"]


def test_sampler_matches_reference_fixture():
    fx = json.load(open(os.path.join(GOLDEN, "reference_sampling_v2.json")))
    for case in fx["cases"]:
        s = plain.PlainSampler(**case["settings"], **case["penalties"])
        for t in case["history"]:
            s.observe(t)
        for expected in case["expected_ids"]:
            tok = s.sample(case["logits"], case["allowed"])
            assert tok == expected, case["id"]
            s.observe(tok)


def test_rms_norm_literal():
    # crates/coheryn-engine/src/cpu.rs:232-234
    out = plain.rms_norm(np.array([[3., 4.]], np.float32), np.ones(2, np.float32), 0.0)
    assert abs(out[0, 0] - 0.84852815) < 1e-6


def test_rope_literals():
    # crates/coheryn-engine/src/cpu.rs:235-239
    x = np.array([[1., 2., 3., 4.]], np.float32)
    assert np.array_equal(plain.rope(x, [0], 4, 10000.0), x)
    y = plain.rope(x, [1], 4, 10000.0)
    assert abs(y[0, 0] - (np.cos(np.float32(1)) - 3 * np.sin(np.float32(1)))) < 1e-6


def test_attention_two_keys_closed_form():
    # crates/coheryn-engine/src/cpu.rs:241-256: q=[1,0], keys [1,0],[0,1], values [2,4],[6,8]
    q = np.array([[0., 0.], [1., 0.]], np.float32)
    k = np.array([[1., 0.], [0., 1.]], np.float32)
    v = np.array([[2., 4.], [6., 8.]], np.float32)
    out = plain.attention(q, k, v, 1, 1, 2)[1]
    p = np.exp(np.float32(1) / np.sqrt(np.float32(2)))
    assert abs(out[0] - (2 * p + 6) / (p + 1)) < 1e-6
    assert abs(out[1] - (4 * p + 8) / (p + 1)) < 1e-6


def test_dot_keeps_small_terms():
    # crates/coheryn-engine/src/cpu.rs:226-228
    y = plain.linear(np.array([[1e8, 1., -1e8]], np.float32), np.ones((1, 3), np.float32))
    assert y[0, 0] == 1.0


def test_window_hides_old_keys():
    rng = np.random.default_rng(0)
    q = rng.standard_normal((6, 8)).astype(np.float32)
    k, v = (rng.standard_normal((6, 4)).astype(np.float32) for _ in range(2))
    full = plain.attention(q, k, v, 2, 1, 4)
    win = plain.attention(q, k, v, 2, 1, 4, window=3)
    assert np.allclose(full[:3], win[:3]) and not np.allclose(full[5], win[5])
    # a window as long as the sequence changes nothing
    assert np.array_equal(plain.attention(q, k, v, 2, 1, 4, window=6), full)


def test_zero_matrices_give_zero_logits(tmp_path):
    # the reference's synthetic model: embeddings 1, every matrix 0 => logits 0 => greedy
    # token 0 (crates/coheryn-engine/tests/common/mod.rs:99-118, tests/engine.rs:35-59)
    cfg = dict(num_hidden_layers=1, hidden_size=4, num_attention_heads=2, num_key_value_heads=1,
               intermediate_size=8, vocab_size=259, rms_norm_eps=1e-6, rope_theta=1e6)
    w = {"model.embed_tokens.weight": np.ones((259, 4), np.float32),
         "model.norm.weight": np.ones(4, np.float32),
         "lm_head.weight": np.zeros((259, 4), np.float32)}
    p = "model.layers.0."
    for n, shape in [("self_attn.q_proj.weight", (4, 4)), ("self_attn.k_proj.weight", (2, 4)),
                     ("self_attn.v_proj.weight", (2, 4)), ("self_attn.o_proj.weight", (4, 4)),
                     ("mlp.gate_proj.weight", (8, 4)), ("mlp.up_proj.weight", (8, 4)),
                     ("mlp.down_proj.weight", (4, 8)), ("self_attn.q_proj.bias", (4,)),
                     ("self_attn.k_proj.bias", (2,)), ("self_attn.v_proj.bias", (2,))]:
        w[p + n] = np.zeros(shape, np.float32)
    w[p + "input_layernorm.weight"] = np.ones(4, np.float32)
    w[p + "post_attention_layernorm.weight"] = np.ones(4, np.float32)
    assert not plain.forward(cfg, w, [5, 6, 7]).any()
    assert plain.greedy(cfg, w, [5], 3) == [0, 0, 0]


def test_prefix_logits_do_not_depend_on_the_future(tmp_path):
    import tiny
    d = tiny.make_folder(tmp_path, "A")
    cfg, w = plain.read_model(d)
    ids = tiny.prompt(3, 20, cfg["vocab_size"])
    full = plain.forward(cfg, w, ids)
    part = plain.forward(cfg, w, ids[:11])
    assert np.allclose(full[:11], part, atol=1e-6)


def test_the_bfloat16_bound_sees_one_wrong_token(tmp_path):
    """The bound that the bfloat16 model tests allow (a share of the spread of the plain row) is
    smaller than what ONE wrong token among the keys does to the last row, at the start and in the
    middle of sequences as long as those tests replay: widening the bound until it swallows such a
    fault fails here."""
    import tiny
    from replay import assert_bound_sees_a_wrong_token
    for name in tiny.CONFIGS:
        folder = tiny.make_folder(tmp_path, name)
        V = tiny.CONFIGS[name][0].vocab_size
        assert assert_bound_sees_a_wrong_token(folder, tiny.prompt(20, 90, V)) > 1.25
        if name.endswith("loud"):
            assert assert_bound_sees_a_wrong_token(folder, tiny.prompt(20, 150, V)) > 1.25
