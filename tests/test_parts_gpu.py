"""Each part of a layer alone against the plain implementation, and the generality of
the assembly: a model whose schedule names a layer twice, lets an entry read another
entry's cache, uses a window in some layers, and holds a toy mixer with state of its own, a
toy feed-forward that routes tokens to experts and a second position encoding, all defined
HERE and registered without touching the framework's files."""
import json
import os

import numpy as np
import pytest
import torch

import plain_qwen2 as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def rt(dtype=torch.float32):
    from coheryn_ai_studio_b200.parts import Runtime
    return Runtime(dtype, DEV)


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV).to(dtype)


def one_request_step(tokens_n, start, page_size, pages_needed, groups=1):
    """A StepContext for one request that brings tokens_n tokens at positions start.."""
    from coheryn_ai_studio_b200.parts import StepContext
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    pos = list(range(start, start + tokens_n))
    table = list(range(pages_needed))[::-1]                      # pages in reverse order
    slots = [table[p // page_size] * page_size + p % page_size for p in pos]
    return StepContext(num_tokens=tokens_n, num_requests=1, token_ids=i32([0] * tokens_n), positions=i32(pos),
                       token_req=i32([0] * tokens_n), cu_q=i32([0, tokens_n]), kv_lens=i32([start + tokens_n]),
                       block_tables=[i32([table])] * groups, slots=[i32(slots)] * groups, state_slots=i32([0]),
                       q_lens=[tokens_n], kv_lens_host=[start + tokens_n], max_q_len=tokens_n,
                       max_kv_len=start + tokens_n)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from coheryn_ai_studio_b200.parts.norm import RMSNorm
    rng = np.random.default_rng(0)
    n = RMSNorm(rt(dtype), size=100, eps=1e-5)
    assert n.tensor_specs()["weight"].shape == (100,)
    w = (1 + 0.1 * rng.standard_normal(100)).astype(np.float32)
    n.bind({"weight": dev(w)})
    resid, delta = rng.standard_normal((5, 100)).astype(np.float32), rng.standard_normal((5, 100)).astype(np.float32)
    r = dev(resid)
    d = dev(delta, dtype)
    out = n.forward(r, d)
    x = resid + d.float().cpu().numpy()
    ref = plain.rms_norm(x, w, 1e-5)
    assert out.dtype == dtype and np.abs(out.float().cpu().numpy() - ref).max() <= (1e-5 if dtype == torch.float32 else 0.03)
    assert np.array_equal(r.cpu().numpy(), x)


def test_rope_part_angles():
    from coheryn_ai_studio_b200.parts.position import RotateHalfRope
    p = RotateHalfRope(rt(), head_dim=48, rotary_dim=48, theta=1e6, max_positions=700)
    table = p.cos_sin().cpu().numpy()
    for pos in (0, 1, 511, 699):
        ang = plain.rope_angles(pos, 48, 1e6)
        assert np.array_equal(table[pos, :, 0], np.cos(ang, dtype=np.float32))
        assert np.array_equal(table[pos, :, 1], np.sin(ang, dtype=np.float32))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window", [(6, 2, 32, None), (5, 5, 16, 7), (4, 1, 64, None)])
def test_attention_part_in_two_portions(dtype, nh, nkv, hd, window):
    """The mixer alone: a sequence in two portions through its own cache equals plain
    attention over the whole sequence."""
    from coheryn_ai_studio_b200.parts import LayerCache
    from coheryn_ai_studio_b200.parts.attention import Attention
    from coheryn_ai_studio_b200.parts.position import RotateHalfRope
    rng = np.random.default_rng(nh)
    H, T, page = 72, 29, 8
    pos = RotateHalfRope(rt(dtype), hd, hd, 1e4, 64)
    att = Attention(rt(dtype), hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd, qkv_bias=True,
                    o_bias=False, window=window, scale=1 / np.sqrt(hd), position=pos)
    w = {k: (rng.standard_normal(s.shape) * (0.2 if "weight" in k else 0.5)).astype(np.float32)
         for k, s in att.tensor_specs().items()}
    att.bind({k: dev(v, dtype) for k, v in w.items()})
    wq = {k: dev(v, dtype).float().cpu().numpy() for k, v in w.items()}
    x = rng.standard_normal((T, H)).astype(np.float32)
    xd = dev(x, dtype)
    xq = xd.float().cpu().numpy()
    pages = -(-T // page)
    k_cache = torch.zeros(pages, nkv, page, hd, dtype=dtype, device=DEV)
    cache = LayerCache(kind="paged", group=0, page_size=page, k=k_cache, v=torch.zeros_like(k_cache))
    out = torch.cat([att.forward(xd[:18], one_request_step(18, 0, page, pages), cache),
                     att.forward(xd[18:], one_request_step(T - 18, 18, page, pages), cache)])
    q = plain.linear(xq, wq["q_proj.weight"], wq["q_proj.bias"])
    k = plain.linear(xq, wq["k_proj.weight"], wq["k_proj.bias"])
    v = plain.linear(xq, wq["v_proj.weight"], wq["v_proj.bias"])
    positions = np.arange(T)
    o = plain.attention(plain.rope(q, positions, hd, 1e4), plain.rope(k, positions, hd, 1e4), v, nh, nkv, hd, window)
    ref = plain.linear(o, wq["o_proj.weight"])
    tol = 2e-4 if dtype == torch.float32 else 0.03 * np.abs(ref).max()
    assert np.abs(out.float().cpu().numpy() - ref).max() <= tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_mlp_part(dtype):
    from coheryn_ai_studio_b200.parts.feedforward import GatedMLP
    rng = np.random.default_rng(1)
    ff = GatedMLP(rt(dtype), hidden_size=72, intermediate_size=200, activation="silu")
    w = {k: (rng.standard_normal(s.shape) * 0.2).astype(np.float32) for k, s in ff.tensor_specs().items()}
    ff.bind({k: dev(v, dtype) for k, v in w.items()})
    wq = {k: dev(v, dtype).float().cpu().numpy() for k, v in w.items()}
    xd = dev(rng.standard_normal((9, 72)).astype(np.float32), dtype)
    xq = xd.float().cpu().numpy()
    ref = plain.linear(plain.swiglu(plain.linear(xq, wq["gate_proj.weight"]), plain.linear(xq, wq["up_proj.weight"])),
                       wq["down_proj.weight"])
    out = ff.forward(xd, None)
    tol = 1e-4 if dtype == torch.float32 else 0.03 * np.abs(ref).max()
    assert np.abs(out.float().cpu().numpy() - ref).max() <= tol
    with pytest.raises(RuntimeError, match="gelu"):
        GatedMLP(rt(dtype), 8, 8, "gelu")


# ---------------------------------------------------------------------------------------
# A toy architecture, defined and registered here.
# ---------------------------------------------------------------------------------------
def toy_decay_mixer_class():
    from coheryn_ai_studio_b200 import ops
    from coheryn_ai_studio_b200.parts import FixedState, Mixer
    from coheryn_ai_studio_b200.weights import TensorSpec

    class DecayMixer(Mixer):
        """State of its own: s_t = decay * s_{t-1} + x_t per request; y_t = W s_t."""
        capturable = False   # reads the step's layout on the host

        def __init__(self, runtime, hidden_size, decay, position=None):
            super().__init__(runtime)
            self.hidden_size, self.decay = hidden_size, decay

        def cache_requirement(self):
            return FixedState((self.hidden_size,), torch.float32)

        def tensor_specs(self):
            return {"mix.weight": TensorSpec((self.hidden_size, self.hidden_size))}

        def bind(self, tensors):
            self.w = tensors["mix.weight"]

        def forward(self, x, step, cache):
            assert cache.kind == "state"
            out = torch.empty_like(x, dtype=torch.float32)
            cu = step.cu_q.tolist()
            for b, slot in enumerate(step.state_slots.tolist()):
                s = cache.state[slot]
                for t in range(cu[b], cu[b + 1]):
                    s = self.decay * s + x[t].float()
                    out[t] = s
                cache.state[slot] = s
            return ops.linear(out.to(x.dtype), self.w)
    return DecayMixer


def toy_routed_ff_class():
    from coheryn_ai_studio_b200 import ops
    from coheryn_ai_studio_b200.parts import FeedForward
    from coheryn_ai_studio_b200.weights import TensorSpec

    class HashRoutedFF(FeedForward):
        """Routing: token id modulo the number of experts picks the expert; each expert is
        down(relu(up x)).  The tokens of an expert are gathered, run and scattered back."""
        capturable = False   # the number of rows per expert is read on the host

        def __init__(self, runtime, hidden_size, intermediate_size, experts):
            super().__init__(runtime)
            self.hidden_size, self.intermediate_size, self.experts = hidden_size, intermediate_size, experts

        def tensor_specs(self):
            specs = {}
            for e in range(self.experts):
                specs[f"experts.{e}.up.weight"] = TensorSpec((self.intermediate_size, self.hidden_size))
                specs[f"experts.{e}.down.weight"] = TensorSpec((self.hidden_size, self.intermediate_size))
            return specs

        def bind(self, tensors):
            self.up = [tensors[f"experts.{e}.up.weight"] for e in range(self.experts)]
            self.down = [tensors[f"experts.{e}.down.weight"] for e in range(self.experts)]

        def forward(self, x, step):
            route = step.token_ids.long() % self.experts
            out = torch.zeros_like(x)
            for e in range(self.experts):
                rows = torch.nonzero(route == e).flatten()
                if rows.numel():
                    h = torch.relu(ops.linear(x.index_select(0, rows).contiguous(), self.up[e]))
                    out.index_copy_(0, rows, ops.linear(h, self.down[e]))
            return out
    return HashRoutedFF


def toy_arrangement_class():
    from coheryn_ai_studio_b200.parts import Arrangement

    class SandwichMixer(Arrangement):
        """x += norm_after(mixer(norm_before(x))) and nothing else: three slots, no feed-forward."""
        SLOTS = {"mixer": "mixer", "before": "norm", "after": "norm"}

        def parts(self):
            return {"before": self.before, "self_attn": self.mixer, "after": self.after}

        def forward(self, residual, delta, step, cache):
            mixed = self.mixer.forward(self.before.forward(residual, delta), step, cache)
            if mixed.dim() == 3:
                mixed = mixed.sum(0)
            scratch = mixed.float().contiguous()              # the second norm normalises the mixer's output alone
            return residual, self.after.forward(scratch, None)
    return SandwichMixer


def toy_position_class():
    from coheryn_ai_studio_b200.parts import Position

    class LinearAngles(Position):
        """Another encoding behind the same interface (rotary_dim, cos_sin()): pair i of the
        first rotary_dim elements turns by position * rate * (i + 1); the rest of the head
        is left as it is."""

        def __init__(self, runtime, head_dim, rotary_dim, rate, max_positions):
            super().__init__(runtime)
            self.head_dim, self.rotary_dim, self.rate, self.max_positions = head_dim, rotary_dim, rate, max_positions
            self._table = None

        def cos_sin(self):
            if self._table is None:
                ang = linear_angles(np.arange(self.max_positions), self.rotary_dim, self.rate)
                t = np.stack([np.cos(ang, dtype=np.float32), np.sin(ang, dtype=np.float32)], axis=-1)
                self._table = torch.from_numpy(np.ascontiguousarray(t)).to(self.runtime.device)
            return self._table
    return LinearAngles


def linear_angles(positions, rotary_dim, rate):
    i = np.arange(1, rotary_dim // 2 + 1, dtype=np.float32)
    return (np.asarray(positions, dtype=np.float32)[:, None] * np.float32(rate) * i[None, :]).astype(np.float32)


def plain_linear_rope(x, positions, head_dim, rotary_dim, rate):
    T, half = x.shape[0], rotary_dim // 2
    h = x.astype(np.float32).reshape(T, -1, head_dim).copy()
    ang = linear_angles(positions, rotary_dim, rate)
    c, s = np.cos(ang, dtype=np.float32)[:, None, :], np.sin(ang, dtype=np.float32)[:, None, :]
    a, b = h[:, :, :half].copy(), h[:, :, half:rotary_dim].copy()
    h[:, :, :half] = a * c - b * s
    h[:, :, half:rotary_dim] = a * s + b * c
    return h.reshape(T, -1)


def toy_spec(c):
    from coheryn_ai_studio_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, prenorm_layer
    H = c["hidden_size"]
    norm = PartSpec("rmsnorm", {"size": H, "eps": c["rms_norm_eps"]})
    rope = PartSpec("rope_rotate_half", {"head_dim": c["head_dim"], "rotary_dim": c["head_dim"],
                                         "theta": c["rope_theta"], "max_positions": c["max_position_embeddings"]})
    def attn(window):
        return PartSpec("attention", {"hidden_size": H, "num_heads": c["num_attention_heads"],
                                      "num_kv_heads": c["num_key_value_heads"], "head_dim": c["head_dim"],
                                      "qkv_bias": True, "o_bias": False, "window": window,
                                      "scale": c["head_dim"] ** -0.5})
    ff = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": c["intermediate_size"], "activation": "silu"})
    routed = PartSpec("test_hash_routed", {"hidden_size": H, "intermediate_size": c["expert_size"], "experts": c["experts"]})
    linear = PartSpec("test_linear_angles", {"head_dim": c["head_dim"], "rotary_dim": c["toy_rotary_dim"],
                                             "rate": c["toy_rate"], "max_positions": c["max_position_embeddings"]})
    layers = [
        prenorm_layer("model.layers.0", attn(None), ff, norm, norm, rope),
        prenorm_layer("model.layers.1", PartSpec("test_decay", {"hidden_size": H, "decay": 0.5}), routed, norm, norm),
        prenorm_layer("model.layers.2", attn(c["window"]), ff, norm, norm, linear),
        # another arrangement, defined in this file: a mixer between two norms and no feed-forward
        LayerSpec("model.layers.3", "test_sandwich_mixer", {"mixer": attn(None), "before": norm, "after": norm}, rope),
    ]
    # layer 0 twice (two caches), the toy layer, the windowed layer, then layer 0 a third
    # time reading the cache its FIRST run wrote
    schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(2), ScheduleEntry(3),
                ScheduleEntry(0, cache_from=0)]
    return ModelSpec("ToyStateForCausalLM", H, c["vocab_size"], c["max_position_embeddings"], "model.embed_tokens",
                     layers, schedule, norm, "model.norm", "lm_head", embedding_scale=c["embedding_scale"],
                     logit_scale=c["logit_scale"], head_bias_name="lm_head.bias")


class ToyConfig(dict):
    def to_dict(self):
        return dict(self)


TOY = ToyConfig(architectures=["ToyStateForCausalLM"], hidden_size=48, num_attention_heads=3, num_key_value_heads=1,
                head_dim=16, intermediate_size=80, vocab_size=130, rms_norm_eps=1e-5, rope_theta=1e4,
                max_position_embeddings=128, window=11, experts=3, expert_size=40, toy_rotary_dim=8, toy_rate=0.01,
                embedding_scale=1.75, logit_scale=0.5)


def toy_plain_forward(cfg, w, ids):
    """The toy model over a whole sequence, from the plain parts."""
    T = len(ids)
    positions = np.arange(T)
    hd, nh, nkv = cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    x = (plain.embedding(w["model.embed_tokens.weight"], ids) * np.float32(cfg["embedding_scale"])).astype(np.float32)
    kept = {}

    def turn(x, i):
        if i == 2:
            return plain_linear_rope(x, positions, hd, cfg["toy_rotary_dim"], cfg["toy_rate"])
        return plain.rope(x, positions, hd, cfg["rope_theta"])

    def attention_layer(x, i, window, entry, cache_from=None):
        p = f"model.layers.{i}."
        y = plain.rms_norm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        q = turn(plain.linear(y, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"]), i)
        if cache_from is None:
            k = turn(plain.linear(y, w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"]), i)
            v = plain.linear(y, w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"])
            kept[entry] = (k, v)
        else:
            k, v = kept[cache_from]
        o = plain.attention(q, k, v, nh, nkv, hd, window)
        return (x + plain.linear(o, w[p + "self_attn.o_proj.weight"])).astype(np.float32)

    def decay_layer(x, i):
        p = f"model.layers.{i}."
        y = plain.rms_norm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        s, rows = np.zeros(y.shape[1], np.float32), []
        for t in range(T):
            s = (np.float32(0.5) * s + y[t]).astype(np.float32)
            rows.append(s)
        return (x + plain.linear(np.stack(rows), w[p + "self_attn.mix.weight"])).astype(np.float32)

    def mlp(x, i):
        p = f"model.layers.{i}."
        y = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        a = plain.swiglu(plain.linear(y, w[p + "mlp.gate_proj.weight"]), plain.linear(y, w[p + "mlp.up_proj.weight"]))
        return (x + plain.linear(a, w[p + "mlp.down_proj.weight"])).astype(np.float32)

    def routed(x, i):
        p = f"model.layers.{i}."
        y = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        out = np.zeros_like(y)
        for t, tok in enumerate(ids):
            e = int(tok) % cfg["experts"]
            h = np.maximum(plain.linear(y[t:t + 1], w[p + f"mlp.experts.{e}.up.weight"]), 0)
            out[t] = plain.linear(h, w[p + f"mlp.experts.{e}.down.weight"])[0]
        return (x + out).astype(np.float32)

    x = mlp(attention_layer(x, 0, None, 0), 0)
    x = routed(decay_layer(x, 1), 1)
    x = mlp(attention_layer(x, 0, None, 2), 0)
    x = mlp(attention_layer(x, 2, cfg["window"], 3), 2)
    def sandwich(x, i, entry):
        p = f"model.layers.{i}."
        y = plain.rms_norm(x, w[p + "before.weight"], cfg["rms_norm_eps"])
        q = turn(plain.linear(y, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"]), i)
        k = turn(plain.linear(y, w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"]), i)
        v = plain.linear(y, w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"])
        o = plain.linear(plain.attention(q, k, v, nh, nkv, hd, None), w[p + "self_attn.o_proj.weight"])
        return (x + plain.rms_norm(o, w[p + "after.weight"], cfg["rms_norm_eps"])).astype(np.float32)

    x = sandwich(x, 3, 4)
    x = mlp(attention_layer(x, 0, None, 5, cache_from=0), 0)
    logits = plain.linear(plain.rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"]), w["lm_head.weight"])
    return (logits * np.float32(cfg["logit_scale"]) + w["lm_head.bias"].astype(np.float32)).astype(np.float32)


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    from coheryn_ai_studio_b200.config import register_architecture, unregister_architecture
    from coheryn_ai_studio_b200.engine import write_random_model
    from coheryn_ai_studio_b200.parts import (ARRANGEMENTS, FEED_FORWARDS, MIXERS, POSITIONS, register_arrangement,
                                              register_feed_forward, register_mixer, register_position)
    from coheryn_ai_studio_b200.weights import InitPolicy
    register_mixer("test_decay", toy_decay_mixer_class())
    register_feed_forward("test_hash_routed", toy_routed_ff_class())
    register_position("test_linear_angles", toy_position_class())
    register_arrangement("test_sandwich_mixer", toy_arrangement_class())
    register_architecture("ToyStateForCausalLM", lambda obj: ToyConfig(obj), toy_spec)
    d = str(tmp_path_factory.mktemp("toy") / "model")
    write_random_model(d, TOY, 7, InitPolicy(0.08, 0.2, 0.05))
    yield d
    unregister_architecture("ToyStateForCausalLM")
    MIXERS.pop("test_decay", None)
    FEED_FORWARDS.pop("test_hash_routed", None)
    POSITIONS.pop("test_linear_angles", None)
    ARRANGEMENTS.pop("test_sandwich_mixer", None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_steps_through_the_engine(toy_folder, dtype):
    """Registered, built from config.json, loaded by tensor name and stepped in portions
    beside another request, with no change to the framework."""
    from replay import Replay, tol_bf16_spread
    cfg, w = plain.read_model(toy_folder)
    assert "model.layers.1.self_attn.mix.weight" in w and "model.layers.1.self_attn.q_proj.weight" not in w
    assert "model.layers.1.mlp.experts.2.up.weight" in w and "model.layers.1.mlp.gate_proj.weight" not in w
    rng = np.random.default_rng(3)
    seqs = {"a": rng.integers(0, 130, 45).tolist(), "b": rng.integers(0, 130, 30).tolist()}
    r = Replay(toy_folder, dtype, max_tokens=128, page_size=8)
    assert len(r.cache.groups) == 2                       # full attention (3 entries) and the window
    assert [len(g.entries) for g in r.cache.groups] == [3, 1]
    r.step([("a", seqs["a"][:20], list(range(20)))])
    r.step([("a", seqs["a"][20:23], [0, 1, 2]), ("b", seqs["b"][:17], list(range(17)))])
    r.step([("a", seqs["a"][23:], list(range(22))), ("b", seqs["b"][17:19], [0, 1])])
    for t in range(19, 30):
        r.step([("b", [seqs["b"][t]], [0])])
    # the window (11) has passed the first pages of 8: they went back to the pool
    assert r.cache.block_table("a", 1)[:4] == [-1] * 4 and r.cache.block_table("a", 0)[0] >= 0
    for rid, seq in seqs.items():
        ref = toy_plain_forward(cfg, w, seq)
        for (k, pos), row in r.rows.items():
            if k == rid:
                tol = 2e-4 if dtype == "float32" else tol_bf16_spread(ref[pos], 0.1)
                assert np.abs(row - ref[pos]).max() <= tol, (rid, pos)
    r.cache.free("a"); r.cache.free("b"); r.cache.check()
    assert r.cache.available_pages() == [16, 16]


def test_toy_architecture_generates_through_the_entry_point(toy_folder):
    """The same folder through the Python entry point (scheduler, sampler, graphs requested):
    its parts are not capturable, so the engine steps it without graphs; greedy tokens equal
    the plain implementation's."""
    from coheryn_ai_studio_b200.api import generate
    cfg, w = plain.read_model(toy_folder)
    prompt = np.random.default_rng(5).integers(0, 130, 9).tolist()
    out = generate(toy_folder, [prompt], max_tokens=6, dtype="float32", context=64)
    seq = list(prompt)
    for _ in range(6):
        seq.append(int(np.argmax(toy_plain_forward(cfg, w, seq)[-1])))
    assert list(out[0]["token_ids"]) == seq[len(prompt):]


# ------------------------------------------------------------------ fixed state and a window under CUDA graphs
def device_decay_mixer_class():
    from coheryn_ai_studio_b200 import ops
    from coheryn_ai_studio_b200.parts import FixedState, Mixer
    from coheryn_ai_studio_b200.weights import TensorSpec

    class DeviceDecayMixer(Mixer):
        """state = decay * state + x per request, kept in a fixed-state slot; never reads a result on
        the host, so a decode step with it can be captured in a CUDA graph (capturable stays True)."""

        def __init__(self, runtime, hidden_size, decay):
            super().__init__(runtime)
            self.hidden_size, self.decay = hidden_size, float(decay)

        def cache_requirement(self):
            return FixedState((self.hidden_size,), torch.float32)

        def tensor_specs(self):
            return {"mix.weight": TensorSpec((self.hidden_size, self.hidden_size))}

        def bind(self, tensors):
            self.w = tensors["mix.weight"]

        def forward(self, x, step, cache):
            xs = x.float()
            if step.max_q_len == 1:
                slots = step.state_slots.long()
                out = cache.state.index_select(0, slots) * self.decay + xs
                cache.state.index_copy_(0, slots, out)
            else:
                out, o = torch.empty_like(xs), 0
                for b, n in enumerate(step.q_lens):
                    slot = step.state_slots[b:b + 1].long()
                    s = cache.state.index_select(0, slot)[0]
                    for t in range(o, o + n):
                        s = self.decay * s + xs[t]
                        out[t] = s
                    cache.state.index_copy_(0, slot, s[None])
                    o += n
            return ops.linear(out.to(x.dtype), self.w)
    return DeviceDecayMixer


GRAPH_TOY = ToyConfig(architectures=["ToyGraphForCausalLM"], hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
                      head_dim=16, intermediate_size=96, vocab_size=200, rms_norm_eps=1e-6, rope_theta=1e4,
                      max_position_embeddings=128, window=7)


def graph_toy_spec(c):
    from coheryn_ai_studio_b200.config import ModelSpec, PartSpec, ScheduleEntry, prenorm_layer
    H = c["hidden_size"]
    norm = PartSpec("rmsnorm", {"size": H, "eps": c["rms_norm_eps"]})
    rope = PartSpec("rope_rotate_half", {"head_dim": c["head_dim"], "rotary_dim": c["head_dim"], "theta": c["rope_theta"],
                                         "max_positions": c["max_position_embeddings"]})
    attn = PartSpec("attention", {"hidden_size": H, "num_heads": c["num_attention_heads"], "num_kv_heads": c["num_key_value_heads"],
                                  "head_dim": c["head_dim"], "qkv_bias": True, "o_bias": False, "window": c["window"],
                                  "scale": c["head_dim"] ** -0.5})
    ff = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": c["intermediate_size"], "activation": "silu"})
    layers = [prenorm_layer("model.layers.0", attn, ff, norm, norm, rope),
              prenorm_layer("model.layers.1", PartSpec("test_device_decay", {"hidden_size": H, "decay": 0.5}), ff, norm, norm)]
    return ModelSpec("ToyGraphForCausalLM", H, c["vocab_size"], c["max_position_embeddings"], "model.embed_tokens", layers,
                     [ScheduleEntry(0), ScheduleEntry(1)], norm, "model.norm", None)


def graph_toy_plain(cfg, w, ids):
    T, positions = len(ids), np.arange(len(ids))
    hd, nh, nkv, eps = cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["rms_norm_eps"]
    x = plain.embedding(w["model.embed_tokens.weight"], ids)

    def mlp(x, p):
        y = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        a = plain.swiglu(plain.linear(y, w[p + "mlp.gate_proj.weight"]), plain.linear(y, w[p + "mlp.up_proj.weight"]))
        return (x + plain.linear(a, w[p + "mlp.down_proj.weight"])).astype(np.float32)
    p = "model.layers.0."
    y = plain.rms_norm(x, w[p + "input_layernorm.weight"], eps)
    q = plain.rope(plain.linear(y, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"]), positions, hd, cfg["rope_theta"])
    k = plain.rope(plain.linear(y, w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"]), positions, hd, cfg["rope_theta"])
    v = plain.linear(y, w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"])
    x = (x + plain.linear(plain.attention(q, k, v, nh, nkv, hd, cfg["window"]), w[p + "self_attn.o_proj.weight"])).astype(np.float32)
    x = mlp(x, p)
    p = "model.layers.1."
    y = plain.rms_norm(x, w[p + "input_layernorm.weight"], eps)
    s, rows = np.zeros(y.shape[1], np.float32), []
    for t in range(T):
        s = (np.float32(0.5) * s + y[t]).astype(np.float32)
        rows.append(s)
    x = (x + plain.linear(np.stack(rows), w[p + "self_attn.mix.weight"])).astype(np.float32)
    x = mlp(x, p)
    return plain.linear(plain.rms_norm(x, w["model.norm.weight"], eps), w["model.embed_tokens.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_fixed_state_and_a_window_under_cuda_graphs(tmp_path, dtype):
    """A model whose parts can all be captured, one of them a mixer with state of its own, the other
    attention with a window (pages go back while decoding): decode steps replayed from CUDA graphs
    give the logits of the plain implementation, for every batch width met, although the capture's
    warm-up runs the step several times (the state is put back) and a window rewrites block-table
    rows in place."""
    from coheryn_ai_studio_b200.config import register_architecture, unregister_architecture
    from coheryn_ai_studio_b200.engine import write_random_model
    from coheryn_ai_studio_b200.parts import MIXERS, register_mixer
    from coheryn_ai_studio_b200.weights import InitPolicy
    from replay import Replay, tol_bf16_spread
    register_mixer("test_device_decay", device_decay_mixer_class())
    register_architecture("ToyGraphForCausalLM", lambda obj: ToyConfig(obj), graph_toy_spec)
    try:
        folder = str(tmp_path / "graph_toy")
        write_random_model(folder, GRAPH_TOY, 13, InitPolicy(0.08, 0.2, 0.05))
        cfg, w = plain.read_model(folder)
        rng = np.random.default_rng(8)
        seqs = {k: rng.integers(0, 200, n).tolist() for k, n in (("a", 40), ("b", 31), ("c", 26))}
        r = Replay(folder, dtype, max_tokens=128, page_size=4, use_graphs=True)
        assert r.runner.use_graphs and r.cache.has_fixed_state
        r.step([("a", seqs["a"][:9], [8]), ("b", seqs["b"][:5], [4])])
        for t in range(20):                                   # widths 2, then 3, then 2 again
            entries = [("a", [seqs["a"][9 + t]], [0]), ("b", [seqs["b"][5 + t]], [0])]
            if 4 <= t < 14:
                entries.append(("c", [seqs["c"][t - 4]], [0]))
            r.step(entries, end=["c"] if t == 13 else ())
        assert sorted(r.runner._graphs) == [2, 3] and all(g.graph is not None for g in r.runner._graphs.values())
        assert r.cache.block_table("a", 0)[:4] == [-1] * 4      # the window of 7 has passed the first pages of 4
        for rid, seq in seqs.items():
            ref = graph_toy_plain(cfg, w, seq)
            rows = [(pos, row) for (k, pos), row in r.rows.items() if k == rid]
            assert len(rows) >= 10
            for pos, row in rows:
                tol = 2e-4 if dtype == "float32" else tol_bf16_spread(ref[pos], 0.1)
                assert np.abs(row - ref[pos]).max() <= tol, (rid, pos)
    finally:
        unregister_architecture("ToyGraphForCausalLM")
        MIXERS.pop("test_device_decay", None)


def test_describe_reports_capabilities_and_cache_cost(toy_folder):
    """The registry's metadata face (crates/coheryn-engine/src/adapters.rs:11-21, 39-58): the toy
    architecture keeps fixed state, so its bytes per request are not zero."""
    from coheryn_ai_studio_b200.config import describe_model
    d = describe_model(toy_folder)
    caps = d["capabilities"]
    assert caps["architecture"] == "ToyStateForCausalLM" and caps["adapter"] == "toystateforcausallm-b200-v1"
    assert caps["fixed_state_bytes_per_request"] == 48 * 4 and caps["paged_kv"]
    # four cache entries hold keys and values (three full, one windowed): 2 * kv heads * head size each
    assert caps["kv_bytes_per_token"] == {"bfloat16": 2 * 4 * 2 * 16, "float32": 4 * 4 * 2 * 16}
    assert d["attention_windows"] == [11] and d["schedule_entries"] == 6 and d["layers"] == 4


@pytest.mark.parametrize("name", ["A_loud", "B_loud"])
def test_block_enqueued_by_one_call_equals_the_parts_bit_for_bit(tmp_path, name):
    """A block of the built-in parts in bfloat16 is enqueued by one call into the library
    (csrc/block_runner.cu), which chooses the kernels as ops.py does; so its logits equal, bit for
    bit, those of the parts run one by one: whole prompts of many lengths (every row wanted), requests
    decoding together, decoded tokens beside prompt portions.  float32 keeps the parts' own path."""
    import tiny
    from coheryn_ai_studio_b200 import ops
    from coheryn_ai_studio_b200.engine import Engine, StepEntry
    from coheryn_ai_studio_b200.parts import native_block
    folder = tiny.make_folder(tmp_path, name)
    cfg = tiny.CONFIGS[name][0]
    context = min(256, cfg.max_position_embeddings)

    def run(native, dtype="bfloat16"):
        ops.set_native_block(native)
        try:
            eng = Engine.from_folder(folder, dtype, context=context, max_num_seqs=4, page_size=16, use_graphs=False)
            before = native_block.runs
            outs = []
            for n in (1, 2, 5, 16, 17, 33, 40, 64, 70, 130, 200):
                eng.cache.admit(f"w{n}")
                outs.append(eng.runner.step([StepEntry(f"w{n}", tiny.prompt(n, n, cfg.vocab_size), list(range(n)))]).clone())
                eng.cache.free(f"w{n}")
            for i, n in enumerate((30, 7, 90)):
                eng.cache.admit(f"r{i}")
                outs.append(eng.runner.step([StepEntry(f"r{i}", tiny.prompt(100 + i, n, cfg.vocab_size), [n - 1])]).clone())
            for t in range(3):
                outs.append(eng.runner.step([StepEntry(f"r{i}", [3 + 5 * t + i], [0]) for i in range(3)]).clone())
            eng.cache.admit("m")
            outs.append(eng.runner.step([StepEntry("r0", [9], [0]), StepEntry("m", tiny.prompt(5, 21, cfg.vocab_size), list(range(21))),
                                         StepEntry("r2", [11, 12], [0, 1])]).clone())
            eng.runner.check_status()
            return outs, native_block.runs - before, eng.model.layers[0]._native
        finally:
            ops.set_native_block(True)

    parts, none_native, _ = run(False)
    whole, some_native, described = run(True)
    assert none_native == 0 and some_native >= len(whole) * (cfg.num_hidden_layers - 1)
    assert isinstance(described, native_block.NativeBlock)
    for k, (a, b) in enumerate(zip(parts, whole)):
        assert torch.isfinite(b).all() and torch.equal(a, b), k
    _, in_float32, described = run(True, "float32")
    assert in_float32 == 0 and described is False
