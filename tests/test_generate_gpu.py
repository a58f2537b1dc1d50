"""Generation through the engine and its entry points: greedy and sampled tokens equal
the plain implementation's, with continuous batching, with preemption and with prefix
reuse."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_qwen2 as plain
import tiny
from replay import assert_greedy_follows_plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("gen")
    return {n: tiny.make_folder(base, n, policy=tiny.POLICY_LOUD) for n in ("A", "B")}


def plain_generate(folder, prompt, steps, sampler=None):
    cfg, w = plain.read_model(folder)
    ids, out = list(prompt), []
    for _ in range(steps):
        logits = plain.forward(cfg, w, ids)[-1]
        tok = int(np.argmax(logits)) if sampler is None else sampler.sample(logits)
        if sampler is not None:
            sampler.observe(tok)
        out.append(tok); ids.append(tok)
    return out


def test_greedy_three_requests_float32(folders):
    """Tiny A: prompts of 5, 17 and 33 ids, 8 greedy tokens each, identical to the plain run."""
    from coheryn_ai_studio_b200.engine import Engine
    eng = Engine.from_folder(folders["A"], "float32", context=128, max_num_seqs=4)
    prompts = [tiny.prompt(60 + i, n, 512) for i, n in enumerate((5, 17, 33))]
    res = eng.generate(prompts, max_tokens=8)
    for p, r in zip(prompts, res):
        assert r.token_ids == plain_generate(folders["A"], p, 8)
        assert r.finish_reason == "length" and r.completion_tokens == 8 and r.prompt_tokens == len(p)
    eng.cache.check()
    assert eng.cache.available_pages() == [eng.cache.num_pages]


def test_continuous_batching_mixed_float32(folders):
    """Tiny B: prompts of 1, 9, 64 and 130 ids as one mixed batch with 16-token portions and
    pages of 16; greedy, and temperature 0.8 with a fixed seed."""
    from coheryn_ai_studio_b200.engine import Engine
    from coheryn_ai_studio_b200.sampling import SamplingParams
    eng = Engine.from_folder(folders["B"], "float32", context=256, max_num_seqs=4,
                             max_num_batched_tokens=16, page_size=16)
    prompts = [tiny.prompt(70 + i, n, 1000) for i, n in enumerate((1, 9, 64, 130))]
    res = eng.generate(prompts, max_tokens=6)
    for p, r in zip(prompts, res):
        assert r.token_ids == plain_generate(folders["B"], p, 6)
    assert eng.scheduler.stats["max_batch_width"] >= 3
    params = [SamplingParams(temperature=0.8, seed=11 + i, top_k=(0, 40, 0, 5)[i], top_p=(1.0, 1.0, 0.9, 1.0)[i])
              for i in range(4)]
    res = eng.generate(prompts, max_tokens=5, params=params)
    for i, (p, r) in enumerate(zip(prompts, res)):
        s = plain.PlainSampler(temperature=0.8, seed=11 + i, top_k=params[i].top_k, top_p=params[i].top_p)
        assert r.token_ids == plain_generate(folders["B"], p, 5, s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_and_prefix_reuse_change_nothing(folders, dtype):
    from coheryn_ai_studio_b200.engine import Engine
    shared = tiny.prompt(80, 40, 512)
    prompts = [shared + tiny.prompt(81 + i, 3 + 5 * i, 512) for i in range(4)]
    def run(**kw):
        eng = Engine.from_folder(folders["A"], dtype, context=128, max_num_seqs=4, page_size=16, **kw)
        if kw.get("prefix_reuse"):
            eng.generate(prompts[:1], max_tokens=2)      # leaves the shared prefix's pages behind
        res = eng.generate(prompts, max_tokens=24)
        eng.cache.check()
        return [r.token_ids for r in res], eng, res
    base, _, _ = run(prefix_reuse=False)
    tight, eng, res = run(prefix_reuse=False, num_pages=12)       # 192 tokens for 4 x ~80
    assert eng.scheduler.stats["preemptions"] > 0 and tight == base
    reuse, eng, res = run(prefix_reuse=True)
    assert reuse == base and sum(r.reused_prompt_tokens for r in res) >= 32
    if dtype == "float32":
        assert base[0] == plain_generate(folders["A"], prompts[0], 24)
    for p, toks in zip(prompts, base):
        assert_greedy_follows_plain(folders["A"], p, toks, dtype, "preemption")


def test_stop_token_and_penalties(folders):
    from coheryn_ai_studio_b200.engine import Engine
    from coheryn_ai_studio_b200.sampling import SamplingParams
    eng = Engine.from_folder(folders["A"], "float32", context=128, max_num_seqs=2)
    p = tiny.prompt(90, 12, 512)
    free = eng.generate([p], max_tokens=10)[0].token_ids
    stop = eng.generate([p], max_tokens=10, stop_tokens=[free[3]])[0]
    k = free.index(free[3])
    assert stop.token_ids == free[:k + 1] and stop.finish_reason == "stop"
    params = SamplingParams(temperature=0.7, seed=5, repetition_penalty=1.3, frequency_penalty=0.4,
                            presence_penalty=0.2, top_p=0.95)
    got = eng.generate([p], max_tokens=8, params=params)[0].token_ids
    s = plain.PlainSampler(temperature=0.7, seed=5, repetition_penalty=1.3, frequency_penalty=0.4,
                           presence_penalty=0.2, top_p=0.95)
    for t in p:
        s.observe(t)
    assert got == plain_generate(folders["A"], p, 8, s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_step_launched_ahead_changes_nothing(folders, dtype):
    """The decode step that is launched before the previous step's ids are read (they pass from
    step to step on the device): the same tokens and reasons as without it, with requests that
    end at different times by length and by a stop token, sampled and greedy, with prefix reuse
    on; no page is lost."""
    from coheryn_ai_studio_b200.engine import Engine
    from coheryn_ai_studio_b200.sampling import SamplingParams
    shared = tiny.prompt(95, 33, 512)
    prompts = [shared + tiny.prompt(96 + i, 2 + 3 * i, 512) for i in range(4)]
    params = [SamplingParams(), SamplingParams(temperature=0.9, seed=3), SamplingParams(), SamplingParams(temperature=0.5, seed=8, top_k=20)]
    def run(lookahead, stop=()):
        eng = Engine.from_folder(folders["A"], dtype, context=128, max_num_seqs=4, page_size=16, lookahead=lookahead)
        ids = [eng.add_request(p, max_tokens=m, params=pr, stop_tokens=stop) for p, m, pr in zip(prompts, (5, 30, 17, 22), params)]
        steps = 0
        while eng.has_work():
            eng.step(); steps += 1
        res = [eng.result(i) for i in ids]
        eng.cache.check()
        assert eng.cache.available_pages() == [eng.cache.num_pages]      # idle hashed pages count as available: none lost
        again = eng.generate(prompts[:2], max_tokens=4)      # the engine goes on after the pipeline drained
        return [(r.token_ids, r.finish_reason) for r in res], [r.token_ids for r in again]
    base, base2 = run(False)
    ahead, ahead2 = run(True)
    assert ahead == base and ahead2 == base2
    stop_tok = base[1][0][6]
    assert run(True, stop=[stop_tok]) == run(False, stop=[stop_tok])


def test_refusals(folders):
    from coheryn_ai_studio_b200.engine import Engine, RequestRefused
    eng = Engine.from_folder(folders["A"], "float32", context=64, max_num_seqs=2)
    with pytest.raises(RequestRefused):
        eng.add_request([], 4)
    with pytest.raises(RequestRefused):
        eng.add_request([1] * 60, 5)
    with pytest.raises(RequestRefused):
        eng.add_request([512], 5)
    with pytest.raises(ValueError):
        Engine.from_folder(folders["A"], "float32", context=1000)      # beyond the model's positions
    assert eng.generate([[1, 2, 3]], max_tokens=0)[0].finish_reason == "length"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_command_line_and_python_entry(folders, dtype):
    from coheryn_ai_studio_b200 import api
    p = tiny.prompt(95, 9, 512)
    want = plain_generate(folders["A"], p, 6)
    out = api.run(folders["A"], tokens=p, max_tokens=6, context=64, dtype=dtype, timeout=900)
    assert out["prompt_tokens"] == 9 and out["completion_tokens"] == 6 and out["finish_reason"] == "length"
    if dtype == "float32":
        assert out["token_ids"] == want
    assert_greedy_follows_plain(folders["A"], p, out["token_ids"], dtype, "entry point")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "coheryn"), "run", folders["A"], "--tokens",
                        ",".join(map(str, p)), "--max-tokens", "6", "--context", "64", "--dtype", dtype, "--stream"],
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and [int(t) for t in r.stdout.split()] == out["token_ids"]
    bad = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "coheryn"), "--json", "run", folders["A"],
                          "--tokens", "1,2", "--max-tokens", "6", "--context", "4"], capture_output=True, text=True)
    assert bad.returncode == 2 and json.loads(bad.stderr.strip().splitlines()[-1])["code"] == "invalid_request"
    assert api.generate(folders["A"], [p], max_tokens=6, context=64, dtype=dtype)[0]["token_ids"] == out["token_ids"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_zero_matrices_generate_token_zero(tmp_path, dtype):
    """The reference's synthetic model (crates/coheryn-engine/tests/common/mod.rs:99-118,
    tests/engine.rs:35-59): embeddings 1, every matrix 0, so all logits are 0 and greedy
    generation emits token 0 for ever (the first maximum)."""
    import torch
    from coheryn_ai_studio_b200.api import generate
    from coheryn_ai_studio_b200.weights.loader import write_model_folder
    H, V, I = 32, 259, 48
    cfg = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=1, hidden_size=H,
               num_attention_heads=2, num_key_value_heads=1, intermediate_size=I, vocab_size=V, rms_norm_eps=1e-6,
               rope_theta=1e6, max_position_embeddings=64, hidden_act="silu", tie_word_embeddings=False)
    bf = torch.bfloat16
    w = {"model.embed_tokens.weight": torch.ones(V, H, dtype=bf), "model.norm.weight": torch.ones(H),
         "lm_head.weight": torch.zeros(V, H, dtype=bf)}
    p = "model.layers.0."
    for n, shape in [("self_attn.q_proj.weight", (H, H)), ("self_attn.k_proj.weight", (H // 2, H)),
                     ("self_attn.v_proj.weight", (H // 2, H)), ("self_attn.o_proj.weight", (H, H)),
                     ("mlp.gate_proj.weight", (I, H)), ("mlp.up_proj.weight", (I, H)), ("mlp.down_proj.weight", (H, I))]:
        w[p + n] = torch.zeros(shape, dtype=bf)
    for n, size in [("self_attn.q_proj.bias", H), ("self_attn.k_proj.bias", H // 2), ("self_attn.v_proj.bias", H // 2)]:
        w[p + n] = torch.zeros(size)
    w[p + "input_layernorm.weight"] = torch.ones(H)
    w[p + "post_attention_layernorm.weight"] = torch.ones(H)
    folder = str(tmp_path / "zeros")
    write_model_folder(folder, cfg, w)
    out = generate(folder, [[5], [7, 8, 9]], max_tokens=4, dtype=dtype, context=32)
    assert [r["token_ids"] for r in out] == [[0, 0, 0, 0], [0, 0, 0, 0]]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_draining_batch_replays_padded_graphs(folders, dtype):
    """Twelve requests that end at different times: the decode batch shrinks from 12 to 1, batches of
    9 to 12 rows replay the graph of width 16 with padding rows on the cache's spare page, and the
    tokens equal those of an engine that steps without graphs."""
    from coheryn_ai_studio_b200.engine import Engine
    prompts = [tiny.prompt(70 + i, 3 + 2 * i, tiny.CONFIGS["B"][0].vocab_size) for i in range(12)]
    limits = [3 + (5 * i) % 11 for i in range(12)]

    def run(use_graphs):
        eng = Engine.from_folder(folders["B"], dtype, context=128, max_num_seqs=12, use_graphs=use_graphs)
        ids = [eng.add_request(p, max_tokens=n) for p, n in zip(prompts, limits)]
        while eng.has_work():
            eng.step()
        eng.cache.check()
        return [eng.result(i).token_ids for i in ids], eng
    with_graphs, eng = run(True)
    without, _ = run(False)
    assert [len(t) for t in with_graphs] == limits
    widths = sorted(eng.runner._graphs)
    assert 16 in widths and not any(8 < w < 16 for w in widths)
    if dtype == "float32":
        assert with_graphs == without
    # bfloat16 kernels are chosen by the batch's width, so the two runs may part at a near-tie; every
    # token of both is the plain implementation's choice given the tokens before it
    for p, a, b in zip(prompts, with_graphs, without):
        assert_greedy_follows_plain(folders["B"], p, a, dtype, "graphs")
        assert_greedy_follows_plain(folders["B"], p, b, dtype, "no graphs")


def test_decode_steps_queued_behind_a_busy_device_keep_their_own_inputs(folders):
    """Decode steps replayed from graphs take their positions, lengths, slots and block tables from a
    pinned staging buffer by an asynchronous copy, which reads the buffer when the DEVICE gets to it.
    With the device a long way behind (a queue of heavy products in front) and the host running many
    steps ahead without waiting, every step must still see its own inputs: the logits equal those of
    the same steps run one at a time."""
    import torch
    from coheryn_ai_studio_b200 import ops
    from coheryn_ai_studio_b200.cache import CacheManager
    from coheryn_ai_studio_b200.engine import StepEntry, StepRunner, load_model
    dev = torch.device("cuda:0")
    model = load_model(folders["B"], "float32")[1]
    V = tiny.CONFIGS["B"][0].vocab_size
    seqs = [tiny.prompt(40 + i, 40 + 3 * i, V) for i in range(3)]
    heavy_x = torch.randn(2048, 2048, device=dev)
    heavy_out = torch.empty(2048, 2048, device=dev)

    def run(lagging):
        cache = CacheManager(model.cache_requirements(), [None] * len(model.spec.schedule), torch.float32, dev,
                             page_size=4, num_pages=64, max_requests=4, prefix_reuse=False)
        runner = StepRunner(model, cache, use_graphs=True, graph_max_kv_len=64)
        for i, s in enumerate(seqs):
            cache.admit(f"r{i}")
        runner.step([StepEntry(f"r{i}", s[:10], []) for i, s in enumerate(seqs)])
        runner.step([StepEntry(f"r{i}", [s[10]], [0]) for i, s in enumerate(seqs)])      # captures the graph
        torch.cuda.synchronize()
        if lagging:
            for _ in range(40):                                # tens of milliseconds of queued work
                ops.gemm_simt(heavy_x, heavy_x, None, heavy_out)
        out = []
        for t in range(11, 35):
            logits = runner.step([StepEntry(f"r{i}", [s[t]], [0]) for i, s in enumerate(seqs)])
            out.append(logits.clone())
            if not lagging:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        runner.check_status()
        return torch.stack(out).cpu()
    assert torch.equal(run(True), run(False))


def test_trace_command_prints_layer_outputs_and_logits(folders):
    """``coheryn trace``: per position one line for every layer's output and one for the logits
    (crates/coheryn-engine/src/inference.rs:541-556, crates/coheryn-cli/src/main.rs:487-506), equal
    to the plain implementation's."""
    p = tiny.prompt(97, 6, 512)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "coheryn"), "trace", folders["A"], "--tokens",
                        ",".join(map(str, p)), "--context", "64", "--dtype", "float32"], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert [(l["position"], l["name"]) for l in lines] == [(t, n) for t in range(6) for n in ("blk.0.output", "blk.1.output", "logits")]
    cfg, w = plain.read_model(folders["A"])
    layers = []
    ref = plain.forward(cfg, w, p, layer_outputs=layers)
    for l in lines:
        want = ref[l["position"]] if l["name"] == "logits" else layers[int(l["name"].split(".")[1])][l["position"]]
        assert np.abs(np.asarray(l["values"], np.float32) - want).max() <= 1e-4 * max(1.0, float(np.abs(want).max()))
