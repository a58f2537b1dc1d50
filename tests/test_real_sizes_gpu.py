"""The engine at the layer sizes of Qwen2.5-1.5B, 7B and 14B (two layers of each: the widths, head
counts, intermediate sizes and vocabularies of the full configurations, which have 28, 28 and 48
layers) against the plain implementation, in float32 and in bfloat16.

These are the shapes that the benchmark's kernels run: a 2,048-token portion goes through the
products by CTA pairs, the tcgen05 attention and the last layer's shortcut; a mixed step puts a
decoded token beside portions of two other prompts; 32 decode steps replay CUDA graphs.  The
weights are the seeded random weights of the random-weights mode (matrices and biases N(0, 0.02^2),
norm weights 1), made on the device; a sample of every tensor is checked bit for bit against the
numpy restatement of the generator, and the plain implementation computes with exactly those values.
The reference compares every layer output and all logits of its pinned models within
0.003 + 0.001 |ref| (fixtures/models.json:48-53, crates/coheryn-engine/tests/reference.rs:9-46); here
the float32 path has to meet 1e-4 with the same first maximum, the bfloat16 path the bound of
tests/replay.py (twice what rounding to bfloat16 between the parts costs the plain model itself)."""
import time

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
import plain_random as pr
from replay import TOL_F32, Replay, bf16_excess

pytestmark = pytest.mark.gpu

SIZES = {
    "1.5b": dict(vocab_size=151936, hidden_size=1536, intermediate_size=8960, num_attention_heads=12,
                 num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6, tie_word_embeddings=True, layers_of_config=28),
    "7b": dict(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_attention_heads=28,
               num_key_value_heads=4, head_dim=128, rms_norm_eps=1e-6, tie_word_embeddings=False, layers_of_config=28),
    "14b": dict(vocab_size=152064, hidden_size=5120, intermediate_size=13824, num_attention_heads=40,
                num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5, tie_word_embeddings=False, layers_of_config=48),
}
LAYERS = 2
SEED = 2024


def build(size):
    from coheryn_ai_studio_b200.config import Qwen2Config, qwen2_model_spec
    from coheryn_ai_studio_b200.parts import DecoderModel, Runtime
    from coheryn_ai_studio_b200.weights import InitPolicy, kept_dtype, random_tensors
    sizes = dict(SIZES[size])
    sizes.pop("layers_of_config")
    cfg = Qwen2Config(num_hidden_layers=LAYERS, max_position_embeddings=32768, rope_theta=1e6, **sizes)
    spec = qwen2_model_spec(cfg)
    dev = torch.device("cuda:0")
    policy = InitPolicy(matrix_std=0.02, bias_std=0.02, norm_jitter=0.0)
    specs = DecoderModel(spec, Runtime(torch.bfloat16, dev)).tensor_specs()
    raw = random_tensors(specs, SEED, policy, store=torch.bfloat16, device=dev)

    # a sample of every tensor, bit for bit against the numpy generator
    rng = np.random.default_rng(1)
    for name, t in raw.items():
        n = t.numel()
        idx = np.unique(np.concatenate([rng.integers(0, n, 1500), [0, n - 1]])).astype(np.uint64)
        mean, dev_ = {"normal": (0.0, policy.matrix_std), "bias": (0.0, policy.bias_std), "norm": (1.0, 0.0)}[specs[name].init]
        want = pr.values(pr.tensor_key(SEED, name), idx, mean, dev_)
        if t.dtype == torch.bfloat16:
            want = pr.round_bf16(want)
        got = t.flatten()[torch.from_numpy(idx.astype(np.int64)).to(dev)].float().cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), name

    def model(dtype):
        m = DecoderModel(spec, Runtime(dtype, dev))
        m.bind({n: t.to(kept_dtype(specs[n], t.dtype, dtype)).contiguous() for n, t in raw.items()})
        return m
    weights = {n: t.float().cpu().numpy() for n, t in raw.items()}
    return cfg, model, weights


def script(V):
    rng = np.random.default_rng(5)
    seqs = {"a": rng.integers(0, V, 2048 + 2 + 31).tolist(), "b": rng.integers(0, V, 300 + 1 + 31).tolist(),
            "c": rng.integers(0, V, 40).tolist()}
    steps = [
        [("a", seqs["a"][:2048], [0, 777, 2047])],                                              # few rows: the shortcut
        [("a", seqs["a"][2048:2049], [0]), ("b", seqs["b"][:300], [5, 299]), ("c", seqs["c"][:2], [1])],
        [("a", seqs["a"][2049:2050], [0]), ("b", seqs["b"][300:301], [0]), ("c", seqs["c"][2:], [37])],
    ]
    for t in range(31):                                                                         # decoding, from graphs
        steps.append([("a", [seqs["a"][2050 + t]], [0]), ("b", [seqs["b"][301 + t]], [0])])
    compared = {"a": [0, 777, 2047, 2048, 2049, 2050, 2066, 2080], "b": [5, 299, 300, 301, 317, 331], "c": [1, 39]}
    return seqs, steps, compared


@pytest.mark.parametrize("size", ["1.5b", "7b", "14b"])
def test_layer_sizes_against_the_plain_implementation(size):
    t0 = time.time()
    cfg, model, weights = build(size)
    seqs, steps, compared = script(cfg.vocab_size)
    plain_cfg = cfg.to_dict()
    ref = {rid: plain.forward(plain_cfg, weights, seqs[rid], rows=rows) for rid, rows in compared.items()}
    twin = {rid: plain.forward(plain_cfg, weights, seqs[rid], rows=rows, rounded=True) for rid, rows in compared.items()}
    t_plain = time.time() - t0
    for dtype in ("float32", "bfloat16"):
        r = Replay(None, dtype, max_tokens=2112 + 384 + 64, model=model(torch.float32 if dtype == "float32" else torch.bfloat16),
                   use_graphs=True)
        for entries in steps:
            r.step(entries)
        assert len(r.runner._graphs) == 1 and next(iter(r.runner._graphs.values())).graph is not None
        worst, largest = 0.0, 0.0
        for rid, rows in compared.items():
            for i, pos in enumerate(rows):
                got, want = r.rows[(rid, pos)], ref[rid][i]
                diff = float(np.abs(got - want).max())
                excess = diff / TOL_F32 if dtype == "float32" else bf16_excess(got, want, twin[rid][i], record=True)
                worst = max(worst, excess)
                largest = max(largest, diff if dtype == "float32" else diff / float(np.std(want)))
                if dtype == "float32":
                    assert diff <= TOL_F32, f"{size} {rid}@{pos}: |d| = {diff:.3e}"
                    top = np.sort(want)[-2:]
                    assert int(got.argmax()) == int(want.argmax()) or top[1] - top[0] < 2 * TOL_F32, f"{size} {rid}@{pos}: argmax"
                else:
                    assert excess <= 1.0, f"{size} {rid}@{pos}: {excess:.2f} of the bfloat16 bound (largest |d| = {diff:.3e})"
        print(f"[real sizes] {size} x {LAYERS} layers (of {SIZES[size]['layers_of_config']}) {dtype}: "
              f"largest |d| = {largest:.2e}" + ("" if dtype == "float32" else " of the row's spread")
              + f", {worst:.2f} of the bound; plain {t_plain:.0f} s, total {time.time() - t0:.0f} s")
        del r
        torch.cuda.empty_cache()


def test_block_enqueued_by_one_call_chooses_the_kernels_of_the_parts_at_real_widths():
    """The library's one-call block (csrc/block_runner.cu) restates the choice of kernels by row count
    that ops.py makes; only real widths reach every branch of it (K slices left to the consumer need
    K >= 1,024, the few-rows product a weight that it does not cut).  At the 1.5B layer sizes (a small
    vocabulary: every row's logits are compared) whole prompts on both sides of every row threshold,
    requests decoding together (attention merged into the output projection) and decoded tokens
    beside prompt portions give the same bits either way."""
    from coheryn_ai_studio_b200 import ops
    from coheryn_ai_studio_b200.config import Qwen2Config
    from coheryn_ai_studio_b200.engine import Engine, StepEntry, random_model_on_device
    from coheryn_ai_studio_b200.parts import native_block
    sizes = dict(SIZES["1.5b"], vocab_size=2048)
    sizes.pop("layers_of_config")
    cfg = Qwen2Config(num_hidden_layers=LAYERS, max_position_embeddings=32768, rope_theta=1e6, **sizes)
    model = random_model_on_device(cfg, SEED)
    V = cfg.vocab_size

    def run(native):
        ops.set_native_block(native)
        try:
            eng = Engine(model, context=4096, max_num_seqs=8, kv_cache_tokens=8 * 4200, prefix_reuse=False, use_graphs=False)
            rng = np.random.default_rng(7)
            before, outs = native_block.runs, []
            for T in (1, 8, 16, 17, 32, 33, 64, 65, 128, 129, 256, 257, 512, 2048):
                eng.cache.admit(f"w{T}")
                want = list(range(T)) if T <= 256 else [T - 1]
                outs.append((f"whole {T}", eng.runner.step([StepEntry(f"w{T}", rng.integers(0, V, T).tolist(), want)]).clone()))
                eng.cache.free(f"w{T}")
            for i, n in enumerate((300, 17, 1000, 64)):
                eng.cache.admit(f"r{i}")
                outs.append((f"prompt {i}", eng.runner.step([StepEntry(f"r{i}", rng.integers(0, V, n).tolist(), [n - 1])]).clone()))
            for s in range(2):
                outs.append((f"decode {s}", eng.runner.step([StepEntry(f"r{i}", [int(rng.integers(0, V))], [0])
                                                             for i in range(4)]).clone()))
            eng.cache.admit("m")
            outs.append(("mixed", eng.runner.step([StepEntry("r0", [5], [0]), StepEntry("m", rng.integers(0, V, 40).tolist(), list(range(40))),
                                                   StepEntry("r2", [9], [0])]).clone()))
            eng.runner.check_status()
            return outs, native_block.runs - before
        finally:
            ops.set_native_block(True)

    parts, none = run(False)
    whole, some = run(True)
    assert none == 0 and some >= len(whole) * (LAYERS - 1)
    for (name, a), (_, b) in zip(parts, whole):
        assert torch.isfinite(b).all() and torch.equal(a, b), name
