"""Replay on the GPU: the same requests whole, with the last 32 tokens one by one, in
portions of changing size, and mixed with other requests under a pool so small that pages
are used again; in float32 and in bfloat16; against the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import tiny
from replay import Replay, bf16_excess, compare, plain_logits, tol_bf16_spread

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]
# The two tiny configurations with the baseline's deviations, and again with louder weights: logits
# of a wider spread, on which a wrong key or page moves a row by a larger share of the bound.
NAMES = ["A", "B", "A_loud", "B_loud"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("models")
    return {n: tiny.make_folder(base, n) for n in NAMES}


@pytest.fixture(scope="module")
def models(folders):
    from coheryn_ai_studio_b200.engine import load_model
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            cache[(name, dtype)] = load_model(folders[name], dtype)[1]
        return cache[(name, dtype)]
    return get


def vocab(name):
    return tiny.CONFIGS[name][0].vocab_size


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole(name, dtype, folders, models):
    lengths = [5, 17, 33, 100] if name.startswith("A") else [1, 9, 64, 130, 200]
    for i, n in enumerate(lengths):
        seq = tiny.prompt(10 + i, n, vocab(name))
        r = Replay(folders[name], dtype, max_tokens=256, model=models(name, dtype))
        r.step([("r", seq, list(range(n)))], end=["r"])
        compare(r, folders[name], {"r": seq}, f"whole {n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_one_by_one(name, dtype, folders, models):
    n = 90 if name.startswith("A") else 150
    seq = tiny.prompt(20, n, vocab(name))
    r = Replay(folders[name], dtype, max_tokens=192, model=models(name, dtype))
    head = n - 32
    r.step([("r", seq[:head], list(range(head)))])
    for t in range(head, n):
        r.step([("r", [seq[t]], [0])])
    assert len(r.rows) == n
    compare(r, folders[name], {"r": seq}, "tail")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_changing_portions(name, dtype, folders, models):
    portions = [7, 2, 16, 3, 2, 33, 1, 15, 2, 17, 2, 5]
    n = sum(portions)
    seq = tiny.prompt(21, n, vocab(name))
    r = Replay(folders[name], dtype, max_tokens=128, model=models(name, dtype))
    o = 0
    for p in portions:
        r.step([("r", seq[o:o + p], list(range(p)))])
        o += p
    compare(r, folders[name], {"r": seq}, "portions")


def mixed_script(rng, sequences, max_live, max_portion):
    """Steps that keep up to ``max_live`` requests alive: each step gives every live
    request either a portion of its prompt (2..max_portion tokens) or, once past 60 % of
    its tokens, a single token; some requests sit a step out."""
    pending = list(sequences)
    live, done_at = {}, {}
    steps = []
    while pending or live:
        while pending and len(live) < max_live:
            live[pending.pop(0)] = 0
        entries, end = [], []
        for rid in list(live):
            seq, o = sequences[rid], live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue                                   # left out of this step
            left = len(seq) - o
            n = 1 if o >= 0.6 * len(seq) else int(min(left, rng.integers(2, max_portion + 1)))
            want = sorted(set(rng.integers(0, n, size=min(n, 3)).tolist() + [n - 1]))
            entries.append((rid, seq[o:o + n], want))
            live[rid] = o + n
            if live[rid] == len(seq):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append((entries, end))
    return steps


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_with_page_reuse(name, dtype, folders, models):
    rng = np.random.default_rng(5)
    lengths = [60, 33, 64, 47, 62, 21, 58, 64, 40, 9]
    sequences = {f"q{i}": tiny.prompt(30 + i, n, vocab(name)) for i, n in enumerate(lengths)}
    # four live requests of at most 64 tokens: 256 tokens = 16 pages of 16
    r = Replay(folders[name], dtype, max_tokens=256, model=models(name, dtype))
    steps = mixed_script(rng, sequences, max_live=4, max_portion=19)
    first_owner, reused = {}, 0
    for entries, end in steps:
        assert len(entries) <= 4
        r.step(entries, end)
        for rid, _, _ in entries:
            if rid in r.cache.requests:
                for p in r.cache.block_table(rid, 0):
                    if first_owner.setdefault(p, rid) != rid:
                        reused += 1
    assert any(len(e) > 1 and min(len(t) for _, t, _ in e) == 1 and max(len(t) for _, t, _ in e) > 1
               for e, _ in steps), "no step mixed a prompt portion with a single token"
    assert reused > 0, "the pool was never short enough to use a page again"
    assert r.cache.available_pages() == [16]
    compare(r, folders[name], sequences, "mixed")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype, folders, models):
    name = "B"
    n = 300
    seq = tiny.prompt(40, n, vocab(name))
    r = Replay(folders[name], dtype, max_tokens=320, model=models(name, dtype))
    r.step([("r", seq[:8], [7])])
    for t in range(8, n):
        r.step([("r", [seq[t]], [0] if t % 7 == 0 or t > n - 5 else [])])
    compare(r, folders[name], {"r": seq}, "long")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_first_tokens(name, dtype, folders, models):
    seq = tiny.prompt(41, 4, vocab(name))
    r = Replay(folders[name], dtype, max_tokens=64, model=models(name, dtype))
    for t in range(4):
        r.step([("r", [seq[t]], [0])])
    compare(r, folders[name], {"r": seq}, "first")
    r2 = Replay(folders[name], dtype, max_tokens=64, model=models(name, dtype))
    r2.step([("r", seq[:2], [0, 1])])
    r2.step([("r", seq[2:], [0, 1])])
    compare(r2, folders[name], {"r": seq}, "first pairs")


@pytest.mark.parametrize("dtype", DTYPES)
def test_cutting_agrees_with_itself(dtype, folders, models):
    """Beyond the comparison with the plain implementation: two ways of cutting the same
    sequence agree with each other to rounding."""
    name = "A"
    seq = tiny.prompt(42, 70, vocab(name))
    a = Replay(folders[name], dtype, max_tokens=128, model=models(name, dtype))
    a.step([("r", seq, list(range(70)))])
    b = Replay(folders[name], dtype, max_tokens=128, model=models(name, dtype))
    for o in range(0, 70, 5):
        b.step([("r", seq[o:o + 5], list(range(5)))])
    for k in a.rows:
        bound = 2e-5 if dtype == "float32" else 2 * tol_bf16_spread(a.rows[k])
        assert float(np.abs(a.rows[k] - b.rows[k]).max()) <= bound, k


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program(dtype, folders, tmp_path):
    """bin/trace_run as a user runs it: JSON lines in, <step>.f32 files and 'done' lines out."""
    name = "A"
    seqs = {"a": tiny.prompt(50, 37, vocab(name)), "b": tiny.prompt(51, 20, vocab(name))}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": seqs["a"][:30], "want": [0, 29]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": seqs["a"][30:32], "want": [1]},
                                {"id": "b", "tokens": seqs["b"][:18], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": seqs["b"][18:], "want": [0, 1]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": seqs["a"][32:], "want": [4]}], "end": ["a"]},
    ]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders[name],
                        "--dtype", dtype, "--out", str(out), "--max-tokens", "128"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", text=True,
                       capture_output=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    assert sorted(f.name for f in out.iterdir()) == ["0.f32", "1.f32", "2.f32", "3.f32"]      # and nothing else
    V = vocab(name)
    got = {i: np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V) for i in (0, 1, 2, 3)}
    ref_a, ref_b = plain_logits(folders[name], seqs["a"]), plain_logits(folders[name], seqs["b"])
    rnd_a, rnd_b = plain_logits(folders[name], seqs["a"], True), plain_logits(folders[name], seqs["b"], True)
    assert got[0].shape[0] == 2 and got[1].shape[0] == 1 and got[2].shape[0] == 2 and got[3].shape[0] == 1
    for rows, ref, rnd in ((got[0], ref_a[[0, 29]], rnd_a[[0, 29]]), (got[1], ref_a[[31]], rnd_a[[31]]),
                           (got[2], ref_b[[18, 19]], rnd_b[[18, 19]]), (got[3], ref_a[[36]], rnd_a[[36]])):
        for row, want, twin in zip(rows, ref, rnd):
            assert np.abs(row - want).max() <= 1e-4 if dtype == "float32" else bf16_excess(row, want, twin, record=True) <= 1.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_few_wanted_rows_take_the_last_layers_shortcut(name, dtype, folders, models):
    """Steps that want few rows (or none) run the last layer for those rows only: the logits
    equal the plain implementation's, the cache that later steps read is complete, and
    switching the shortcut off changes nothing beyond rounding."""
    n = 77 if name.startswith("A") else 131
    seq = tiny.prompt(33, n, vocab(name))
    other = tiny.prompt(34, 40, vocab(name))
    runs = {}
    for shortcut in (True, False):
        r = Replay(folders[name], dtype, max_tokens=256, model=models(name, dtype))
        r.runner.tail_shortcut = shortcut
        r.step([("r", seq[:30], [])])                                   # nothing wanted
        r.step([("r", seq[30:60], [29, 3]), ("o", other[:20], [19])])    # few rows, out of order, two requests
        r.step([("r", seq[60:n - 5], [0]), ("o", other[20:], [])])
        r.step([("r", seq[n - 5:], list(range(5)))])                     # everything wanted: no shortcut
        assert set(k for k in r.rows if k[0] == "r") == {("r", p) for p in [59, 33, 60] + list(range(n - 5, n))}
        compare(r, folders[name], {"r": seq, "o": other}, f"shortcut {shortcut}")
        runs[shortcut] = r.rows
    for key, row in runs[True].items():
        tol = 1e-4 if dtype == "float32" else 2 * tol_bf16_spread(row)
        assert np.abs(row - runs[False][key]).max() <= tol, key


ODD = {
    "mha": dict(vocab_size=517, hidden_size=80, intermediate_size=136, num_hidden_layers=1, num_attention_heads=5,
                num_key_value_heads=5, head_dim=16, tie_word_embeddings=True),
    "group16": dict(vocab_size=640, hidden_size=256, intermediate_size=520, num_hidden_layers=2, num_attention_heads=16,
                    num_key_value_heads=1, head_dim=16, tie_word_embeddings=False),
    "group32": dict(vocab_size=333, hidden_size=512, intermediate_size=264, num_hidden_layers=1, num_attention_heads=32,
                    num_key_value_heads=1, head_dim=16, tie_word_embeddings=True),
    "width100": dict(vocab_size=211, hidden_size=100, intermediate_size=150, num_hidden_layers=1, num_attention_heads=5,
                     num_key_value_heads=1, head_dim=32, tie_word_embeddings=True),
    "head128": dict(vocab_size=300, hidden_size=256, intermediate_size=344, num_hidden_layers=2, num_attention_heads=2,
                    num_key_value_heads=1, head_dim=128, tie_word_embeddings=True),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ODD))
def test_other_shapes_of_the_architecture(name, dtype, tmp_path):
    """Further shapes of the same architecture: no grouping, groups of 16 and 32 heads (more rows per
    kv head than the decode kernel takes), a width that is no multiple of 8 (no tensor-core product
    takes it), a head size unequal to width / heads, odd vocabularies; portions, mixed steps and
    decoding of three requests against the plain implementation."""
    from coheryn_ai_studio_b200.config import Qwen2Config
    from coheryn_ai_studio_b200.engine import write_random_model
    cfg = Qwen2Config(max_position_embeddings=256, rms_norm_eps=1e-5, rope_theta=1e5, **ODD[name])
    folder = str(tmp_path / name)
    write_random_model(folder, cfg, 3, tiny.POLICY_LOUD)
    V = cfg.vocab_size
    a, b, c = tiny.prompt(1, 90, V), tiny.prompt(2, 50, V), tiny.prompt(3, 30, V)
    r = Replay(folder, dtype, max_tokens=192)
    r.step([("a", a[:60], list(range(60)))])
    r.step([("a", a[60:63], [0, 1, 2]), ("b", b[:33], list(range(33)))])
    r.step([("a", a[63:70], list(range(7))), ("b", b[33:35], [0, 1]), ("c", c[:17], [16])])
    for t in range(70, 90):
        entries = [("a", [a[t]], [0])]
        if 35 + t - 70 < 50:
            entries.append(("b", [b[35 + t - 70]], [0]))
        if t == 72:
            entries.append(("c", c[17:], list(range(13))))
        r.step(entries)
    compare(r, folder, {"a": a, "b": b, "c": c}, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A_loud", "B"])
def test_shared_prefix_pages_are_mapped_and_used_again(name, dtype, folders, models):
    """A second request whose prompt starts like the first one's maps the first one's full pages
    from the page hash table instead of computing them (never the page with its last token);
    when both have gone the pages return and a third request, with another prompt, takes them.
    Every row equals the plain implementation's of the request's whole sequence."""
    V = vocab(name)
    shared = tiny.prompt(60, 52, V)
    a = shared + tiny.prompt(61, 9, V)
    b = shared + tiny.prompt(62, 14, V)
    c = tiny.prompt(63, 70, V)
    r = Replay(folders[name], dtype, max_tokens=160, model=models(name, dtype), prefix_reuse=True)   # 10 pages of 16
    r.step([("a", a[:40], [0, 39])])
    r.step([("a", a[40:], list(range(len(a) - 40)))])
    got = r.admit("b", b)
    assert got == 48                                          # three full pages of the shared 52 tokens
    assert r.cache.block_table("b", 0)[:3] == r.cache.block_table("a", 0)[:3]
    r.step([("b", b[got:got + 7], list(range(7))), ("a", [a[-1]], [])])      # a decodes nothing new: one more token
    r.step([("b", b[got + 7:], list(range(len(b) - got - 7)))], end=["a"])
    r.step([("b", [5], [0])], end=["b"])
    b_full = b + [5]
    assert r.cache.available_pages() == [10]
    # c needs 5 pages; the pool holds 10, of which the idle hashed ones are wiped last-recently-used first
    r.step([("c", c[:33], [32])])
    r.step([("c", c[33:], list(range(37)))])
    assert r.admit("d", b[:60]) == 48                         # b's prompt again: its idle pages are found by their hashes
    r.step([("d", b[48:60], [0, 11])], end=["d", "c"])
    assert r.cache.available_pages() == [10]
    compare(r, folders[name], {"a": a + [a[-1]], "b": b_full, "c": c, "d": b[:60]}, "prefix")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B_loud"])
def test_layer_outputs_equal_the_plain_layers(name, dtype, folders, models):
    """Every layer's output, as a trace hands it out, against the plain implementation's layer by
    layer: a wrong layer shows where it is, not only in the logits."""
    import plain_qwen2 as plain
    V = vocab(name)
    seq = tiny.prompt(70, 45, V)
    r = Replay(folders[name], dtype, max_tokens=64, model=models(name, dtype), layer_outputs=True)
    r.step([("r", seq[:30], [29])])                 # few rows wanted: with an observer the last layer still runs whole
    r.step([("r", seq[30:32], [0, 1])])
    for t in range(32, 45):
        r.step([("r", [seq[t]], [0])])
    cfg, w = plain.read_model(folders[name])
    layers, rounded = [], []
    plain.forward(cfg, w, seq, layer_outputs=layers)
    plain.forward(cfg, w, seq, layer_outputs=rounded, rounded=True)
    assert len(r.layers) == 45
    for (rid, pos), got in r.layers.items():
        assert got.shape == (cfg["num_hidden_layers"], cfg["hidden_size"])
        for i in range(cfg["num_hidden_layers"]):
            want = layers[i][pos]
            if dtype == "float32":
                bound = 1e-5 * max(1.0, float(np.abs(want).max()))
            else:
                bound = max(0.02 * float(np.std(want)), 2.0 * float(np.abs(rounded[i][pos] - want).max()))
            assert np.abs(got[i] - want).max() <= bound, (pos, i)
    compare(r, folders[name], {"r": seq}, "layers")
