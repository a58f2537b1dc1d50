#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode throughput at the layer sizes of
Qwen2.5-1.5B (random bfloat16 weights, batch 8, context 4,096), plus prefill of a
2,048-token prompt, decode at batch 1 and 64, and the achieved fraction of the roofline.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  ``value`` is decoded tokens per second
from CUDA events around K back-to-back decode steps (inputs of every step copied from
pinned host memory, no host synchronisation inside the timed region).  ``e2e`` is the
same workload through ``Engine.step()``, the call a user makes: host token ids in, host
token ids out, every step.

The cache of the timed requests is filled with random keys and values (their prompts are
not run); weights and caches are far larger than the 126 MB L2, so every step streams
them from HBM.  One JSON line is printed.

``--workload serving-7b`` and ``--workload long-14b`` run the two further workloads that the
baseline names instead (their own JSON line, through ``Engine.generate``): continuous
batching of 64 requests at the 7B layer sizes (prompts uniform in [128, 2048], 256 output
tokens each, context 8,192, pages of 16), and a 16,384-token context at the 14B layer sizes
whose prefix 8 requests share (prefill in 2,048-token portions, prefix pages reused), then
decoding at batch 8.  ``--workload chat-1.5b`` is this repository's own: 256 short requests at the
1.5B layer sizes (prompts uniform in [16, 256], 16 to 128 output tokens each, at most 32 running), so
that requests end and begin all the time and many steps carry a new prompt beside decoded tokens,
which no graph replays: it measures what such steps cost the host.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# The headline configuration: Qwen2.5-1.5B layer sizes.
SIZES = dict(vocab_size=151936, hidden_size=1536, intermediate_size=8960, num_hidden_layers=28,
             num_attention_heads=12, num_key_value_heads=2, head_dim=128,
             max_position_embeddings=32768, rms_norm_eps=1e-6, rope_theta=1e6,
             tie_word_embeddings=True)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
# The two further workloads: Qwen2.5-7B and 14B layer sizes.
SIZES_7B = dict(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
                num_attention_heads=28, num_key_value_heads=4, head_dim=128, max_position_embeddings=32768,
                rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
SIZES_14B = dict(vocab_size=152064, hidden_size=5120, intermediate_size=13824, num_hidden_layers=48,
                 num_attention_heads=40, num_key_value_heads=8, head_dim=128, max_position_embeddings=32768,
                 rms_norm_eps=1e-5, rope_theta=1e6, tie_word_embeddings=False)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    src = "fallback"
    p = dict(FALLBACK_PEAKS)
    if os.path.isfile(path):
        try:
            obj = json.load(open(path))
            flat = {}

            def walk(o):
                if isinstance(o, dict):
                    for k, v in o.items():
                        if isinstance(v, (int, float)) and not isinstance(v, bool):
                            flat.setdefault(k, float(v))
                        else:
                            walk(v)
            walk(obj)
            if "hbm_gbs" in flat:
                p["hbm_gbs"] = flat["hbm_gbs"]
            if "bf16_tflops" in flat:
                p["bf16_tflops"] = flat["bf16_tflops"]
            if "bf16_tflops_sustained" in flat:
                p["bf16_tflops_sustained"] = flat["bf16_tflops_sustained"]
            src = "measured"
        except Exception:
            pass
    p["source"] = src
    return p


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def window(self, t0, t1):
        rows = [l.split(", ") for t, l in self.lines if t0 <= t <= t1 + 0.15 and l]
        if not rows:
            rows = [l.split(", ") for _, l in self.lines[-3:] if l]
        return rows

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=3)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    @staticmethod
    def summary(rows):
        mhz, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                mhz.append(int(r[0])); mx = max(mx, int(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[2:6]):
                if v.strip().lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def other_workload(args) -> int:
    """configs[3] (serving-7b) or configs[4] (long-14b) of the baseline through Engine.generate, or the
    short-request workload of this repository (chat-1.5b) through Engine.add_request / step."""
    import numpy as np
    import torch

    from coheryn_ai_studio_b200.config import Qwen2Config
    from coheryn_ai_studio_b200.engine import Engine, random_model_on_device
    serving = args.workload == "serving-7b"
    chat = args.workload == "chat-1.5b"
    sizes = dict(SIZES if chat else SIZES_7B if serving else SIZES_14B)
    full_layers = sizes["num_hidden_layers"]
    if args.layers != SIZES["num_hidden_layers"]:
        sizes["num_hidden_layers"] = args.layers
    cfg = Qwen2Config(**sizes)
    model = random_model_on_device(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    rng = np.random.default_rng(0)
    V = cfg.vocab_size
    if chat:
        eng = Engine(model, context=1024, max_num_seqs=32, max_num_batched_tokens=2048, page_size=16,
                     kv_cache_tokens=32 * 448, prefix_reuse=False, use_graphs=not args.no_graphs)
        prompts = [rng.integers(0, V, int(n)).tolist() for n in rng.integers(16, 257, 256)]
        outs = [int(n) for n in rng.integers(16, 129, 256)]

        def run_all():
            ids = [eng.add_request(p, n) for p, n in zip(prompts, outs)]
            steps = 0
            while eng.scheduler.has_work():
                eng.step()
                steps += 1
            return [eng.result(rid) for rid in ids], steps
        run_all()                                          # untimed: compilation, a graph per batch width met
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        res, steps = run_all()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        out_tokens = sum(r.completion_tokens for r in res)
        line = {"metric": "serving_output_tokens_per_s", "value": round(out_tokens / dt, 1), "unit": "tok/s",
                "seconds": round(dt, 3), "prompt_tokens": sum(len(p) for p in prompts), "output_tokens": out_tokens,
                "steps": steps, "ms_per_step": round(dt / steps * 1e3, 3),
                "preemptions": eng.scheduler.stats["preemptions"]}
        what = "Qwen2.5-1.5B layer sizes, 256 requests, prompts uniform[16,256], 16..128 outputs, 32 running, page 16"
    elif serving:
        eng = Engine(model, context=8192, max_num_seqs=64, max_num_batched_tokens=2048, page_size=16,
                     kv_cache_tokens=64 * 2400, prefix_reuse=False, use_graphs=not args.no_graphs)
        prompts = [rng.integers(0, V, int(n)).tolist() for n in rng.integers(128, 2049, 64)]
        outs = 256
        eng.generate(prompts, max_tokens=outs)             # untimed: compilation, a graph per batch width met
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        res = eng.generate(prompts, max_tokens=outs)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        out_tokens = sum(r.completion_tokens for r in res)
        line = {"metric": "serving_output_tokens_per_s", "value": round(out_tokens / dt, 1), "unit": "tok/s",
                "seconds": round(dt, 3), "prompt_tokens": sum(len(p) for p in prompts), "output_tokens": out_tokens,
                "total_tokens_per_s": round((sum(len(p) for p in prompts) + out_tokens) / dt, 1),
                "preemptions": eng.scheduler.stats["preemptions"]}
        what = "Qwen2.5-7B layer sizes, 64 requests, prompts uniform[128,2048], 256 outputs, context 8192, page 16"
    else:
        ctx, outs = 16384, 64
        eng = Engine(model, context=ctx + outs + 16, max_num_seqs=8, max_num_batched_tokens=2048, page_size=16,
                     kv_cache_tokens=3 * ctx, prefix_reuse=True, use_graphs=not args.no_graphs)
        warm = rng.integers(0, V, 2100).tolist()
        eng.generate([warm], max_tokens=4)                  # first-use compilation and graph capture
        shared = rng.integers(0, V, ctx - 256).tolist()
        prompts = [shared + rng.integers(0, V, 256).tolist() for _ in range(8)]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.generate(prompts[:1], max_tokens=1)             # the shared prefix is computed once
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        res = eng.generate(prompts, max_tokens=outs)
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        decode_s = max(r.decode_ms for r in res) / 1e3
        line = {"metric": "long_context_decode_tokens_per_s", "value": round(8 * (outs - 1) / decode_s, 1), "unit": "tok/s",
                "prefill_tokens_per_s": round(ctx / (t1 - t0), 1), "prefill_seconds": round(t1 - t0, 3),
                "shared_prefix_seconds": round(t2 - t1, 3),
                "reused_prompt_tokens": [r.reused_prompt_tokens for r in res]}
        what = "Qwen2.5-14B layer sizes, 16384-token context, prefix shared by 8 requests, decode at batch 8"
    eng.cache.check()
    line.update({"n_gpus": 1, "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "impl": "ours",
                 "config": {"model": what, "layers": cfg.num_hidden_layers, "layers_of_config": full_layers}})
    print(json.dumps(line))
    return 0


def timeline(args, make_engine, StepEntry, ops, torch) -> int:
    """Where a decode step's time goes, kernel by kernel, measured inside graph-replayed steps (the
    kernels overlap through programmatic dependent launch, so a kernel's own duration says little):
    ``advance`` is how far a kernel's end lies behind the end of everything before it; the advances
    add up to the step."""
    import collections
    from torch.profiler import ProfilerActivity, profile
    eng, lens, rng = make_engine(args.batch)
    ids = [f"t{i}" for i in range(args.batch)]
    for rid, n in zip(ids, lens):
        assert eng.cache.admit(rid) is not None and eng.cache.reserve(rid, [0] * n)
        eng.cache.commit(rid)
    out = torch.empty(args.batch, dtype=torch.int32, device="cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")

    def one():
        logits = eng.runner.step([StepEntry(rid, [5], [0]) for rid in ids])
        ops.argmax(logits, out, status)
    for _ in range(max(args.warmup, 4)):
        one()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(4):
            one()
        torch.cuda.synchronize()
    events = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
              and "emcpy" not in e.name and "emset" not in e.name]
    events.sort(key=lambda e: e.time_range.start)
    first = [i for i, e in enumerate(events) if "embed_gather" in e.name][-1]
    step = events[first:]
    t0 = prev_end = step[0].time_range.start
    rows = collections.OrderedDict()
    for e in step:
        start, end = e.time_range.start, e.time_range.end
        name = e.name.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0]
        r = rows.setdefault(name, [0, 0.0, 0.0])
        r[0] += 1
        r[1] += end - start
        r[2] += max(0.0, end - prev_end)
        prev_end = max(prev_end, end)
    print(f"decode step, batch {args.batch}, {args.layers} layers: {prev_end - t0:.1f} us from the first kernel's start to the last one's end")
    print(f"{'launches':>8} {'duration us':>12} {'advance us':>11} {'step share':>10}  kernel")
    for name, (n, dur, adv) in rows.items():
        print(f"{n:8d} {dur / n:12.2f} {adv / n:11.2f} {adv / (prev_end - t0):10.3f}  {name}")
    if args.timeline_raw:
        # every kernel of the step with its own start and end, relative to the step's start
        print(f"{'start us':>9} {'end us':>9}  kernel")
        for e in step:
            name = e.name.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0]
            print(f"{e.time_range.start - t0:9.1f} {e.time_range.end - t0:9.1f}  {name}")
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=SIZES["num_hidden_layers"],
                    help="fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--skip-points", action="store_true", help="skip the batch 1 / 64 points")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--workload", default="decode", choices=["decode", "serving-7b", "long-14b", "chat-1.5b"],
                    help="decode: the contract's line (default); the others: see the header")
    ap.add_argument("--timeline-raw", action="store_true", help="with --timeline: also every kernel's start and end")
    ap.add_argument("--timeline", action="store_true",
                    help="instead of the benchmark: the kernels of one graph-replayed decode step with their times "
                         "inside the step (CUPTI through torch.profiler), one text line per kernel")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace (no setup.py/pyproject.toml, pip reports "
                          "'not installable') and this image has no cargo/rustc; it is CPU-only"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.workload != "decode":
        return other_workload(args)

    import numpy as np
    import torch

    from coheryn_ai_studio_b200 import ops
    from coheryn_ai_studio_b200.config import Qwen2Config
    from coheryn_ai_studio_b200.engine import Engine, StepEntry, random_model_on_device
    from coheryn_ai_studio_b200.engine.scheduler import Request
    from coheryn_ai_studio_b200.sampling import RequestSampler, SamplingParams

    pk = peaks()
    sizes = dict(SIZES, num_hidden_layers=args.layers)
    cfg = Qwen2Config(**sizes)
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    model = random_model_on_device(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    V, H, I, L = cfg.vocab_size, cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers
    nh, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    layer_params = (nh + 2 * nkv) * hd * H + H * nh * hd + 3 * H * I
    weight_bytes = 2 * (L * layer_params + V * H) + 2 * L * ((nh + 2 * nkv) * hd + 2 * H) + 4 * H
    kv_bytes_per_token = 2 * L * nkv * hd * 2
    total_steps = args.warmup + args.steps

    sampler = ClockSampler()
    sampler.start()

    def make_engine(batch, context=None):
        margin = 2 * total_steps + 8
        context = context or args.context
        eng = Engine(model, dtype="bfloat16", context=context, max_num_seqs=batch,
                     max_num_batched_tokens=max(2048, args.prefill_tokens), page_size=args.page_size,
                     kv_cache_tokens=batch * (context + 64), prefix_reuse=False,
                     use_graphs=not args.no_graphs)
        for g in eng.cache.groups:
            g.tensor.normal_(0.0, 1.0)
        rng = np.random.default_rng(1234 + batch)
        lens = np.minimum(rng.integers(512, args.context + 1, size=batch), args.context - margin)
        return eng, [int(x) for x in lens], rng

    def inject(eng, lens, rng):
        """Requests that have 'run' their prompts: pages reserved and committed, contents
        random.  Returns the Request objects (already in the scheduler's running list)."""
        reqs = []
        for i, n in enumerate(lens):
            prompt = rng.integers(0, V, size=n).tolist()
            req = Request(f"bench-{i}", prompt, max_tokens=min(4 * total_steps + 64, args.context - n), params=SamplingParams())
            req.sampler = RequestSampler(req.params)
            req.arrival = i
            assert eng.cache.admit(req.request_id) is not None
            assert eng.cache.reserve(req.request_id, prompt[:-1])
            eng.cache.commit(req.request_id)
            eng.scheduler.adopt_running(req, n - 1)
            eng._requests[req.request_id] = req
            from coheryn_ai_studio_b200.engine.engine import _Timing
            eng._timing[req.request_id] = _Timing(time.perf_counter())
            reqs.append(req)
        return reqs

    def decode_device_timed(batch, steps, warmup):
        """K decode steps back to back, timed on the device."""
        eng, lens, rng = make_engine(batch)
        ids = [f"d{i}" for i in range(batch)]
        for rid, n in zip(ids, lens):
            assert eng.cache.admit(rid) is not None
            assert eng.cache.reserve(rid, [0] * n)
            eng.cache.commit(rid)
        out = torch.empty(batch, dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        toks = rng.integers(0, V, size=(warmup + steps, batch))

        def one(k):
            logits = eng.runner.step([StepEntry(rid, [int(toks[k, b])], [0]) for b, rid in enumerate(ids)])
            ops.argmax(logits, out, status)
        for k in range(warmup):
            one(k)
        torch.cuda.synchronize()
        l0 = ops.total_launch_count() + eng.runner.graph_launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record()
        for k in range(warmup, warmup + steps):
            one(k)
        e1.record()
        torch.cuda.synchronize()
        t1 = time.time()
        ms = e0.elapsed_time(e1)
        eng.runner.check_status()          # a kernel that gave up a wait would have timed garbage
        launches = ops.total_launch_count() + eng.runner.graph_launches - l0
        mean_ctx = float(np.mean(lens)) + warmup + steps / 2
        step_bytes = weight_bytes + batch * mean_ctx * kv_bytes_per_token
        del eng
        torch.cuda.empty_cache()
        return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "launches": launches,
                "bytes_per_step": step_bytes, "window": (t0, t1), "mean_ctx": mean_ctx}

    def decode_end_to_end(batch, steps, warmup):
        eng, lens, rng = make_engine(batch)
        inject(eng, lens, rng)
        for _ in range(warmup):
            eng.step()
        torch.cuda.synchronize()
        h2d = d2h = 0
        t0 = time.perf_counter()
        for _ in range(steps):
            events = eng.step()
            h2d += eng.runner.h2d_bytes
            d2h += 4 * len(events) + 8        # sampled ids and the two status words
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        del eng
        torch.cuda.empty_cache()
        return {"value": batch * steps / dt, "unit": "tok/s", "h2d_bytes_per_step": h2d // steps,
                "d2h_bytes_per_step": d2h // steps, "ms_per_step": dt / steps * 1e3}

    def prefill_timed(tokens, repeats=3):
        eng, _, rng = make_engine(1, max(args.context, tokens + 64))   # a context shorter than the prompt: room for it
        best = None
        for r in range(repeats + 1):            # the first run is the warm-up
            rid = f"p{r}"
            prompt = rng.integers(0, V, size=tokens).tolist()
            eng.cache.admit(rid)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.runner.step([StepEntry(rid, prompt, [tokens - 1])])
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            eng.runner.check_status()
            eng.cache.free(rid)
            if r > 0:
                best = ms if best is None else min(best, ms)
        # What the step computes: every layer in full but the last, which projects q/k/v for all
        # tokens (their keys and values go to the cache) and runs the rest for the one wanted row.
        full = 2.0 * tokens * layer_params + 4.0 * nh * hd * tokens * (tokens + 1) / 2
        last = (2.0 * tokens * (nh + 2 * nkv) * hd * H + 2.0 * (H * nh * hd + 3 * H * I) + 4.0 * nh * hd * tokens
                if eng.runner.tail_shortcut else full)
        flops = (L - 1) * full + last + 2.0 * V * H
        peak = pk.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]) * 1e12
        del eng
        torch.cuda.empty_cache()
        return {"value": tokens / (best / 1e3), "tokens": tokens, "ms": best, "frac": flops / (best / 1e3) / peak,
                "tflops": flops / (best / 1e3) / 1e12}

    if args.timeline:
        sampler.stop()
        return timeline(args, make_engine, StepEntry, ops, torch)

    main_run = decode_device_timed(args.batch, args.steps, args.warmup)
    clocks = ClockSampler.summary(sampler.window(*main_run["window"]))
    e2e = decode_end_to_end(args.batch, args.steps, args.warmup)
    prefill = prefill_timed(args.prefill_tokens)
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            r = decode_device_timed(b, max(16, args.steps // 2), args.warmup)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            points[f"decode_b{b}_hbm_frac"] = round(r["bytes_per_step"] / (r["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"], 4)
    sampler.stop()

    achieved = main_run["bytes_per_step"] / (main_run["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": "decode_tokens_per_s", "value": round(main_run["tok_s"], 1), "unit": "tok/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": "Qwen2.5-1.5B layer sizes, random weights", "global_batch": args.batch,
            "seq_len": args.context, "parallelism": "single-gpu", "layers": L,
            "layers_of_config": SIZES["num_hidden_layers"], "hidden": H, "heads": nh, "kv_heads": nkv,
            "head_dim": hd, "intermediate": I, "vocab": V, "tied_embeddings": True,
            "context_per_request": f"uniform[512,{args.context}]", "mean_context": round(main_run["mean_ctx"], 1),
            "page_size": args.page_size, "cuda_graphs": not args.no_graphs,
            "l2": "weights+cache per step exceed L2 (126 MB)", "peaks": pk["source"],
        },
        "e2e": {k: (round(v, 2) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": int(main_run["launches"]),
        "clocks": clocks,
        "prefill": {"value": round(prefill["value"], 1), "tokens": prefill["tokens"], "ms": round(prefill["ms"], 3),
                    "frac": round(prefill["frac"], 4), "tflops": round(prefill["tflops"], 1)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
