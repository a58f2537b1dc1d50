"""Trace replay: feed given token ids through a model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives the
same model, step function, cache manager and kernels that generation uses.  This is the
engine's counterpart of the reference's teacher-forced ``coheryn trace``
(crates/coheryn-cli/src/main.rs:62-71, crates/coheryn-engine/src/inference.rs:562-580),
extended to several live requests, to portions of prompts and to a bounded cache.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` receives the logits of the
wanted places (order of the entries, then of ``want``) as little-endian float32
``[wanted, vocab]``.  After each step a line ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page (any size)")
    ap.add_argument("--max-requests", type=int, default=8)
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    if args.max_tokens < 1:
        ap.error("--max-tokens must be positive")
    if args.page_size < 1:
        ap.error("--page-size must be positive")

    import torch

    from .cache.manager import CacheManager
    from .engine.loading import load_model, parse_dtype
    from .engine.step import StepEntry, StepRunner

    os.makedirs(args.out, exist_ok=True)
    _, model = load_model(args.model, args.dtype, args.device)
    # --max-tokens counts every live request rounded up to 64 tokens.  Pages that divide 64 hold
    # that exactly; with any other page size a request's last page may stick out of its rounded
    # count, so each request gets one page of slack.
    num_pages = -(-args.max_tokens // args.page_size)
    if 64 % args.page_size:
        num_pages += args.max_requests
    cache = CacheManager(model.cache_requirements(), [e.cache_from for e in model.spec.schedule],
                         parse_dtype(args.dtype), torch.device(args.device), page_size=args.page_size,
                         num_pages=num_pages, max_requests=args.max_requests, prefix_reuse=False)
    runner = StepRunner(model, cache)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        obj = json.loads(line)
        step = obj["step"]
        entries = []
        for e in obj.get("entries", []):
            rid = str(e["id"])
            if rid not in cache.requests:
                if cache.admit(rid) is None:
                    raise RuntimeError(f"more than {args.max_requests} live requests")
            entries.append(StepEntry(rid, e["tokens"], e.get("want", [])))
        if entries:
            logits = runner.step(entries)
            runner.check_status()
            if logits.shape[0]:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                tmp = os.path.join(args.out, f".{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
            else:
                torch.cuda.synchronize()
        for rid in obj.get("end", []):
            cache.free(str(rid))
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
