"""The Python entry point in the reference's manner: its scripts never link the engine,
they spawn the binary and parse ``--json`` output (tools/benchmark.py:24-27,
resources/reference-archive/tools/check_oracle.py.txt:15-19).  :func:`run` does the same
with this package's ``coheryn run``; :func:`generate` is the in-process equivalent.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from typing import Dict, List, Optional, Sequence

_BIN = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "coheryn")


def run(model: str, prompt: Optional[str] = None, tokens: Optional[Sequence[int]] = None,
        max_tokens: int = 128, context: int = 4096, temperature: float = 0.0, top_k: int = 0,
        top_p: float = 1.0, seed: int = 0, stop_tokens: Sequence[int] = (), dtype: str = "bfloat16",
        timeout: Optional[float] = None) -> Dict:
    """Spawn ``coheryn --json run MODEL ...`` and return its result object.  Raises
    RuntimeError carrying the program's JSON error on a non-zero exit."""
    cmd = [sys.executable, _BIN, "--json", "run", model, "--max-tokens", str(max_tokens), "--context",
           str(context), "--temperature", str(temperature), "--top-k", str(top_k), "--top-p", str(top_p),
           "--seed", str(seed), "--dtype", dtype]
    if prompt is not None:
        cmd += ["--prompt", prompt]
    if tokens is not None:
        cmd += ["--tokens", ",".join(str(int(t)) for t in tokens)]
    for t in stop_tokens:
        cmd += ["--stop-token", str(int(t))]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
    if p.returncode != 0:
        raise RuntimeError(f"coheryn run exited with {p.returncode}: {p.stderr.strip().splitlines()[-1:]}")
    return json.loads(p.stdout.strip().splitlines()[-1])


def generate(model: str, prompts: Sequence[Sequence[int]], max_tokens: int = 128, context: int = 4096,
             temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0,
             stop_tokens: Sequence[int] = (), dtype: str = "bfloat16", **engine_options) -> List[Dict]:
    """Load ``model`` in this process and generate for every prompt (token ids) with
    continuous batching; returns one result object per prompt."""
    from .engine import Engine
    from .sampling import SamplingParams
    engine = Engine.from_folder(model, dtype, context=context, **engine_options)
    params = SamplingParams(temperature, top_k, top_p, seed)
    return [r.to_dict() for r in engine.generate(prompts, max_tokens, params, stop_tokens)]
