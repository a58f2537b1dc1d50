"""The ``coheryn`` command line, in the manner of the reference's
(crates/coheryn-cli/src/main.rs:17-190, crates/coheryn-cli/src/daemon.rs:264-339).

    coheryn run MODEL --prompt TEXT | --tokens 1,2,3 [--max-tokens 128] [--context 4096]
                [--stream] [--temperature 0] [--top-k 0] [--top-p 1] [--seed 0]
                [--stop-token ID]... [--repetition-penalty 1] [--frequency-penalty 0]
                [--presence-penalty 0] [--dtype bfloat16|float32] [--json]
    coheryn trace MODEL --tokens 1,2,3          teacher-forced layer outputs and logits as JSON Lines
    coheryn init DIR|FILE.gguf --config CONFIG.json --seed N [--store bfloat16|float32]
    coheryn models inspect MODEL

Options carry the reference's names, defaults and meanings.  ``MODEL`` is a folder with
config.json and safetensors weights.  ``--tokens`` (the reference has it on ``trace``) is
accepted by ``run`` as well and bypasses the tokenizer; ``--prompt`` needs a
``tokenizer.json`` in the model folder and the ``tokenizers`` package.  With ``--json`` the
result goes to standard output as one JSON object and errors to standard error as JSON;
exit codes follow main.rs:545-575 (2 invalid request, 3 I/O, 5 resources, 1 internal).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional


class CliError(Exception):
    def __init__(self, code: str, message: str, exit_code: int):
        super().__init__(message)
        self.code, self.exit_code = code, exit_code


def _tokens(text: str) -> List[int]:
    try:
        return [int(t) for t in text.split(",") if t.strip() != ""]
    except ValueError:
        raise CliError("invalid_request", "--tokens takes comma-separated token ids", 2) from None


def _tokenizer(model_dir: str):
    path = os.path.join(model_dir, "tokenizer.json")
    if not os.path.isfile(path):
        raise CliError("invalid_request", f"{model_dir} has no tokenizer.json: pass --tokens instead "
                       "of --prompt", 2)
    try:
        from tokenizers import Tokenizer
    except ImportError:
        raise CliError("invalid_request", "the 'tokenizers' package is not installed: pass --tokens", 2) from None
    return Tokenizer.from_file(path)


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="coheryn", description="B200 inference engine")
    ap.add_argument("--json", action="store_true", help="machine-readable result and errors")
    sub = ap.add_subparsers(dest="command", required=True)

    run = sub.add_parser("run", help="generate from a prompt")
    run.add_argument("model")
    run.add_argument("--prompt")
    run.add_argument("--tokens", help="comma-separated prompt token ids (bypasses the tokenizer)")
    run.add_argument("--stream", action="store_true")
    run.add_argument("--max-tokens", type=int, default=128)
    run.add_argument("--context", type=int, default=4096)
    run.add_argument("--temperature", type=float, default=0.0)
    run.add_argument("--top-k", type=int, default=0)
    run.add_argument("--top-p", type=float, default=1.0)
    run.add_argument("--seed", type=int, default=0)
    run.add_argument("--stop-token", type=int, action="append", default=[], dest="stop_tokens")
    run.add_argument("--repetition-penalty", type=float, default=1.0)
    run.add_argument("--frequency-penalty", type=float, default=0.0)
    run.add_argument("--presence-penalty", type=float, default=0.0)
    run.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    run.add_argument("--page-size", type=int, default=16)
    run.add_argument("--max-batched-tokens", type=int, default=2048)
    run.add_argument("--device", default="cuda:0")

    tr = sub.add_parser("trace", help="teacher-forced logits as JSON Lines")
    tr.add_argument("model")
    tr.add_argument("--prompt")
    tr.add_argument("--tokens")
    tr.add_argument("--context", type=int, default=4096)
    tr.add_argument("--dtype", default="float32", choices=["bfloat16", "float32"])
    tr.add_argument("--device", default="cuda:0")
    tr.add_argument("--logits-only", action="store_true", help="leave the layer outputs out")

    init = sub.add_parser("init", help="write a model folder (or one .gguf file) with seeded random weights")
    init.add_argument("dir")
    init.add_argument("--config", required=True, help="a config.json to take the sizes from")
    init.add_argument("--seed", type=int, default=0)
    init.add_argument("--store", default="bfloat16", choices=["bfloat16", "float32"])
    init.add_argument("--matrix-std", type=float, default=0.02)
    init.add_argument("--bias-std", type=float, default=0.02)
    init.add_argument("--norm-jitter", type=float, default=0.0)

    models = sub.add_parser("models", help="model folder utilities")
    msub = models.add_subparsers(dest="models_command", required=True)
    ins = msub.add_parser("inspect", help="configuration and tensor inventory, without loading")
    ins.add_argument("model")
    return ap


def _prompt_ids(args, model_dir: str):
    if (args.prompt is None) == (args.tokens is None):
        raise CliError("invalid_request", "exactly one of --prompt and --tokens is required", 2)
    if args.tokens is not None:
        return _tokens(args.tokens), None
    tok = _tokenizer(model_dir)
    return tok.encode(args.prompt).ids, tok


def cmd_run(args) -> int:
    from .engine import Engine, RequestRefused
    from .sampling import SamplingParams
    if args.stream and args.json:
        raise CliError("invalid_request", "--stream conflicts with --json", 2)
    ids, tok = _prompt_ids(args, args.model)
    params = SamplingParams(args.temperature, args.top_k, args.top_p, args.seed, args.repetition_penalty,
                            args.frequency_penalty, args.presence_penalty)
    try:
        params.validate()
        engine = Engine.from_folder(args.model, args.dtype, args.device, context=args.context,
                                    max_num_seqs=1, max_num_batched_tokens=args.max_batched_tokens,
                                    page_size=args.page_size, kv_cache_tokens=args.context)
    except (ValueError, RequestRefused) as e:
        raise CliError("invalid_request", str(e), 2) from None
    streamed: List[int] = []

    def on_token(_, token):
        if not args.stream:
            return
        if tok is not None:
            streamed.append(token)
            text = tok.decode(streamed)
            if not text.endswith("�"):
                sys.stdout.write(text); sys.stdout.flush(); streamed.clear()
        else:
            sys.stdout.write(f"{token} "); sys.stdout.flush()
    try:
        result = engine.generate([ids], args.max_tokens, params, args.stop_tokens, on_token)[0]
    except RequestRefused as e:
        raise CliError("invalid_request", str(e), 2) from None
    stops = set(args.stop_tokens) | set(engine.eos_token_ids)
    visible = [t for t in result.token_ids if t not in stops]     # an end token yields no text
    result.text = tok.decode(visible) if tok is not None else ""
    if args.json:
        print(json.dumps(result.to_dict()))
    elif args.stream:
        print()
    else:
        print(result.text if tok is not None else ",".join(str(t) for t in result.token_ids))
    return 0


def cmd_trace(args) -> int:
    """Teacher-forced, token by token; per position one JSON line for every layer's output
    ({"position", "name": "blk.<i>.output", "values"}, i counting the executions of the schedule) and one
    for the logits ({"position", "name": "logits", "values"}), as crates/coheryn-engine/src/inference.rs:
    541-556 hands them to its observer and crates/coheryn-cli/src/main.rs:487-506 prints them."""
    from .engine import Engine
    ids, _ = _prompt_ids(args, args.model)
    if not ids:
        raise CliError("invalid_request", "trace needs at least one token", 2)
    engine = Engine.from_folder(args.model, args.dtype, args.device, context=args.context, max_num_seqs=1,
                                kv_cache_tokens=args.context, prefix_reuse=False, use_graphs=False)
    from .engine import StepEntry
    engine.cache.admit("trace")
    outputs = []
    if not args.logits_only:
        engine.model.layer_observer = lambda entry, x: outputs.append((entry, x))
    for position, token in enumerate(ids):
        outputs.clear()
        logits = engine.runner.step([StepEntry("trace", [token], [0])])
        engine.runner.check_status()
        for entry, x in outputs:
            print(json.dumps({"position": position, "name": f"blk.{entry}.output", "values": x[0].cpu().tolist()}))
        print(json.dumps({"position": position, "name": "logits", "values": logits[0].cpu().tolist()}))
    return 0


def cmd_init(args) -> int:
    import torch
    from .config import architecture_for, read_config_json
    from .engine import write_random_gguf, write_random_model
    from .weights import InitPolicy
    obj = read_config_json(args.config)
    config = architecture_for(obj).parse_config(obj)
    write = write_random_gguf if args.dir.lower().endswith(".gguf") else write_random_model
    write(args.dir, config, args.seed, InitPolicy(args.matrix_std, args.bias_std, args.norm_jitter),
          store=torch.bfloat16 if args.store == "bfloat16" else torch.float32)
    print(args.dir)
    return 0


def cmd_inspect(args) -> int:
    """What the adapter says of the model (capabilities, configuration, cache cost) and the
    tensor inventory of the files, checked against what the model needs; no payload is read."""
    import torch
    from .config import describe_model, load_config
    from .parts import DecoderModel, Runtime
    from .engine.loading import gguf_rename
    from .weights import check_against, index_model
    _, spec = load_config(args.model)
    entries = index_model(args.model, gguf_rename(args.model))
    model = DecoderModel(spec, Runtime(torch.bfloat16, torch.device("cpu")))
    check_against(model.tensor_specs(), entries)
    report = describe_model(args.model)
    report["files"] = {
        "tensors": len(entries), "tensor_bytes": sum(e.end - e.begin for e in entries.values()),
        "dtypes": sorted({str(e.dtype).replace("torch.", "") for e in entries.values()})}
    print(json.dumps(report, indent=1))
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    ap = build_parser()
    args = ap.parse_args(argv)
    try:
        if args.command == "run":
            return cmd_run(args)
        if args.command == "trace":
            return cmd_trace(args)
        if args.command == "init":
            return cmd_init(args)
        if args.command == "models":
            return cmd_inspect(args)
        raise CliError("invalid_request", f"unknown command {args.command}", 2)
    except CliError as e:
        err, code = {"code": e.code, "message": str(e)}, e.exit_code
    except FileNotFoundError as e:
        err, code = {"code": "io", "message": str(e)}, 3
    except ValueError as e:       # configuration, weights, request validation
        err, code = {"code": "invalid_model", "message": str(e)}, 4
    except MemoryError as e:
        err, code = {"code": "resource_exhausted", "message": str(e)}, 5
    except KeyboardInterrupt:
        err, code = {"code": "cancelled", "message": "interrupted"}, 130
    except RuntimeError as e:     # no GPU, kernels not built, a device fault
        from .ops import KernelError
        unavailable = isinstance(e, KernelError)
        err, code = {"code": "unavailable" if unavailable else "internal", "message": str(e)}, 8 if unavailable else 1
    if args.json:
        print(json.dumps(err), file=sys.stderr)
    else:
        print(f"{err['code']}: {err['message']}", file=sys.stderr)
    return code


if __name__ == "__main__":
    sys.exit(main())
