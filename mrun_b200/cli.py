"""Command line in the manner of ``mrun run`` (crates/mrun/src/cli/run.rs:27-79) and of the
reference's token-ids-in example (crates/mrun-engine/examples/generate.rs:1-13).

    mrun run MODEL --prompt IDS [--max-tokens N] [--temperature T] [--top-p P] [--top-k K]
                   [--min-p P] [--seed S] [--stop IDS]... [--budget-gib GIB | --context TOKENS] [--info]
    mrun random MODEL_DIR --config CONFIG.json --seed S

``MODEL`` is a folder with config.json and safetensors.  ``--prompt`` takes token ids, inline or
as a file, separated by commas or whitespace; this engine has no tokenizer, so the text options
of ``mrun run`` (--system, --think, --mcp) do not exist here, and ``--stop`` (up to 4 times, as
there: crates/mrun/src/cli/run.rs:56, crates/mrun/src/chat/limits.rs:6) takes a stop sequence of
token ids instead of a string: the output ends before the first of them that appears.  The generated ids go to
standard output separated by commas; speeds go to standard error the way the example prints them.
Sampling defaults come from the model's generation_config.json, else temperature 0, top_p 1,
top_k 0, min_p 0 (crates/mrun/src/cli/model.rs:380-399).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import List, Optional


def parse_ids(text: str) -> List[int]:
    if os.path.exists(text):
        with open(text, "r", encoding="utf-8") as f:
            text = f.read()
    out = []
    for piece in text.replace(",", " ").split():
        try:
            out.append(int(piece))
        except ValueError:
            raise SystemExit(f"error: bad token id {piece!r}") from None
    return out


def parse_tokens(text: str) -> int:
    """``64K`` style token counts, as ``--context`` takes them."""
    text = text.strip()
    scale = 1
    if text[-1:] in "kK":
        scale, text = 1024, text[:-1]
    elif text[-1:] in "mM":
        scale, text = 1024 * 1024, text[:-1]
    return int(text) * scale


def parse_budget_gib(text: str) -> int:
    """Whole GiB, at least 1 (crates/mrun/src/cli/model.rs: ``parse_budget_gib``)."""
    try:
        value = int(text)
    except ValueError:
        raise argparse.ArgumentTypeError(f"{text!r} is not a whole number of GiB") from None
    if value < 1:
        raise argparse.ArgumentTypeError("the budget must be at least 1 GiB")
    return value


def generation_defaults(model_dir: str) -> dict:
    defaults = dict(temperature=0.0, top_p=1.0, top_k=0, min_p=0.0)
    path = os.path.join(model_dir, "generation_config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            cfg = json.load(f)
    except (OSError, ValueError):
        return defaults
    if cfg.get("do_sample") is False:
        return defaults
    for key in ("temperature", "top_p", "min_p"):
        if isinstance(cfg.get(key), (int, float)) and not isinstance(cfg.get(key), bool):
            defaults[key] = float(cfg[key])
    if isinstance(cfg.get("top_k"), int) and not isinstance(cfg.get("top_k"), bool):
        defaults["top_k"] = cfg["top_k"]
    return defaults


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="mrun", description="one-GPU inference engine for B200")
    sub = parser.add_subparsers(dest="command", required=True)

    run = sub.add_parser("run", help="generate from token ids")
    run.add_argument("model", help="model folder (config.json + safetensors)")
    run.add_argument("--prompt", required=False, help="token ids, inline or a file")
    run.add_argument("--temperature", type=float, default=None,
                     help="sampling temperature [default: generation_config.json, else 0]")
    run.add_argument("--top-p", type=float, default=None)
    run.add_argument("--top-k", type=int, default=None)
    run.add_argument("--min-p", type=float, default=None)
    run.add_argument("--seed", type=int, default=None)
    run.add_argument("--max-tokens", type=int, default=2048)
    run.add_argument("--budget-gib", type=parse_budget_gib, default=os.environ.get("MRUN_BUDGET_GIB"),
                     help="lower the memory budget to this many GiB [default: the GPU's memory less 2 GiB, "
                          "at most what is free less a margin]; it cannot raise it (MRUN_BUDGET_GIB)")
    run.add_argument("--context", type=parse_tokens, default=os.environ.get("MRUN_CONTEXT"),
                     help="memory for this many tokens of context (64K)")
    run.add_argument("--info", action="store_true", help="print the memory breakdown after loading and exit")
    run.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    run.add_argument("--page-size", type=int, default=16)
    run.add_argument("--max-batch-tokens", type=int, default=2048)
    run.add_argument("--ignore-eos", action="store_true")
    run.add_argument("--stop", action="append", default=[], metavar="IDS",
                     help="a stop sequence of token ids (up to 4 of them): the output ends before it")

    rnd = sub.add_parser("random", help="write a model folder with random weights")
    rnd.add_argument("out", help="folder to write config.json and model.safetensors into")
    rnd.add_argument("--config", required=True, help="a config.json of a supported architecture")
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--std", type=float, default=0.02)
    rnd.add_argument("--norm-noise", type=float, default=0.0)
    rnd.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    return parser


def check_run_args(args) -> Optional[str]:
    """Usage errors found from the flags alone (exit 2), crates/mrun/src/cli/run.rs:105-123."""
    from .sampling.params import SamplingParams
    if args.max_tokens < 1:
        return "--max-tokens must be at least 1"
    if args.budget_gib is not None and args.context is not None:
        return "--context cannot be used with --budget-gib"
    if args.context is not None and args.context < 1:
        return "--context must be at least 1 token"
    try:
        SamplingParams(temperature=args.temperature if args.temperature is not None else 0.0,
                       top_p=args.top_p if args.top_p is not None else 1.0,
                       top_k=args.top_k if args.top_k is not None else 0,
                       min_p=args.min_p if args.min_p is not None else 0.0,
                       seed=args.seed).validate()
    except ValueError as error:
        return str(error)
    return None


def command_run(args) -> int:
    problem = check_run_args(args)
    if problem:
        print(f"error: {problem}", file=sys.stderr)
        return 2
    prompt = parse_ids(args.prompt) if args.prompt else []
    if not prompt and not args.info:
        print("error: the prompt is empty", file=sys.stderr)
        return 2
    from .engine import budget
    from .engine.engine import Engine
    loaded = time.perf_counter()
    try:
        # one request at a time: the cache holds at most the model's longest sequence
        memory = budget.plan(budget.read_device(), args.budget_gib)
        engine = Engine.from_folder(args.model, dtype=args.dtype, page_size=args.page_size,
                                    context=args.context, max_requests=1,
                                    max_batch_tokens=args.max_batch_tokens, memory=memory)
    except budget.BudgetError as error:
        print(f"error: {error}", file=sys.stderr)
        return 4
    info = engine.info()
    gib = lambda b: b / float(1 << 30)
    print(f"loaded {info['architecture']} in {time.perf_counter() - loaded:.1f} s: budget "
          f"{gib(info['memory']['budget_bytes']):.2f} GiB ({info['memory']['binding']}) = weights "
          f"{gib(info['weights_bytes']):.2f} GiB + scratch {gib(info['memory']['scratch_bytes']):.2f} GiB + "
          f"cache {gib(info['cache_bytes']):.2f} GiB "
          f"({info['capacity_tokens']} tokens in {info['num_pages']} pages of {info['page_size']})",
          file=sys.stderr)
    if args.info:
        print(json.dumps(info, indent=2))
        return 0
    defaults = generation_defaults(args.model)
    pick = lambda value, key: defaults[key] if value is None else value
    start = time.perf_counter()
    streamed = []

    def show(_, token):                     # ids go out as they are read back, as `mrun run` streams text
        sys.stdout.write(("," if streamed else "") + str(token))
        sys.stdout.flush()
        streamed.append(token)

    result = engine.generate([prompt], max_tokens=args.max_tokens, on_token=show,
                             temperature=pick(args.temperature, "temperature"),
                             top_p=pick(args.top_p, "top_p"), top_k=pick(args.top_k, "top_k"),
                             min_p=pick(args.min_p, "min_p"), seed=args.seed,
                             ignore_eos=args.ignore_eos, stop=[parse_ids(ids) for ids in args.stop])[0]
    total = time.perf_counter() - start
    if result.finish_reason in ("invalid", "too_long", "queue_full"):
        print(f"error: {result.message}", file=sys.stderr)
        return 1
    print("" if streamed == result.tokens else "\n" + ",".join(map(str, result.tokens)))
    ttft = result.time_to_first_token_s
    print(f"prompt: {len(prompt)} tokens, {len(prompt) / max(ttft, 1e-9):.1f} tokens-per-sec", file=sys.stderr)
    print(f"generation: {len(result.tokens)} tokens, "
          f"{(len(result.tokens) - 1) / max(total - ttft, 1e-9):.1f} tokens-per-sec "
          f"({result.finish_reason}" + (f" {result.stop_sequence}" if result.stop_sequence else "") + ")",
          file=sys.stderr)
    return 0


def command_random(args) -> int:
    from . import registry
    from .config.base import read_json
    from .weights import write_random_model
    cfg = read_json(args.config)
    config = registry.resolve(cfg, args.config).from_dict(cfg, None)
    write_random_model(config, args.out, seed=args.seed, std=args.std, norm_noise=args.norm_noise,
                       dtype=args.dtype)
    print(f"wrote {args.out} ({config.num_parameters():,} parameters, seed {args.seed})", file=sys.stderr)
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    try:
        if args.command == "run":
            return command_run(args)
        return command_random(args)
    except (ValueError, FileNotFoundError, RuntimeError) as error:
        print(f"error: {error}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
