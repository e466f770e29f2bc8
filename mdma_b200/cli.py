"""Command line in the manner of the reference's `mdma run` / `mdma plan`
(src/bin/mdma/run.rs:14-34, src/bin/mdma/plan.rs:10-35) and `mdma-run MODEL
PROMPT [MAX_TOKENS]` (src/bin/mdma-run.rs:40-55).  There is no tokenizer here:
a PROMPT is a list of token ids ("5,17,3" or "5 17 3"); several prompts form a
batch.  Options the reference has keep its names and meanings (--max-tokens,
--vram-bytes, --reserve-mib, --json; MDMA_JSON for mdma-run); --backend and
--gpu-layers do not exist because there is one backend and one device.
`mdma replay ...` is the trace replay program (bin/trace_run); the benchmark is
`bench.py` at the top of the repository.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def parse_ids(text: str) -> list[int]:
    parts = [p for p in text.replace(",", " ").split() if p]
    if not parts:
        raise argparse.ArgumentTypeError("a prompt needs at least one token id")
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise argparse.ArgumentTypeError(f"token ids must be integers: {text!r}") from None


def _add_engine_args(ap):
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-context", type=int, default=None, help="rows a sequence may hold (default: the model's)")
    ap.add_argument("--max-batch", type=int, default=8)
    ap.add_argument("--vram-bytes", type=int, default=None, help="device memory the plan may use")
    ap.add_argument("--reserve-mib", type=int, default=256, help="headroom kept free on the device")


def cmd_run(args) -> int:
    from .engine.generate import Generator
    from .engine.step import Engine, MemoryBudgetError
    from .sampling import SamplingParams
    prompts = [args.prompt] + list(args.more_prompts or [])
    if args.max_tokens <= 0:
        print("--max-tokens must be positive", file=sys.stderr)
        return 2
    need_ctx = max(len(p) for p in prompts) + args.max_tokens
    source = {"model_dir": args.model}
    if args.random_weights is not None:
        # no weights are read: the configuration (a config.json, or a folder that holds one) and a seed
        path = os.path.join(args.model, "config.json") if os.path.isdir(args.model) else args.model
        with open(path, "r", encoding="utf-8") as f:
            source = {"config": json.load(f), "seed": args.random_weights}
    try:
        engine = Engine(**source, dtype=args.dtype, max_batch=min(args.max_batch, len(prompts)),
                        max_context=args.max_context or None, reserve_mib=args.reserve_mib,
                        vram_bytes=args.vram_bytes, context_hint=need_ctx,
                        history_cap=max(64, args.repetition_window))
    except MemoryBudgetError as e:
        print(f"model/request does not fit the device budget: {e}", file=sys.stderr)
        return 1
    if args.greedy or os.environ.get("MDMA_GREEDY") == "1":
        params = SamplingParams.greedy()
    else:
        params = SamplingParams(args.temperature, args.top_p, args.min_p, args.repetition_penalty,
                                args.repetition_window, args.seed)
    stop = parse_ids(args.stop_ids) if args.stop_ids else list(engine.spec.stop_token_ids)
    outs = Generator(engine).generate(prompts, args.max_tokens, params, stop)
    for o in outs:
        if args.json or os.environ.get("MDMA_JSON") is not None:
            print(json.dumps({"prompt_tokens": o.prompt_tokens, "tokens": o.tokens,
                              "finish_reason": o.finish_reason}))
        else:
            print(" ".join(str(t) for t in o.tokens))
    return 0


def cmd_plan(args) -> int:
    from .engine.step import plan_only
    plan = plan_only(args.model, dtype=args.dtype, max_batch=args.batch, max_context=args.ctx,
                     chunk_tokens=max(args.prompt_tokens, 1) * args.batch)
    if args.vram_bytes is not None:
        plan["fits"] = plan["total_bytes"] + args.reserve_mib * (1 << 20) <= args.vram_bytes
    if args.json:
        print(json.dumps(plan))
    else:
        for k, v in plan.items():
            print(f"{k:>18}: {v}")
    return 0


def cmd_init_random(args) -> int:
    import torch
    from .weights import write_random_model
    with open(args.config, "r", encoding="utf-8") as f:
        cfg = json.load(f)
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    write_random_model(args.out, cfg, args.seed, dtype)
    print(args.out)
    return 0


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="mdma", description="Llama generation on one B200")
    sub = ap.add_subparsers(dest="command", required=True)

    run = sub.add_parser("run", help="generate from token-id prompts")
    run.add_argument("model", help="folder with config.json and model.safetensors")
    run.add_argument("prompt", type=parse_ids, help='token ids, e.g. "5,17,3"')
    run.add_argument("--prompt", dest="more_prompts", type=parse_ids, action="append",
                     help="a further prompt of the same batch (repeatable)")
    run.add_argument("--max-tokens", type=int, default=32)
    run.add_argument("--json", action="store_true")
    run.add_argument("--greedy", action="store_true", help="argmax, no penalty (the default temperature is 0 as well)")
    run.add_argument("--temperature", type=float, default=0.0)
    run.add_argument("--top-p", type=float, default=1.0)
    run.add_argument("--min-p", type=float, default=0.0)
    run.add_argument("--repetition-penalty", type=float, default=1.0)
    run.add_argument("--repetition-window", type=int, default=64)
    run.add_argument("--seed", type=int, default=0)
    run.add_argument("--stop-ids", default=None, help="token ids that end a sequence (default: the config's eos)")
    run.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                     help="seeded random weights instead of the folder's (MODEL may then be a config.json)")
    _add_engine_args(run)
    run.set_defaults(fn=cmd_run)

    plan = sub.add_parser("plan", help="print the memory plan without loading weights")
    plan.add_argument("model")
    plan.add_argument("--ctx", type=int, default=512)
    plan.add_argument("--batch", type=int, default=1)
    plan.add_argument("--prompt-tokens", type=int, default=32)
    plan.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    plan.add_argument("--vram-bytes", type=int, default=None)
    plan.add_argument("--reserve-mib", type=int, default=256)
    plan.add_argument("--json", action="store_true")
    plan.set_defaults(fn=cmd_plan)

    sub.add_parser("replay", help="feed given token ids step by step and write logits (= bin/trace_run)", add_help=False)

    init = sub.add_parser("init-random", help="write a model folder with seeded random weights")
    init.add_argument("config", help="a config.json")
    init.add_argument("out")
    init.add_argument("--seed", type=int, default=0)
    init.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    init.set_defaults(fn=cmd_init_random)
    return ap


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "replay":            # its own options, taken as they are
        from .replay import main as replay_main
        return replay_main(argv[1:])
    args = build_parser().parse_args(argv)
    try:
        return args.fn(args)
    except (ValueError, RuntimeError, KeyError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1


def main_run_compat(argv=None) -> int:
    """`mdma-run MODEL PROMPT [MAX_TOKENS]`: greedy, MDMA_JSON selects JSON output."""
    argv = list(sys.argv[1:] if argv is None else argv)
    if not 2 <= len(argv) <= 3:
        print("usage: mdma-run MODEL_DIR PROMPT_IDS [MAX_TOKENS]", file=sys.stderr)
        return 2
    return main(["run", argv[0], argv[1], "--max-tokens", argv[2] if len(argv) == 3 else "32", "--greedy"])
