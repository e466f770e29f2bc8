"""Trace replay: feed given token ids through a model step by step, write logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Reads one JSON object per line from standard input:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step that wants logits it writes OUT/<step>.f32 (little-endian float32,
[wanted, vocab], in the order of the entries and of each `want`), then prints
`done <step>`.  It samples nothing and owns no model code: every step goes
through the engine's own step function, cache and kernels, the ones generation
uses.  `--dtype float32` runs every operation in true 32-bit arithmetic.
`--max-tokens` sizes the cache: the most tokens live requests hold at any time,
each request's count rounded up to a multiple of 64.

Two options exist for tests: `--chunk-tokens N` makes the engine run a step of
more than N tokens as several passes over the cache, and `--poison-unused`
fills, before every step, each cache row that no live request owns with NaN
(rows of free pages, rows beyond a request's length); logits must not change.
"""
import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run")
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--chunk-tokens", type=int, default=None, help="tokens per forward pass (default: the engine's)")
    ap.add_argument("--poison-unused", action="store_true", help="fill cache rows nobody owns with NaN before each step")
    args = ap.parse_args(argv)

    import numpy as np
    from mdma_b200.engine import Engine, StepEntry

    os.makedirs(args.out, exist_ok=True)
    page = 64
    max_tokens = -(-args.max_tokens // page) * page
    probe_cfg = json.load(open(os.path.join(args.model, "config.json")))
    max_context = min(int(probe_cfg.get("max_position_embeddings", max_tokens)), max_tokens)
    extra = {} if args.chunk_tokens is None else {"chunk_tokens": args.chunk_tokens}
    # A step may want the logits of every token it brings, so the logits buffer has a row per token of the
    # cache; but never more than a quarter of the free device memory (a step that wants more rows than
    # that is refused with the engine's own error, not truncated).
    import torch
    logit_rows = max_tokens
    vocab = int(probe_cfg.get("vocab_size", 0))
    if vocab > 0 and torch.cuda.is_available():
        free_bytes, _ = torch.cuda.mem_get_info()
        logit_rows = max(64, min(max_tokens, (free_bytes // 4) // (4 * vocab)))
    engine = Engine(args.model, dtype=args.dtype, max_tokens=max_tokens, max_context=max_context,
                    page_size=page, logit_rows=logit_rows, **extra)
    slots: dict = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        req = json.loads(line)
        step = req["step"]
        entries = []
        for e in req.get("entries", []):
            rid = e["id"]
            if rid not in slots:
                slots[rid] = engine.acquire()
            entries.append(StepEntry(slots[rid], e["tokens"], e.get("want", [])))
        if entries:
            if args.poison_unused:
                engine.cache.poison_unused()
            logits = engine.step(entries)
            engine.check_status()          # a kernel that gave up on a wait: stop here, write nothing
            if logits.shape[0]:
                arr = logits.cpu().numpy().astype("<f4", copy=False)
                with open(os.path.join(args.out, f"{step}.f32"), "wb") as f:
                    f.write(np.ascontiguousarray(arr).tobytes())
        for rid in req.get("end", []):
            if rid in slots:
                engine.release(slots.pop(rid))
        print(f"done {step}", flush=True)
    return 0
