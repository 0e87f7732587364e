"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and owns nothing: model, loader, cache manager, step function and
kernels are the ones generation uses.  Steps come as JSON lines on standard input,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

and for every step in which something is wanted `OUT/<step>.f32` receives the logits at the
wanted places, [wanted, vocab] little-endian fp32, in the order of the entries and of
`want`.  After every step a line `done <step>` goes to standard output.

The reference's nearest pieces are `--cache-prefill-mode token` (apps/hf_infer.cpp:331-339),
which replays a prompt token by token, and `--logits-output` (hf_infer.cpp:1175-1181).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List

TRACE_PAGE_SIZE = 16       # divides the 64-token granularity in which --max-tokens is counted
MAX_LIVE_REQUESTS = 8      # traces hold up to four at a time


def parse_args(argv):
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time (each rounded up to 64)")
    p.add_argument("--page-size", type=int, default=TRACE_PAGE_SIZE)
    p.add_argument("--guard-pages", action="store_true",
                   help="debugging aid: a page of a fixed pattern in front of and behind every cache pool, read back after every step")
    return p.parse_args(argv)


def run(argv: List[str], stdin=None, stdout=None) -> int:
    args = parse_args(argv)
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    if args.max_tokens <= 0 or args.page_size <= 0:
        print("trace_run: --max-tokens and --page-size must be positive", file=sys.stderr)
        return 2
    os.makedirs(args.out, exist_ok=True)
    print(f"[trace_run] loading {args.model} as {args.dtype}", file=sys.stderr, flush=True)
    from .loading import load_engine, pages_for_tokens
    num_pages = pages_for_tokens(args.max_tokens, args.page_size)
    engine = load_engine(args.model, dtype=args.dtype, page_size=args.page_size, num_pages=num_pages,
                         max_requests=MAX_LIVE_REQUESTS, guard_pages=args.guard_pages)
    print(f"[trace_run] ready: {num_pages} pages of {args.page_size} tokens per layer group",
          file=sys.stderr, flush=True)
    def to_file(step, logits):
        logits.numpy().astype("<f4", copy=False).tofile(os.path.join(args.out, f"{step}.f32"))

    def steps():
        for line in stdin:
            line = line.strip()
            if line:
                yield json.loads(line)

    def done(step):
        stdout.write(f"done {step}\n")
        stdout.flush()

    replay(engine, steps(), to_file, done)
    return 0


def replay(engine, steps, sink, done=None) -> None:
    """Drive `engine` through `steps` (dicts of the trace format).  `sink(step, logits)` gets
    the wanted logits of a step as a CPU fp32 tensor [wanted, vocab]; `done(step)` is called
    after each step.  Requests are added to the cache when first seen and released when a
    step lists them under "end"."""
    from .step import StepEntry
    cache = engine.cache
    for msg in steps:
        step = msg["step"]
        entries = []
        for e in msg.get("entries", []):
            if not cache.has(e["id"]):
                if not cache.add(e["id"]):
                    raise RuntimeError(f"step {step}: more live requests than the cache has slots for")
            entries.append(StepEntry(e["id"], e["tokens"], e.get("want", [])))
        if entries:
            logits = engine.step(entries)
            if logits.shape[0] > 0:
                sink(step, logits.detach().to("cpu").contiguous())
            engine.check_device_errors()
        for rid in msg.get("end", []):
            if cache.has(rid):
                cache.release(rid)
        if done is not None:
            done(step)


def main() -> None:
    sys.exit(run(sys.argv[1:]))
