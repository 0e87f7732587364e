"""Command line in the manner of the reference's `microllm_hf_infer` (apps/hf_infer.cpp):
`--name value` pairs, every flag validated, one JSON line on standard output.

Flags with the reference's names keep the reference's meaning (hf_infer.cpp:32-73, rules
:179-285): --config/--weights, --tokens, --device, --workload both|prefill|decode|continuous,
--new-tokens, --batch, --warmup/--steps, --prefill-warmup/--prefill-steps, --top-k (how many
top logits to print), --logits-output, --prefill-logits last|full (full: the head is applied at every prompt
position and --logits-output holds [tokens, vocab]; the top logits are the last position's either way), --cache-logits-output, --cache-prefill-mode
full|token, --bf16-ffn/--bf16-attention, --kv-cache-dtype, --cache-capacity,
--continuous-slots, --continuous-prompt-lengths, --continuous-new-token-lengths,
--continuous-prompt-offsets, --continuous-arrival-steps.  Flags that choose between code paths the reference has
and this engine does not are read and checked as the reference checks them, and accepted with the one value
that describes this engine: --use-cache true (there is no uncached path), --batch-argmax-mode device, --decode-mode generation, --continuous-prefill-batch true,
--continuous-diagnostics false; any other legal value is refused with a sentence that says so, and
--continuous-cache-buckets (a paged cache has no buckets), --kv-cache-fp32-layers and the
tokenizer flags (--text, --vocab, --merges, --tokenizer-family, --chat-user) are refused by name.
--trace-output FILE (with --trace-max-elements N, prefill workload only, as hf_infer.cpp:268-273) writes one JSON line per
intermediate tensor of the prompt's step in the reference's record layout (src/profiling/trace.cpp:156-195): the embedding,
the residual stream and the pending delta after every layer, the final norm and the logits, each with its statistics and
its first N values.  The reference's command line is
always greedy and has no random-weights mode; added here: --model DIR (config.json and
model.safetensors in one folder), --dtype fp32|bf16, --temperature, --sampling-top-k, --seed,
--stop-tokens, --stop-on-eos true|false (the configuration's eos_token_id ends a generation), --page-size,
--num-pages, --max-tokens-per-step, --max-seqs, and
--random-config NAME --random-seed S --write-model DIR to write a random model folder.
Tokenizers are out of scope: prompts are token ids.
"""
from __future__ import annotations

import json
import os
import sys
import time
from typing import Dict, List, Optional

BOOL = {"true": True, "false": False}

DEFAULTS: Dict[str, object] = {
    "config": "", "weights": "", "model": "", "tokens": "", "device": "cuda", "top-k": 10,
    "logits-output": "", "cache-logits-output": "", "new-tokens": 0, "warmup": 0, "steps": 1,
    "prefill-warmup": 0, "prefill-steps": 1, "bf16-ffn": None, "bf16-attention": None, "workload": "both",
    "batch": 1, "cache-prefill-mode": "full", "kv-cache-dtype": "", "cache-capacity": 0, "dtype": "",
    "continuous-slots": 0, "continuous-prompt-lengths": "", "continuous-new-token-lengths": "",
    "continuous-prompt-offsets": "", "continuous-arrival-steps": "",
    "temperature": 0.0, "sampling-top-k": 0, "seed": 1, "stop-tokens": "", "page-size": 16, "num-pages": 0,
    "max-tokens-per-step": 2048, "max-seqs": 64, "random-config": "", "random-seed": 0, "write-model": "",
    "stop-on-eos": "false", "trace-output": "", "trace-max-elements": 4096,
    # the reference's switches between code paths: only the value that describes this engine is accepted
    "use-cache": "true", "prefill-logits": "last", "batch-argmax-mode": "device", "decode-mode": "generation",
    "continuous-prefill-batch": "true", "continuous-diagnostics": "false",
}

# flag -> (legal values in the reference, the one this engine has, what the others would need)
ONE_WAY = {
    "use-cache": (("true", "false"), "true", "there is no uncached forward pass"),
    "batch-argmax-mode": (("device", "host"), "device", "tokens are always selected on the device"),
    "decode-mode": (("generation", "steady"), "generation", "steady decoding of a fixed batch is what bench.py measures"),
    "continuous-prefill-batch": (("true", "false"), "true", "prompt portions always share a step"),
    "continuous-diagnostics": (("true", "false"), "false", "the scheduler's metrics are in the JSON line already"),
}
NOT_HERE = {
    "continuous-cache-buckets": "a paged cache has no capacity buckets",
    "kv-cache-fp32-layers": "the cache has the compute dtype in every layer",
    "bf16-algorithm-index": "the library chooses its own algorithm",
    "text": "tokenizers are not part of this engine: give --tokens",
    "vocab": "tokenizers are not part of this engine: give --tokens",
    "merges": "tokenizers are not part of this engine: give --tokens",
    "tokenizer-family": "tokenizers are not part of this engine: give --tokens",
    "chat-user": "tokenizers are not part of this engine: give --tokens",
}


class UsageError(ValueError):
    pass


class TensorTrace:
    """Collects (name, tensor) from a step and writes them as JSON lines in the reference's record layout
    (src/profiling/trace.cpp:126-195: sequence, kind, name, shape, dtype, statistics over the finite values,
    the first `max_elements` values)."""

    def __init__(self, path: str, max_elements: int, run_id: str):
        self.path, self.max_elements, self.run_id = path, int(max_elements), run_id
        self.records = []

    def __call__(self, name, tensor) -> None:
        import torch
        values = tensor.detach().to(torch.float64).reshape(-1).cpu()
        finite = values[torch.isfinite(values)]
        stats = {"numel": int(values.numel()), "finite_count": int(finite.numel()), "minimum": 0.0, "maximum": 0.0,
                 "mean": 0.0, "l2_norm": 0.0}
        if finite.numel():
            stats.update(minimum=float(finite.min()), maximum=float(finite.max()), mean=float(finite.mean()),
                         l2_norm=float(finite.square().sum().sqrt()))
        head = values[:self.max_elements].tolist()
        shown = [("nan" if v != v else "inf" if v == float("inf") else "-inf" if v == float("-inf") else v) for v in head]
        self.records.append({"schema_version": 1, "framework": "microllm_rocm_b200", "run_id": self.run_id,
                             "phase": "inference-values", "sequence": len(self.records), "iteration": 0,
                             "kind": "model" if name in ("embedding", "final_norm", "logits") else "layer", "name": name,
                             "shape": list(tensor.shape), "dtype": str(tensor.dtype).replace("torch.", ""),
                             "device": str(tensor.device), "wall_ms": 0.0, "statistics": stats,
                             "values_truncated": values.numel() > len(head), "values": shown})

    def write(self) -> int:
        folder = os.path.dirname(os.path.abspath(self.path))
        os.makedirs(folder, exist_ok=True)
        with open(self.path, "w", encoding="utf-8") as f:
            for r in self.records:
                f.write(json.dumps(r) + "\n")
        return len(self.records)


def parse(argv: List[str]) -> Dict[str, object]:
    opts = dict(DEFAULTS)
    if len(argv) % 2:
        raise UsageError("missing CLI value")
    for i in range(0, len(argv), 2):
        name, value = argv[i], argv[i + 1]
        if name.startswith("--") and name[2:] in NOT_HERE:
            raise UsageError(f"{name} is an option of the reference that this engine does not have: {NOT_HERE[name[2:]]}")
        if not name.startswith("--") or name[2:] not in DEFAULTS:
            raise UsageError(f"unknown CLI option: {name}")
        key = name[2:]
        default = DEFAULTS[key]
        try:
            if key in ("bf16-ffn", "bf16-attention"):
                if value not in BOOL:
                    raise UsageError(f"{name} must be true or false")
                opts[key] = BOOL[value]
            elif isinstance(default, bool):
                opts[key] = BOOL[value]
            elif isinstance(default, int):
                opts[key] = int(value)
            elif isinstance(default, float):
                opts[key] = float(value)
            else:
                opts[key] = value
        except (ValueError, KeyError):
            raise UsageError(f"{name}: cannot read {value!r}") from None
    return opts


def int_list(text: str, what: str) -> List[int]:
    try:
        return [int(x) for x in text.split(",") if x != ""]
    except ValueError:
        raise UsageError(f"{what} must be comma-separated integers") from None


def validate(o: Dict[str, object]) -> None:
    if o["prefill-logits"] not in ("last", "full"):
        raise UsageError("--prefill-logits must be last or full")
    if o["stop-on-eos"] not in BOOL:
        raise UsageError("--stop-on-eos must be true or false")
    if o["trace-max-elements"] <= 0:
        raise UsageError("--trace-max-elements must be positive")
    if o["trace-output"] and (o["workload"] != "prefill" or o["prefill-warmup"] != 0 or o["prefill-steps"] != 1):
        raise UsageError("--trace-output requires prefill workload, zero prefill warmup, and one prefill step")
    for key, (legal, ours, why) in ONE_WAY.items():
        if o[key] not in legal:
            raise UsageError(f"--{key} must be {' or '.join(legal)}")
        if o[key] != ours:
            raise UsageError(f"--{key} {o[key]} is not available in this engine ({why}); only --{key} {ours}")
    if o["random-config"] and o["write-model"]:
        return
    if not o["model"] and not (o["config"] and o["weights"]):
        raise UsageError("--config and --weights are required (or --model DIR)")
    if o["device"] not in ("cuda", "cuda:0", "gpu"):
        raise UsageError("--device must be cuda: this engine has no CPU path")
    if o["workload"] not in ("both", "prefill", "decode", "continuous"):
        raise UsageError("--workload must be both, prefill, decode or continuous")
    if o["top-k"] <= 0:
        raise UsageError("--top-k must be positive")
    if o["batch"] <= 0:
        raise UsageError("--batch must be positive")
    if o["cache-prefill-mode"] not in ("full", "token"):
        raise UsageError("--cache-prefill-mode must be full or token")
    if o["new-tokens"] < 0:
        raise UsageError("--new-tokens cannot be negative")
    if o["cache-capacity"] < 0:
        raise UsageError("--cache-capacity cannot be negative")
    if o["warmup"] < 0 or o["steps"] <= 0 or o["prefill-warmup"] < 0 or o["prefill-steps"] <= 0:
        raise UsageError("--warmup must be nonnegative and --steps positive")
    if o["workload"] == "decode" and o["new-tokens"] <= 0:
        raise UsageError("decode workload requires positive --new-tokens")
    if o["workload"] == "prefill" and o["new-tokens"] != 0:
        raise UsageError("prefill workload requires --new-tokens 0")
    if o["bf16-attention"] and not o["bf16-ffn"]:
        raise UsageError("--bf16-attention requires --bf16-ffn true")
    if o["bf16-ffn"] and o["bf16-attention"] is False:
        raise UsageError("this engine keeps all matrices in one dtype: give both --bf16-ffn and --bf16-attention, or --dtype")
    if o["dtype"] not in ("", "fp32", "bf16", "float32", "bfloat16"):
        raise UsageError("--dtype must be fp32 or bf16")
    if o["cache-logits-output"] and o["new-tokens"] < 2:
        raise UsageError("--cache-logits-output needs at least two new tokens")
    if o["workload"] == "continuous":
        if o["continuous-slots"] <= 0 or not o["continuous-prompt-lengths"] or not o["continuous-new-token-lengths"]:
            raise UsageError("continuous workload requires --continuous-slots, --continuous-prompt-lengths and "
                             "--continuous-new-token-lengths")
    elif not o["tokens"]:
        raise UsageError("--tokens is required (tokenizers are not part of this engine)")


def compute_dtype(o) -> str:
    if o["dtype"]:
        return "float32" if o["dtype"] in ("fp32", "float32") else "bfloat16"
    if o["bf16-ffn"] or o["bf16-attention"]:
        return "bfloat16"
    return "float32"                     # the reference's default is fp32 as well


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv in (["--help"], ["-h"]):             # the reference has no such flag; its options are `--name value` pairs
        print(__doc__.strip())
        print("\nOptions and their defaults:")
        for name, value in DEFAULTS.items():
            print(f"  --{name} {value!r}")
        return 0
    try:
        o = parse(argv)
        validate(o)
    except UsageError as e:
        print(json.dumps({"schema_version": 1, "status": "error", "error": str(e)}))
        return 2
    if o["random-config"] and o["write-model"]:
        from .config import find_preset, parameter_count
        from .weights import write_random_model
        try:
            arch, cfg = find_preset(o["random-config"])
        except KeyError as e:
            print(json.dumps({"schema_version": 1, "status": "error", "error": str(e.args[0])}))
            return 2
        write_random_model(arch, cfg, o["random-seed"], o["write-model"],
                           {"fp32": "float32", "bf16": "bfloat16"}.get(o["dtype"], o["dtype"] or None))
        print(json.dumps({"schema_version": 1, "status": "pass", "wrote": o["write-model"], "architecture": arch.name,
                          "parameter_count": parameter_count(arch, cfg)}))
        return 0
    return run(o)


def run(o) -> int:
    import torch

    from .engine.llm import LLM
    from .engine.loading import load_engine, pages_for_tokens
    from .engine.step import StepEntry
    from .sampling import GenerationConfig

    dtype = compute_dtype(o)
    if o["kv-cache-dtype"] and {"fp32": "float32", "bf16": "bfloat16"}.get(o["kv-cache-dtype"]) != dtype:
        print(json.dumps({"schema_version": 1, "status": "error",
                          "error": "--kv-cache-dtype must equal the compute dtype in this engine"}))
        return 2
    folder = o["model"] or os.path.dirname(os.path.abspath(o["config"]))
    ids = int_list(o["tokens"], "--tokens")
    batch, new_tokens, page = o["batch"], o["new-tokens"], o["page-size"]
    if o["workload"] == "continuous":
        lengths = int_list(o["continuous-prompt-lengths"], "--continuous-prompt-lengths")
        news = int_list(o["continuous-new-token-lengths"], "--continuous-new-token-lengths")
        if len(news) == 1:
            news = news * len(lengths)
        if len(news) != len(lengths):
            raise SystemExit("--continuous-new-token-lengths must have one value or one per prompt")
        need = sum(-(-(l + n) // page) * page for l, n in zip(lengths, news))
        slots = o["continuous-slots"]
    else:
        need = batch * (-(-(len(ids) + new_tokens + 1) // page) * page)
        slots = batch
    capacity = max(o["cache-capacity"] * max(1, slots), need)
    num_pages = o["num-pages"] or pages_for_tokens(capacity, page)
    t0 = time.perf_counter()
    engine = load_engine(folder, dtype=dtype, page_size=page, num_pages=num_pages, max_requests=max(slots, 1),
                         config_path=o["config"] or None, weights_path=o["weights"] or None)
    torch.cuda.synchronize()
    load_ms = (time.perf_counter() - t0) * 1e3
    cfg = engine.config
    props = torch.cuda.get_device_properties(engine.device)
    out = {"schema_version": 1, "status": "pass", "device": str(engine.device), "device_name": props.name,
           "architecture": f"sm_{props.major}{props.minor}", "device_total_bytes": props.total_memory,
           "compute_dtype": dtype, "workload": o["workload"], "parameter_count": engine.parameter_count,
           "loaded_tensors": len(engine.model.expected_tensors()), "token_count": len(ids), "batch": batch,
           "cache_prefill_mode": o["cache-prefill-mode"], "kv_cache_dtype": dtype, "page_size": page,
           "num_pages": num_pages, "warmup": o["warmup"], "steps": o["steps"], "load_ms": load_ms}
    stop_tokens = int_list(o["stop-tokens"], "--stop-tokens")
    if BOOL[o["stop-on-eos"]]:
        # The reference parses eos_token_id and never uses it (src/model/huggingface.cpp:178-179); here it becomes a
        # stop token on request.  A configuration may name one id or a list of them.
        eos = getattr(cfg, "eos_token_id", None)
        eos_ids = [] if eos is None else (list(eos) if isinstance(eos, (list, tuple)) else [eos])
        if not eos_ids:
            print(json.dumps({"schema_version": 1, "status": "error", "error": "--stop-on-eos true: config.json names no eos_token_id"}))
            return 2
        stop_tokens = list(dict.fromkeys(stop_tokens + [int(t) for t in eos_ids]))
        out["stop_on_eos"] = eos_ids
    sampling = GenerationConfig(max_new_tokens=max(new_tokens, 0), temperature=o["temperature"],
                                top_k=o["sampling-top-k"], seed=o["seed"], stop_tokens=tuple(stop_tokens))

    def timed(fn):
        torch.cuda.synchronize()
        a = time.perf_counter()
        r = fn()
        torch.cuda.synchronize()
        return r, (time.perf_counter() - a) * 1e3

    full_logits = o["prefill-logits"] == "full"
    tracer = TensorTrace(o["trace-output"], o["trace-max-elements"], dtype) if o["trace-output"] else None

    def prefill_once():
        cache = engine.cache
        rows = [f"p{b}" for b in range(batch)]
        for r in rows:
            cache.add(r)
        try:
            if o["cache-prefill-mode"] == "token":          # the prompt one token at a time
                logits = None
                pieces = []
                for i, t in enumerate(ids):
                    logits = engine.step([StepEntry(r, [t], [0] if (full_logits or i == len(ids) - 1) else []) for r in rows])
                    if full_logits:
                        pieces.append(logits[:1])
                if full_logits:
                    logits = torch.cat(pieces)                # the first request's rows, one per position
            else:
                want = list(range(len(ids))) if full_logits else [len(ids) - 1]
                logits = engine.step([StepEntry(r, ids, want) for r in rows], tensor_sink=tracer)
            engine.check_device_errors()
            return logits
        finally:
            for r in rows:
                cache.release(r)

    if o["workload"] in ("prefill", "both"):
        for _ in range(o["prefill-warmup"]):
            prefill_once()
        total = 0.0
        for _ in range(o["prefill-steps"]):
            logits, ms = timed(prefill_once)
            total += ms
        first = logits[:len(ids)].to("cpu") if full_logits else logits[:1].to("cpu")     # the first request's rows
        row = first[-1]
        if o["logits-output"]:
            (first if full_logits else row).numpy().astype("<f4").tofile(o["logits-output"])
        top = torch.topk(row, min(o["top-k"], row.numel()))
        out.update({"prefill_warmup": o["prefill-warmup"], "prefill_steps": o["prefill-steps"],
                    "prefill_logits_mode": o["prefill-logits"],
                    "forward_ms": total / o["prefill-steps"],
                    "prefill_tokens_per_second": batch * len(ids) * o["prefill-steps"] / (total / 1e3),
                    "top_logits": [{"token": int(i), "logit": float(v)} for v, i in zip(top.values, top.indices)]})
        if tracer is not None:
            out["trace_record_count"] = tracer.write()

    if o["workload"] in ("decode", "both") and new_tokens > 0:
        llm = LLM(engine, max_tokens_per_step=o["max-tokens-per-step"], max_seqs=max(batch, o["max-seqs"]))
        for _ in range(o["warmup"]):
            llm.generate([ids] * batch, sampling)
        total, generated = 0.0, None
        for _ in range(o["steps"]):
            steps_before = engine.steps_run
            generated, ms = timed(lambda: llm.generate([ids] * batch, sampling))
            total += ms
            forward_steps = engine.steps_run - steps_before
        measured = sum(len(g) for g in generated)
        out.update({"generation_ms": total, "mean_generation_ms": total / o["steps"], "measured_tokens": measured,
                    "measured_forward_steps": forward_steps,
                    "decode_step_semantics": "first token from the prompt's step, then one step per token",
                    "decode_tokens_per_second": measured * o["steps"] / (total / 1e3),
                    "decode_milliseconds_per_token": (total / o["steps"]) / max(1, measured // batch),
                    "generated_tokens": generated[0], "kv_cache_actual_bytes": engine.cache.kv_bytes(),
                    "kv_cache_capacity_tokens": num_pages * page})
        if o["cache-logits-output"]:
            # logits after the last cached decode step: the step that fed generated[-2]
            cache = engine.cache
            cache.add("c")
            seq = ids + generated[0][:-1]
            engine.step([StepEntry("c", ids, [])])
            logits = None
            for t in seq[len(ids):]:
                logits = engine.step([StepEntry("c", [t], [0])])
            cache.release("c")
            logits[0].to("cpu").numpy().astype("<f4").tofile(o["cache-logits-output"])
            out["cache_logits_step"] = new_tokens - 1

    if o["workload"] == "continuous":
        import random
        offsets = int_list(o["continuous-prompt-offsets"], "--continuous-prompt-offsets") or [0] * len(lengths)
        arrivals = int_list(o["continuous-arrival-steps"], "--continuous-arrival-steps") or [0] * len(lengths)
        if len(offsets) != len(lengths) or len(arrivals) != len(lengths):
            raise SystemExit("--continuous-prompt-offsets/--continuous-arrival-steps need one value per prompt")
        base = ids or [random.Random(7).randrange(cfg.vocab_size) for _ in range(max(lengths) + max(offsets))]
        while len(base) < max(l + f for l, f in zip(lengths, offsets)):
            base = base + base
        prompts = [base[f:f + l] for l, f in zip(lengths, offsets)]
        llm = LLM(engine, max_tokens_per_step=o["max-tokens-per-step"], max_seqs=slots)
        # arrival steps are meant exactly: a request that arrives at step k is planned in step k.  A step issued
        # ahead of its predecessor's results would already be on its way when the request arrives, so that is
        # switched off when arrivals are spread over steps.
        llm.lookahead = not any(a > 0 for a in arrivals)
        pending = sorted(range(len(prompts)), key=lambda i: arrivals[i])
        submitted: Dict[int, int] = {}

        def drive():
            step = 0
            queue = list(pending)
            while queue or llm.has_work():
                while queue and arrivals[queue[0]] <= step:
                    i = queue.pop(0)
                    submitted[i] = llm.submit(prompts[i], GenerationConfig(
                        max_new_tokens=news[i], temperature=o["temperature"], top_k=o["sampling-top-k"], seed=o["seed"]))
                if llm.has_work():
                    llm.step()
                step += 1
            return step

        steps, ms = timed(drive)
        reqs = [llm.poll(submitted[i]) for i in range(len(prompts))]
        m = llm.metrics()
        out.update({"continuous_slots": slots, "requests": len(prompts), "scheduler_steps": m["steps"],
                    "admissions": m["admissions"], "preemptions": m["preemptions"],
                    "prompt_tokens": m["prompt_tokens"], "decode_tokens": m["decode_tokens"],
                    "generated_token_count": m["tokens_generated"], "generation_ms": ms,
                    "tokens_per_second": m["tokens_generated"] / (ms / 1e3),
                    "first_token_steps": [r.first_token_step for r in reqs],
                    "completion_steps": [r.completion_step for r in reqs],
                    "generated_tokens": [r.generated for r in reqs], "cache": m["cache"]})
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
