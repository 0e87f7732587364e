"""Decode throughput of the engine on one B200, with prefill and roofline figures.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]
                    [--model PRESET] [--batch B] [--prompt P] [--context C]
                    [--workload decode|mixed] [--requests R] [--new-tokens N] [--chunk T]

The model has the layer sizes of the Qwen2.5-1.5B shape (BASELINE.json configs[2]) with
random bf16 weights; the default run decodes a batch of 8 requests that hold 2,048-token
prompts (context budget 4,096).  One "step" is one decode step: every live request gets one
new token from one pass through the model.  It prints ONE JSON line:

  value        decoded tokens per second, K steps timed on the device with CUDA events
  e2e          the same through the Python entry point (LLM.submit/step): token ids start
               on the host, every step copies its inputs host->device from pinned memory and
               its selected tokens device->host
  prefill      one 2,048-token prompt: tokens/s, ms, fraction of the bf16 tensor peak
  roofline     bytes the decode step must read (every weight once + the live cache) / time
  points       decode tokens/s at batch 1 and 64
  families     share of the decode step's kernel time by kernel family (products, attention, norms and rotation,
               sampling), from the device's own kernel records of a few replays; null where they cannot be had
  clocks       SM clock and throttle reasons sampled with nvidia-smi during the timed region

`--workload mixed` is the serving workload of BASELINE.json's configs[3]: R requests (64) with prompt lengths
uniform in [128, 2048], prompts cut into portions under a budget of T tokens a step (512) beside the decode tokens
of the requests already running, N new tokens each (128), all through LLM.submit/step.  It prints one line with
generated and processed tokens per second, steps, preemptions, and two views of who waits for whom: the share of the
wall time the host spent blocked in a step's device-to-host read (the GPU was busy for all of that; the rest is the
host preparing and issuing steps, during which the GPU may or may not have work queued) and the driver's own
utilisation samples (coarse: its sampling window is a good part of a second).
`--model qwen2.5-14b --prompt 8192 --context 8448` gives configs[4] (decode at context 8,192, prefill of 2,048).

Each decode step reads ~3 GB of weights, far more than the 126 MB L2, so no L2 flush is
needed between timed iterations.  The reference (walkinglabs/microLLM-rocm) is HIP/ROCm
code without a CUDA path; its CPU build is single-threaded scalar code that needs minutes for one layer of this
shape, so `--impl reference` reports that it is unavailable and why.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from typing import List, Sequence

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
# The reference's own published steady-decode figure for this layer shape (DeepSeek-R1-Distill-Qwen-1.5B, context
# 2,048, batch 8, BF16 weights) -- measured on an AMD MI300X with a real checkpoint: other hardware, orientation only.
BASELINE_DECODE_B8 = 435.0
BASELINE_NOTE = "reference's published steady decode, same layer shape, context 2048, batch 8, on an AMD MI300X (other hardware; orientation, not a like-for-like ratio)"
REFERENCE_UNAVAILABLE = ("walkinglabs/microLLM-rocm is a CMake C++/HIP project for ROCm (gfx942) with no CUDA path and no "
                         "pip-installable package, so its GPU path cannot run on a B200; its CPU build (-DMICROLLM_ENABLE_HIP=OFF) "
                         "runs single-threaded scalar loops and took 103 s for one pass of a 256-token prompt plus 4 tokens through "
                         "ONE layer of this shape, so 28 layers with 8 x 2048-token prompts are far outside the time limit")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            raw = json.load(open(path))
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"])), "source": "measured"}
        except Exception:
            pass
    out = dict(FALLBACK_PEAKS)
    out["bf16_tflops_sustained"] = 1400.0
    return out


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 20 ms while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,utilization.gpu")

    def __init__(self):
        self.samples, self.proc = [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        mhz = [float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[3 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": float(self.samples[0][1]),
                "reasons": reasons, "samples": len(self.samples)}

    def utilization(self):
        """Mean of the driver's `utilization.gpu` samples (share of each sampling period with a kernel running)."""
        values = [float(s[7]) for s in self.samples if len(s) > 7 and s[7].replace(".", "").isdigit()]
        return sum(values) / len(values) / 100.0 if values else None


def decode_bytes(cfg, layers, batch, context, dtype_bytes=2):
    """Bytes one decode step has to read: every weight it uses once (the embedding rows it
    gathers are negligible; a tied table is read once, as the head) plus the K and V of the
    live requests."""
    h, d = cfg.hidden_size, cfg.head_size
    q, kv = cfg.num_attention_heads * d, cfg.num_key_value_heads * d
    per_layer = (h * (q + 2 * kv) + q * h + 3 * h * cfg.intermediate_size) * dtype_bytes + ((q + 2 * kv) + 2 * h) * 4
    weights = layers * per_layer + cfg.vocab_size * h * dtype_bytes + h * 4
    cache = layers * batch * context * 2 * kv * dtype_bytes
    return weights + cache


def prefill_flops(cfg, layers, tokens):
    h, d = cfg.hidden_size, cfg.head_size
    q, kv = cfg.num_attention_heads * d, cfg.num_key_value_heads * d
    linear = 2 * tokens * layers * (h * (q + 2 * kv) + q * h + 3 * h * cfg.intermediate_size)
    attention = layers * 2 * 2 * cfg.num_attention_heads * d * tokens * (tokens + 1) // 2
    head = 2 * h * cfg.vocab_size
    return linear + attention + head


# ---------------------------------------------------------------------------------- steady decode of a fixed batch
# Prompts are prefilled in portions, then every step() feeds each request the token it was given last and
# selects the next one greedily.  Counted tokens equal forward passes, as in the reference's steady decode
# accounting (apps/hf_infer.cpp:1464-1468).
class DecodeSession:
    def __init__(self, engine, prompts: Sequence[Sequence[int]], max_steps: int, prefill_budget: int = 2048,
                 use_graph: bool = True):
        import torch

        from microllm_rocm_b200.engine.decode_graph import DecodeGraphPool, graph_capable
        from microllm_rocm_b200.engine.step import StepEntry
        from microllm_rocm_b200.kernels import ops
        from microllm_rocm_b200.sampling import GenerationConfig
        self.engine = engine
        self.ids = [f"bench{i}" for i in range(len(prompts))]
        cache = engine.cache
        for rid in self.ids:
            if not cache.add(rid):
                raise RuntimeError("not enough request slots for the benchmark batch")
        self.tokens: List[int] = [0] * len(prompts)
        out = torch.empty(1, dtype=torch.int32, device=engine.device)
        for i, (rid, prompt) in enumerate(zip(self.ids, prompts)):
            at = 0
            while at < len(prompt):
                n = min(prefill_budget, len(prompt) - at)
                last = at + n == len(prompt)
                logits = engine.step([StepEntry(rid, prompt[at:at + n], [n - 1] if last else [])])
                at += n
            ops.argmax_rows(logits, out)
            self.tokens[i] = int(out.item())
        self.picked = torch.empty(len(prompts), dtype=torch.int32, device=engine.device)
        self.graph = None
        if use_graph and graph_capable(engine):
            greedy = GenerationConfig(max_new_tokens=max_steps, temperature=0.0)
            self.lengths = [cache.length(rid) for rid in self.ids]
            for rid, n in zip(self.ids, self.lengths):
                if not cache.reserve(rid, n + 1):
                    raise RuntimeError("no pages for the benchmark batch")
            pool = DecodeGraphPool(engine)
            self.graph = pool.get(self.ids, headroom_tokens=max_steps)
            state = (self.tokens, self.lengths, [greedy] * len(self.ids), [1] * len(self.ids))
            self.graph.load(self.ids, *state)
            pool.ensure_captured(self.graph)
            self.graph.load(self.ids, *state)

    def step(self) -> None:
        if self.graph is None:
            from microllm_rocm_b200.engine.step import StepEntry
            from microllm_rocm_b200.kernels import ops
            logits = self.engine.step([StepEntry(rid, [t], [0]) for rid, t in zip(self.ids, self.tokens)])
            ops.argmax_rows(logits, self.picked)
            self.tokens = self.picked.tolist()
            return
        cache = self.engine.cache
        for i, rid in enumerate(self.ids):                       # a page for the token this step stores
            if not cache.reserve(rid, self.lengths[i] + 1):
                raise RuntimeError("the benchmark batch ran out of pages")
        self.graph.refresh_tables()
        self.graph.replay()
        for i, rid in enumerate(self.ids):
            self.lengths[i] += 1
            cache.commit(rid, self.lengths[i])

    def context_length(self) -> int:
        return max(self.engine.cache.length(rid) for rid in self.ids)

    def close(self) -> None:
        for rid in self.ids:
            self.engine.cache.release(rid)


def count_launches(session: DecodeSession) -> int:
    """Kernels of this library launched by one decode step."""
    from microllm_rocm_b200.kernels.build import LaunchCounter
    if session.graph is not None:
        return session.graph.launches_per_replay
    before = LaunchCounter.own
    session.step()
    return LaunchCounter.own - before


FAMILIES = (("attention", ("fa_", "paged_attention")), ("products", ("gemv", "gemm", "nvjet", "cutlass", "sm100", "sm90")),
            ("norm_rope_act", ("rmsnorm", "rope", "silu", "add_inplace", "embed")), ("sampling", ("argmax", "sample", "decode_advance")))


def _kernel_records(session, replays: int = 3):
    """(name, start us, end us) of every kernel of `replays` decode steps, from the device's kernel records (CUPTI
    through the tensor framework's profiler), in order of start."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(replays):
            session.step()
        torch.cuda.synchronize()
    records = []
    for event in prof.events():
        if event.device_type != torch.autograd.DeviceType.CUDA:
            continue
        name = event.name
        if "memcpy" in name.lower() or "memset" in name.lower():
            continue
        records.append((name, float(event.time_range.start), float(event.time_range.end)))
    records.sort(key=lambda r: r[1])
    return records


def _exposed(records):
    """Kernels of a captured step start early and overlap: what a kernel adds to the step is the time from the
    latest end of everything before it to its own end.  Yields (name, duration, exposed); the exposed times of a
    step add up to its span."""
    frontier = records[0][1] if records else 0.0
    for name, start, end in records:
        yield name, end - start, max(0.0, end - max(frontier, min(start, frontier)))
        frontier = max(frontier, end)


def kernel_families(session):
    """Share of a decode step's time by kernel family.  A kernel's share is its EXPOSED time (see _exposed), so the
    shares add up to the step; the plain sum of kernel durations is given beside it (it counts overlaps twice).
    None when the kernel records cannot be had."""
    try:
        records = _kernel_records(session, 3)
        totals, total, durations = {}, 0.0, 0.0
        for name, duration, exposed in _exposed(records):
            family = next((f for f, marks in FAMILIES if any(m in name.lower() for m in marks)), "other")
            totals[family] = totals.get(family, 0.0) + exposed
            total += exposed
            durations += duration
        if total <= 0:
            return None
        out = {f: round(v / total, 4) for f, v in sorted(totals.items())}
        out["step_ms_by_records"] = round(total / 3 / 1e3, 4)
        out["kernel_ms_per_step"] = round(durations / 3 / 1e3, 4)
        return out
    except Exception:
        return None


def step_timeline(session):
    """Per kernel name of one decode step: launches, duration and exposed time in microseconds."""
    records = _kernel_records(session, 3)
    per_step = len(records) // 3
    records = records[per_step:2 * per_step]
    rows = {}
    for name, duration, exposed in _exposed(records):
        short = name.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0].split("<")[0]
        row = rows.setdefault(short, [0, 0.0, 0.0])
        row[0] += 1
        row[1] += duration
        row[2] += exposed
    span = records[-1][2] - records[0][1] if records else 0.0
    return span, sorted(rows.items(), key=lambda kv: -kv[1][2])


def run_mixed(args):
    """BASELINE.json configs[3]: many requests of assorted prompt lengths through the scheduler, prompts in portions
    under a token budget beside the decode tokens of the others."""
    import random

    import torch

    from microllm_rocm_b200.config import preset
    from microllm_rocm_b200.engine.llm import LLM
    from microllm_rocm_b200.engine.loading import random_engine
    from microllm_rocm_b200.kernels.build import LaunchCounter
    from microllm_rocm_b200.sampling import GenerationConfig

    full = preset(args.model)
    layers = args.layers or full.num_hidden_layers
    cfg = preset(args.model, num_hidden_layers=layers)
    page = 64
    rng = random.Random(args.seed)
    lengths = [rng.randint(args.min_prompt, args.max_prompt) for _ in range(args.requests)]
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in lengths]
    tokens_needed = sum(-(-(n + args.new_tokens) // page) * page for n in lengths) + page
    if args.pool_tokens:
        tokens_needed = args.pool_tokens
    engine = random_engine(cfg, seed=0, dtype="bfloat16", page_size=page, max_tokens=tokens_needed,
                           max_requests=args.requests, draw_on_device=True)
    llm = LLM(engine, max_tokens_per_step=args.chunk, max_seqs=args.requests)
    config = GenerationConfig(max_new_tokens=args.new_tokens, temperature=0.0)

    kinds = {}

    def run_once():
        ids = [llm.submit(p, config) for p in prompts]
        launches0, steps, wait0 = LaunchCounter.own, 0, llm.wait_s
        kinds.clear()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        while llm.has_work():
            graph_steps, captures, t1 = llm.graph_steps, llm.graphs.captures if llm.graphs else 0, time.perf_counter()
            llm.step()
            # a step ends with the read of its tokens, so its wall time is its own
            kind = ("capturing" if llm.graphs and llm.graphs.captures > captures else
                    "captured" if llm.graph_steps > graph_steps else "mixed")
            entry = kinds.setdefault(kind, [0, 0.0])
            entry[0] += 1
            entry[1] += time.perf_counter() - t1
            steps += 1
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        generated = sum(len(llm.poll(i).generated) for i in ids)
        for i in ids:
            del llm.scheduler.requests[i]
        return wall, steps, generated, LaunchCounter.own - launches0, llm.wait_s - wait0

    run_once()                                   # warm-up: compiles nothing new afterwards, captures the decode steps
    metrics0 = dict(llm.metrics())
    sampler = ClockSampler()
    with sampler:
        time.sleep(0.3)
        wall, steps, generated, launches, waited = run_once()
    metrics = llm.metrics()
    processed = sum(lengths) + generated
    out = {
        "metric": f"mixed serving: generated tokens/s ({args.model}-shape, bf16, {args.requests} requests, prompts "
                  f"U[{args.min_prompt},{args.max_prompt}], {args.new_tokens} new tokens, {args.chunk}-token steps)",
        "value": generated / wall, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": 1,
        "ms_per_step": wall / steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": f"synthetic: random weights N(0,0.02) seed 0, uniform random token ids, prompt lengths from seed {args.seed}",
        "impl": "ours",
        "config": {"model": args.model + "-shape", "layers": layers, "layers_of_model": full.num_hidden_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_size, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "requests": args.requests, "min_prompt": args.min_prompt, "max_prompt": args.max_prompt,
                   "new_tokens": args.new_tokens, "max_tokens_per_step": args.chunk, "page_size": page,
                   "pool_tokens": tokens_needed, "parallelism": "single-gpu"},
        "processed_tokens_per_s": processed / wall, "prompt_tokens": sum(lengths), "generated_tokens": generated,
        "wall_s": wall, "host_waits_for_gpu_frac": waited / wall, "gpu_utilization_sampled": sampler.utilization(),
        "gpu_launches": launches,
        "preemptions": metrics.get("preemptions", 0) - metrics0.get("preemptions", 0),
        # steps that hold prompt portions (issued kernel by kernel), steps of decoded tokens only (a captured
        # step replayed) and steps that had to capture one first: how many, and their wall time in ms
        "step_kinds": {k: {"steps": n, "ms": round(t * 1e3, 1)} for k, (n, t) in sorted(kinds.items())},
        "clocks": sampler.summary(),
    }
    print(json.dumps(out))
    return 0


def run_ours(args):
    import torch

    from microllm_rocm_b200.config import preset
    from microllm_rocm_b200.engine.llm import LLM
    from microllm_rocm_b200.engine.loading import random_engine
    from microllm_rocm_b200.engine.step import StepEntry
    from microllm_rocm_b200.sampling import GenerationConfig

    pk = peaks()
    full = preset(args.model)
    layers = args.layers or full.num_hidden_layers
    cfg = preset(args.model, num_hidden_layers=layers)
    prompt_len, context, page = args.prompt, args.context, 64
    max_batch = max(args.batch, 64 if not (args.skip_points or args.only) else args.batch)
    tokens_needed = max_batch * (context + page)
    engine = random_engine(cfg, seed=0, dtype="bfloat16", page_size=page, max_tokens=tokens_needed,
                           max_requests=max_batch, draw_on_device=True)
    gen = torch.Generator().manual_seed(0)

    def prompts(n):
        return [torch.randint(0, cfg.vocab_size, (prompt_len,), generator=gen).tolist() for _ in range(n)]

    # ---- prefill of 2,048 tokens ------------------------------------------------------------
    def prefill_once():
        engine.cache.add("pf")
        toks = prompts(1)[0][:args.prefill_tokens]
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.step([StepEntry("pf", toks, [len(toks) - 1])])
        end.record()
        torch.cuda.synchronize()
        engine.cache.release("pf")
        return start.elapsed_time(end)

    if args.only == "prefill-timeline":
        # one prompt step kernel by kernel: launches, busy time, and the GPU's idle time in front of each kernel
        class _Prompt:
            def step(self_inner):
                prefill_once()
        for _ in range(max(3, args.warmup)):
            prefill_once()
        records = _kernel_records(_Prompt(), 3)
        per_step = len(records) // 3
        records = records[per_step:2 * per_step]
        rows, frontier, idle_total = {}, records[0][1], 0.0
        for name, begin, end in records:
            short = name.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0].split("<")[0]
            idle, busy = max(0.0, begin - frontier), max(0.0, end - max(frontier, begin))
            row = rows.setdefault(short, [0, 0.0, 0.0])
            row[0] += 1
            row[1] += busy
            row[2] += idle
            idle_total += idle
            frontier = max(frontier, end)
        span = records[-1][2] - records[0][1]
        print(f"prompt step of {args.prefill_tokens} tokens, {layers} layers of {args.model}: {span:.0f} us from the first kernel's "
              f"start to the last one's end, of which the GPU idles {idle_total:.0f} us")
        print(f"{'kernel':44s} {'launches':>8s} {'busy us':>9s} {'idle before, us':>16s} {'each':>6s}")
        for name, (count, busy, idle) in sorted(rows.items(), key=lambda kv: -kv[1][1]):
            print(f"{name[:44]:44s} {count:8d} {busy:9.1f} {idle:16.1f} {idle / count:6.2f}")
        return 0
    if args.only == "timeline":
        # one captured decode step kernel by kernel: launches, summed durations, and what each adds to the step
        session = DecodeSession(engine, prompts(args.batch), args.warmup + 8)
        for _ in range(args.warmup):
            session.step()
        torch.cuda.synchronize()
        span, rows = step_timeline(session)
        session.close()
        print(f"decode step, batch {args.batch}, {layers} layers of {args.model}, context {prompt_len}: {span:.1f} us by the kernel records")
        print(f"{'kernel':40s} {'launches':>8s} {'duration us':>12s} {'exposed us':>11s} {'share':>6s}")
        for name, (count, duration, exposed) in rows:
            print(f"{name[:40]:40s} {count:8d} {duration:12.1f} {exposed:11.1f} {exposed / span:6.1%}")
        return 0
    if args.only == "decode":
        prefill_ms = float("nan")
    else:
        for _ in range(max(3, args.warmup)):
            prefill_once()
        prefill_ms = statistics.median([prefill_once() for _ in range(1 if args.only == "prefill" else 5)])
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "ms": prefill_ms, "tokens": args.prefill_tokens, "layers": layers}))
        return 0
    pf_flops = prefill_flops(cfg, layers, args.prefill_tokens)
    # one step of a few milliseconds timed alone is the burst case of the tensor peak; the sustained figure beside it
    prefill = {"value": args.prefill_tokens / (prefill_ms / 1e3), "tokens": args.prefill_tokens, "ms": prefill_ms,
               "frac": pf_flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12),
               "frac_of_sustained_peak": pf_flops / (prefill_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12)}

    # ---- decode, device-timed ------------------------------------------------------------------
    family_shares = {}

    def decode_device(batch, steps, warmup, sampler=None, families=False):
        session = DecodeSession(engine, prompts(batch), steps + warmup + 1 + (4 if families else 0))
        for _ in range(warmup):
            session.step()
        torch.cuda.synchronize()
        launches = count_launches(session)
        if families:
            family_shares.update(kernel_families(session) or {})
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if sampler:
            sampler.__enter__()
            time.sleep(0.3)                 # let the first samples arrive before the timed steps
        start.record()
        for _ in range(steps):
            session.step()
        end.record()
        torch.cuda.synchronize()
        if sampler:
            sampler.__exit__()
        ms = start.elapsed_time(end) / steps
        ctx = session.context_length()
        session.close()
        return ms, launches * steps, ctx

    sampler = ClockSampler()
    ms_per_step, launches, ctx_len = decode_device(args.batch, args.steps, args.warmup, sampler)
    value = args.batch / (ms_per_step / 1e3)
    bytes_step = decode_bytes(cfg, layers, args.batch, ctx_len)
    achieved = bytes_step / (ms_per_step / 1e3) / 1e9
    points = {}
    if not args.skip_points and not args.only:
        for b in (1, 64):
            ms_b, _, _ = decode_device(b, max(8, args.steps // 2), args.warmup)
            points[f"decode_b{b}"] = b / (ms_b / 1e3)

    if args.only == "decode":
        print(json.dumps({"only": "decode", "ms_per_step": ms_per_step, "batch": args.batch, "layers": layers,
                          "context": ctx_len, "launches_per_step": launches // args.steps,
                          "hbm_frac": achieved / pk["hbm_gbs"]}))
        return 0

    # ---- decode, end to end through the Python entry point -----------------------------------
    llm = LLM(engine, max_tokens_per_step=max(2048, args.batch), max_seqs=max_batch)
    host_prompts = prompts(args.batch)
    # requests whose prompt is through decode while the others' prompts still run: allow for those tokens, so that
    # no request ends (and the batch shrinks) inside the timed steps
    early = args.batch * -(-prompt_len // llm.scheduler.max_tokens_per_step)
    ids = [llm.submit(p, GenerationConfig(max_new_tokens=args.steps + args.warmup + early + 8, temperature=0.0)) for p in host_prompts]
    while any(llm.poll(i).computed < prompt_len for i in ids):          # prompts in, first token out
        llm.step()
    for _ in range(args.warmup):
        llm.step()
    h2d0, d2h0 = llm.h2d_bytes, llm.d2h_bytes
    import gc
    gc.collect()                      # what the set-up above left behind is collected now, not inside the timed steps
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ended = 0
    for _ in range(args.steps):
        ended += len(llm.step())
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if ended:
        raise RuntimeError(f"{ended} request(s) ended inside the timed end-to-end steps: the batch was not {args.batch} throughout")
    for i in ids:
        llm.cancel(i)
    e2e = {"value": args.batch * args.steps / e2e_s, "unit": "tokens/s",
           "h2d_bytes_per_step": (llm.h2d_bytes - h2d0) // args.steps, "d2h_bytes_per_step": (llm.d2h_bytes - d2h0) // args.steps}

    # The kernel families' shares come from the device's kernel records, i.e. through the profiling interface: last,
    # so that nothing timed above runs with it attached (once used it stays loaded and every launch pays for it).
    decode_device(args.batch, 2, args.warmup, families=True)

    out = {
        "metric": f"decode tokens/s ({args.model[:1].upper() + args.model[1:-1] + args.model[-1:].upper()} shape, bf16, "
                  f"batch {args.batch}, {prompt_len}-token prompts)", "value": value,
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / BASELINE_DECODE_B8 if (args.model, args.batch, prompt_len) == ("qwen2.5-1.5b", 8, 2048) else None,
        "baseline": {"value": BASELINE_DECODE_B8, "unit": "tokens/s", "what": BASELINE_NOTE},
        "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02) seed 0, uniform random token ids", "impl": "ours",
        "config": {"model": args.model + "-shape", "layers": layers, "layers_of_model": full.num_hidden_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_size, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "tied": cfg.tie_word_embeddings, "global_batch": args.batch, "seq_len": prompt_len,
                   "context": context, "decode_context": ctx_len, "page_size": page, "parallelism": "single-gpu",
                   "l2": f"step reads {bytes_step / 1e9:.1f} GB, larger than L2", "peaks": pk["source"]},
        "e2e": e2e, "gpu_launches": launches, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "bytes_per_step": bytes_step},
        "points": points, "families": family_shares or None, "clocks": sampler.summary(),
    }
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen2.5-1.5b", help="a preset's layer shapes (default: the benchmark model)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0: all)")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--only", default="", choices=["", "decode", "prefill", "timeline", "prefill-timeline"],
                    help="run just one timed part and print a short line (for profiler captures)")
    ap.add_argument("--workload", default="decode", choices=["decode", "mixed"])
    ap.add_argument("--requests", type=int, default=64, help="mixed: how many requests")
    ap.add_argument("--min-prompt", type=int, default=128)
    ap.add_argument("--max-prompt", type=int, default=2048)
    ap.add_argument("--new-tokens", type=int, default=128, help="mixed: tokens generated per request")
    ap.add_argument("--chunk", type=int, default=512, help="mixed: token budget of a step (max_tokens_per_step)")
    ap.add_argument("--pool-tokens", type=int, default=0, help="mixed: size the page pool for this many tokens (0: all requests fit)")
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.workload == "mixed":
        return run_mixed(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
