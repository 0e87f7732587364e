"""Shared pieces of the tests: the two tiny configurations, model folders in temporary
places, ways of cutting requests into trace steps, and the comparison with the plain
implementation."""
from __future__ import annotations

import functools
import os
import random
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

from microllm_rocm_b200.config import Qwen2Config, get_architecture
from microllm_rocm_b200.weights import write_random_model
from tests.plain import qwen2_plain as plain

# Two tiny configurations that differ in every size and option: layers, width, heads, kv
# heads and group size, head size, intermediate size (neither a multiple of 128), vocabulary,
# theta, eps, tied/untied head, window off/on.
TINY = {
    "a": dict(vocab_size=256, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1,
              intermediate_size=176, max_position_embeddings=512, rope_theta=10000.0, rms_norm_eps=1e-6,
              tie_word_embeddings=True, use_sliding_window=False, torch_dtype="float32"),
    "b": dict(vocab_size=384, hidden_size=192, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=2,
              intermediate_size=512, max_position_embeddings=512, rope_theta=1e6, rms_norm_eps=1e-5,
              tie_word_embeddings=False, use_sliding_window=True, sliding_window=32, max_window_layers=1,
              torch_dtype="float32"),
    # sized for the tensor-memory kernels (head size 64, prompts of several hundred tokens); used by the tests
    # that must reach them, not by the whole matrix of cuts
    "c": dict(vocab_size=500, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              intermediate_size=392, max_position_embeddings=1024, rope_theta=1e5, rms_norm_eps=1e-6,
              tie_word_embeddings=False, use_sliding_window=True, sliding_window=200, max_window_layers=1,
              torch_dtype="float32"),
    # the benchmark model's head geometry in small: head size 128, one kv head for six query heads, a width that is
    # no multiple of 256, page sizes chosen by the tests
    "d": dict(vocab_size=300, hidden_size=768, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=1,
              intermediate_size=520, max_position_embeddings=1024, rope_theta=1e6, rms_norm_eps=1e-6,
              tie_word_embeddings=True, use_sliding_window=False, torch_dtype="float32"),
}
SEEDS = {"a": 0, "b": 1, "c": 2, "d": 3}

# fp32: engine and plain differ only by summation order.  bf16: both round to bf16 at the
# same places, so what remains is summation order times bf16 steps of the intermediate values.
# Measured over every schedule of the engine tests (printed by compare_with_plain): fp32 worst |error| 8.3e-7,
# bf16 worst 0.0054 of the largest |logit|.  The limits are a few times that.
FP32_ATOL = 4e-6
BF16_REL = 0.015         # of the largest |logit| of the compared rows


def tiny_config(key: str) -> Qwen2Config:
    return Qwen2Config.from_dict(TINY[key])


def make_folder(tmp_path_factory, key: str, storage: str = "float32") -> str:
    folder = str(tmp_path_factory.mktemp(f"tiny_{key}_{storage}"))
    write_random_model(get_architecture("Qwen2ForCausalLM"), tiny_config(key), SEEDS[key], folder, storage)
    return folder


@functools.lru_cache(maxsize=None)
def _plain_inputs(folder: str):
    return (plain.read_safetensors(os.path.join(folder, "model.safetensors")),
            plain.read_config(os.path.join(folder, "config.json")))


_plain_cache: Dict[Tuple[str, tuple, str], torch.Tensor] = {}


def plain_logits(folder: str, tokens: Sequence[int], precision: str = "float32") -> torch.Tensor:
    """[T, V] logits of the plain implementation for one whole sequence (memoised)."""
    key = (folder, tuple(tokens), precision)
    if key not in _plain_cache:
        weights, cfg = _plain_inputs(folder)
        _plain_cache[key] = plain.forward_logits(weights, cfg, list(tokens), precision)
    return _plain_cache[key]


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


# ----------------------------------------------------------------------------- ways of cutting
def steps_whole(requests: Dict[str, List[int]]) -> List[dict]:
    """Each request alone and whole, one step each."""
    out = []
    for i, (rid, toks) in enumerate(requests.items()):
        out.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]})
    return out


def steps_prefill_then_decode(requests: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Most of a request in one step, then its last `tail` tokens one by one."""
    out, step = [], 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        out.append({"step": step, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        step += 1
        for i in range(head, len(toks)):
            out.append({"step": step, "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                        "end": [rid] if i == len(toks) - 1 else []})
            step += 1
        if head == len(toks):
            out[-1]["end"] = [rid]
    return out


def steps_portions(requests: Dict[str, List[int]], sizes=(7, 5, 3, 2, 11, 2, 16, 1, 33, 2)) -> List[dict]:
    """Portions of changing size, down to two tokens (and one)."""
    out, step = [], 0
    for rid, toks in requests.items():
        at, i = 0, 0
        while at < len(toks):
            n = min(sizes[i % len(sizes)], len(toks) - at)
            i += 1
            out.append({"step": step, "entries": [{"id": rid, "tokens": toks[at:at + n], "want": list(range(n))}],
                        "end": [rid] if at + n == len(toks) else []})
            at += n
            step += 1
    return out


def steps_mixed(requests: Dict[str, List[int]], max_live: int = 4, seed: int = 0, decode_tail: int = 12):
    """Up to `max_live` requests at a time; each step gives some of them a portion of their
    prompt and others (those in their tail) one token, and leaves some out.  Returns
    (steps, max_tokens): the most tokens live at once, each request rounded up to 64."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: Dict[str, int] = {}                      # id -> tokens fed so far
    steps, step, peak = [], 0, 0
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.6):
            rid, _ = waiting.pop(0)
            live[rid] = 0
        entries, ended = [], []
        for rid in list(live):
            toks = requests[rid]
            at = live[rid]
            if len(live) > 1 and rng.random() < 0.25:
                continue                             # left out of this step, goes on later
            left = len(toks) - at
            if left <= decode_tail:
                n = 1
            else:
                n = min(rng.choice([2, 3, 5, 8, 13, 21, 40]), left - decode_tail)
            entries.append({"id": rid, "tokens": toks[at:at + n], "want": list(range(n))})
            live[rid] = at + n
            if live[rid] == len(toks):
                ended.append(rid)
        peak = max(peak, sum(-(-n // 64) * 64 for n in live.values() if n > 0))
        if entries:
            steps.append({"step": step, "entries": entries, "end": ended})
            step += 1
        for rid in ended:
            del live[rid]
    return steps, peak


# ----------------------------------------------------------------------------- running and comparing
def collect(engine, steps: List[dict]) -> Dict[Tuple[str, int], torch.Tensor]:
    """Replay `steps`; returns (request, position) -> logits row (CPU fp32)."""
    from microllm_rocm_b200.engine.trace import replay
    fed: Dict[str, int] = {}
    wanted: Dict[int, List[Tuple[str, int]]] = {}
    for msg in steps:
        for e in msg["entries"]:
            base = fed.get(e["id"], 0)
            for w in e.get("want", []):
                wanted.setdefault(msg["step"], []).append((e["id"], base + w))
            fed[e["id"]] = base + len(e["tokens"])
        for rid in msg.get("end", []):
            fed.pop(rid, None)
    out: Dict[Tuple[str, int], torch.Tensor] = {}

    def sink(step, logits):
        keys = wanted[step]
        assert logits.shape[0] == len(keys)
        for k, row in zip(keys, logits):
            assert k not in out, f"{k} produced twice"
            out[k] = row.clone()

    replay(engine, steps, sink)
    engine.cache.check()
    assert not engine.cache.requests, "requests left live after the trace"
    return out


def compare_with_plain(got: Dict[Tuple[str, int], torch.Tensor], folder: str, requests: Dict[str, List[int]],
                       precision: str) -> float:
    """Every (request, position) against the plain implementation; returns the worst error."""
    worst, worst_ratio = 0.0, 0.0
    for rid, toks in requests.items():
        ref = plain_logits(folder, toks, precision)
        rows = torch.stack([got[(rid, p)] for p in range(len(toks))])
        err = (rows - ref).abs()
        if precision == "float32":
            bad = (err > FP32_ATOL + FP32_ATOL * ref.abs())
            tol_desc = f"{FP32_ATOL} abs+rel"
        else:
            bad = err > BF16_REL * ref.abs().max()
            tol_desc = f"{BF16_REL} of max |logit| {float(ref.abs().max()):.4f}"
        if bad.any():
            pos = int(bad.any(dim=1).nonzero()[0])
            raise AssertionError(f"request {rid}: first wrong position {pos} of {len(toks)} "
                                 f"(max err there {float(err[pos].max()):.3e}, tolerance {tol_desc})")
        worst = max(worst, float(err.max()))
        worst_ratio = max(worst_ratio, float(err.max() / ref.abs().max()))
    print(f"[parity] {precision}: worst |error| {worst:.3e} = {worst_ratio:.5f} of the largest |logit|")
    return worst
