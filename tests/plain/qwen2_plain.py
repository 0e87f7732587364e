"""Plain implementation of the Qwen2 dense decoder: whole sequences, no cache, no batching,
one function per part, CPU only.  It shares no code with the engine (it even reads
safetensors files itself) and exists to be obviously right; every test compares the engine
with it.

It rests on the formulas of walkinglabs/microLLM-rocm, cited per function as file:line of
that project, and was compared once with that project's own CPU build on a tiny random model
(tests/golden/make_golden.py; the outputs it made are committed beside it).

`precision="bfloat16"` rounds to bfloat16 at the places where the serving path stores
bfloat16 (weights, inputs of the matrix products, keys/values, the activation) and computes
everything else in fp32, so that the comparison with the bf16 engine can stay tight.
"""
from __future__ import annotations

import json
import math
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


# ----------------------------------------------------------------------------- file reading
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """Minimal reader (container layout: src/io/safetensors.cpp:492-526): u64 header length,
    JSON header, payload.  Returns fp32 CPU tensors."""
    kinds = {"F32": (np.float32, 4), "BF16": (np.uint16, 2), "F16": (np.float16, 2)}
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        payload = f.read()
    out = {}
    for name, d in header.items():
        if name == "__metadata__":
            continue
        np_dtype, _ = kinds[d["dtype"]]
        b, e = d["data_offsets"]
        a = np.frombuffer(payload[b:e], dtype=np_dtype).reshape(d["shape"])
        if d["dtype"] == "BF16":     # widen: bf16 bits are the top half of an fp32
            a = (a.astype(np.uint32) << 16).view(np.float32)
        out[name] = torch.from_numpy(np.array(a, dtype=np.float32))
    return out


def read_config(path: str) -> dict:
    with open(path, "r", encoding="utf-8") as f:
        return json.load(f)


# ----------------------------------------------------------------------------- rounding hook
def _bf16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(torch.float32)


class Rounding:
    """Where the bf16 path stores bf16.  In fp32 precision every hook is the identity."""

    def __init__(self, precision: str):
        if precision not in ("float32", "bfloat16"):
            raise ValueError(precision)
        self.on = precision == "bfloat16"

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return _bf16(x) if self.on else x


# ----------------------------------------------------------------------------- parts
def embedding(table: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """x[t,:] = E[id[t],:]  (src/ops/ops.cpp:581-618; out-of-range ids throw there too)."""
    for i in ids:
        if not 0 <= int(i) < table.shape[0]:
            raise IndexError("token id outside the vocabulary")
    return table[torch.tensor(list(ids), dtype=torch.long)].clone()


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """ss = sum x^2; r = 1/sqrt(ss/W + eps); y = x * r * w   (src/ops/ops.cpp:684-699)."""
    out = torch.empty_like(x)
    width = x.shape[-1]
    for t in range(x.shape[0]):
        ss = (x[t] * x[t]).sum()
        r = 1.0 / torch.sqrt(ss / width + eps)
        out[t] = x[t] * r * weight
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x W^T (+ b) with W stored [out, in] as in the checkpoint; the reference transposes
    at load and multiplies x[M,K] W[K,N] (src/model/model.cpp:332-335, mapping :1939-1961)."""
    y = x @ weight.t()
    return y + bias if bias is not None else y


def rope_split_half(x: torch.Tensor, positions: Sequence[int], theta: float) -> torch.Tensor:
    """x [T, heads, D].  For pair i < D/2: angle = float(pos) * theta^(-2 i / D) in fp32,
    out[i] = x[i] cos - x[i+D/2] sin, out[i+D/2] = x[i] sin + x[i+D/2] cos
    (src/ops/ops.cpp:861-879; angle expression :863-865)."""
    T, H, D = x.shape
    half = D // 2
    i = np.arange(half, dtype=np.float32)
    inv = np.power(np.float32(theta), (np.float32(-2.0) * i) / np.float32(D), dtype=np.float32)
    out = x.clone()
    for t in range(T):
        angle = (np.float32(positions[t]) * inv).astype(np.float32)
        c = torch.from_numpy(np.cos(angle)).to(x.dtype)
        s = torch.from_numpy(np.sin(angle)).to(x.dtype)
        a, b = x[t, :, :half], x[t, :, half:]
        out[t, :, :half] = a * c - b * s
        out[t, :, half:] = a * s + b * c
    return out


def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int]) -> torch.Tensor:
    """q [T, NH, D], k/v [T, NKV, D] -> [T, NH, D].  Head h uses kv head h // (NH/NKV); for
    query i the keys j <= i (and j >= i - window + 1 for a windowed layer) get
    s_j = dot(q_i, k_j) * (1/sqrt(D)), p = softmax(s), o = sum_j p_j v_j, with the
    probability normalised before it multiplies v (src/ops/ops.cpp:2343-2384).  The window
    is this engine's own extension: the reference rejects it (src/model/huggingface.cpp:159-161)."""
    T, NH, D = q.shape
    NKV = k.shape[1]
    repeats = NH // NKV
    scale = 1.0 / math.sqrt(float(D))
    out = torch.zeros_like(q)
    for h in range(NH):
        g = h // repeats
        for i in range(T):
            lo = 0 if window is None else max(0, i - window + 1)
            keys = k[lo:i + 1, g]                       # [n, D]
            s = (keys @ q[i, h]) * scale
            s = s - s.max()
            p = torch.exp(s)
            p = p / p.sum()
            out[i, h] = p @ v[lo:i + 1, g]
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """g * sigmoid(g) * u with the two-branch sigmoid (src/ops/ops.cpp:72-76, 760-785)."""
    pos = 1.0 / (1.0 + torch.exp(-gate.clamp(min=0)))
    e = torch.exp(gate.clamp(max=0))
    neg = e / (1.0 + e)
    sig = torch.where(gate >= 0, pos, neg)
    return gate * sig * up


# ----------------------------------------------------------------------------- the model
def layer_window(cfg: dict, layer: int) -> Optional[int]:
    """Layer l is windowed iff use_sliding_window and l >= max_window_layers (this engine's
    reading of the config keys; the reference never reads them)."""
    if cfg.get("use_sliding_window", False) and cfg.get("sliding_window") and layer >= cfg.get("max_window_layers", 0):
        return int(cfg["sliding_window"])
    return None


def block(x, w, prefix, cfg, positions, window, rnd):
    """x + attn(norm(x)), then + mlp(norm(.))  (src/model/model.cpp:834-849)."""
    H = cfg["hidden_size"]
    NH, NKV = cfg["num_attention_heads"], cfg.get("num_key_value_heads", cfg["num_attention_heads"])
    D = cfg.get("head_dim") or H // NH
    eps = cfg["rms_norm_eps"]
    T = x.shape[0]
    h = rnd(rms_norm(x, w[prefix + "input_layernorm.weight"], eps))
    a = prefix + "self_attn."
    q = linear(h, w[a + "q_proj.weight"], w.get(a + "q_proj.bias")).view(T, NH, D)
    k = linear(h, w[a + "k_proj.weight"], w.get(a + "k_proj.bias")).view(T, NKV, D)
    v = linear(h, w[a + "v_proj.weight"], w.get(a + "v_proj.bias")).view(T, NKV, D)
    q = rnd(rope_split_half(q, positions, cfg["rope_theta"]))
    k = rnd(rope_split_half(k, positions, cfg["rope_theta"]))
    v = rnd(v)
    o = rnd(causal_gqa_attention(q, k, v, window)).reshape(T, NH * D)
    x = x + linear(o, w[a + "o_proj.weight"])
    h = rnd(rms_norm(x, w[prefix + "post_attention_layernorm.weight"], eps))
    m = prefix + "mlp."
    gate = rnd(linear(h, w[m + "gate_proj.weight"]))
    up = rnd(linear(h, w[m + "up_proj.weight"]))
    act = rnd(swiglu(gate, up))
    return x + linear(act, w[m + "down_proj.weight"])


def forward_logits(weights: Dict[str, torch.Tensor], cfg: dict, tokens: Sequence[int],
                   precision: str = "float32", dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Logits [T, V] for every position of one whole sequence (positions 0..T-1)
    (src/model/model.cpp:1043-1087)."""
    rnd = Rounding(precision)
    w = {}
    for name, t in weights.items():
        t = t.to(torch.float32)
        if rnd.on and t.dim() >= 2:
            t = _bf16(t)                         # matrices and tables live in bf16 on that path
        w[name] = t.to(dtype)
    positions = list(range(len(tokens)))
    x = embedding(w["model.embed_tokens.weight"], tokens)
    for l in range(cfg["num_hidden_layers"]):
        x = block(x, w, f"model.layers.{l}.", cfg, positions, layer_window(cfg, l), rnd)
    x = rnd(rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"]))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return linear(x, head)


# ----------------------------------------------------------------------------- sampling
GOLDEN = 0x9E3779B97F4A7C15
MASK = (1 << 64) - 1


def uniform_from(seed: int, draw: int) -> float:
    """SplitMix64 of (seed + GOLDEN * (draw + 1)); 53 bits -> [0, 1).  This engine's own
    definition: the reference draws from std::mt19937_64 through std::discrete_distribution
    (src/inference/generator.cpp:66-68), which no other library reproduces."""
    z = (seed + GOLDEN * (draw + 1)) & MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
    z ^= z >> 31
    return (z >> 11) * (1.0 / 9007199254740992.0)


def sample_token(logits: Sequence[float], temperature: float, top_k: int, seed: int, draw: int) -> int:
    """Greedy when temperature == 0 or top_k == 1: first maximum (src/inference/generator.cpp:46-49).
    Otherwise candidates = top_k largest (all if 0; ties at the edge to the smaller index),
    weight = exp(double(l/T - l_max/T)) with fp32 division and subtraction (generator.cpp:59-64),
    first candidate in index order whose running sum exceeds u * total."""
    l = np.asarray(logits, dtype=np.float32)
    if l.size == 0:
        raise ValueError("cannot sample empty logits")
    if not np.isfinite(temperature) or temperature < 0:
        raise ValueError("temperature must be finite and non-negative")
    if top_k < 0 or top_k > l.size:
        raise ValueError("top_k is outside the vocabulary")
    if not np.all(np.isfinite(l)):
        return -1
    if temperature == 0 or top_k == 1:
        return int(np.argmax(l))
    k = l.size if top_k == 0 else top_k
    order = sorted(range(l.size), key=lambda i: (-float(l[i]), i))[:k]
    cand = sorted(order)
    T = np.float32(temperature)
    mx = np.float32(l.max()) / T
    weights = [math.exp(float(np.float32(l[i] / T) - mx)) for i in cand]
    total = 0.0
    for wgt in weights:
        total += wgt
    target = uniform_from(seed, draw) * total
    running = 0.0
    for i, wgt in zip(cand, weights):
        running += wgt
        if running > target:
            return int(i)
    return int(cand[-1])


def generate(weights, cfg, prompt: Sequence[int], max_new_tokens: int, temperature: float = 0.0, top_k: int = 0,
             seed: int = 1, stop_tokens: Sequence[int] = (), precision: str = "float32") -> List[int]:
    """Recompute the whole sequence for every new token (no cache); a stop token is appended
    and then ends the run (src/inference/generator.cpp:129-149)."""
    seq = list(prompt)
    out: List[int] = []
    for step in range(max_new_tokens):
        logits = forward_logits(weights, cfg, seq, precision)[-1]
        token = sample_token(logits.numpy(), temperature, top_k, seed, step)
        out.append(token)
        seq.append(token)
        if token in stop_tokens:
            break
    return out
