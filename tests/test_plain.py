"""The plain implementation against the reference's own CPU output (recorded once by
tests/golden/make_golden.py), and against itself where the reference has nothing to say
(window, sampling)."""
import json
import os

import numpy as np
import pytest
import torch

from tests.plain import qwen2_plain as plain

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def golden():
    with open(os.path.join(GOLDEN, "reference_logits.json")) as f:
        return json.load(f)


@pytest.mark.parametrize("key", ["a", "b"])
def test_plain_matches_reference_cpu_logits(golden, key):
    folder = os.path.join(GOLDEN, f"model_{key}")
    weights = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    cfg = plain.read_config(os.path.join(folder, "config.json"))
    for entry in golden[key]:
        ref = np.asarray(entry["last_logits"], dtype=np.float32)
        got = plain.forward_logits(weights, cfg, entry["prompt"])[-1].numpy()
        assert np.abs(got - ref).max() <= 2e-6, (key, entry["prompt"])
        # the reference's greedy continuation, and its logits after the last cached decode step
        gen = entry["generated"]
        assert plain.generate(weights, cfg, entry["prompt"], len(gen)) == gen
        cached = np.asarray(entry["cached_logits"], dtype=np.float32)
        got2 = plain.forward_logits(weights, cfg, entry["prompt"] + gen[:-1])[-1].numpy()
        assert np.abs(got2 - cached).max() <= 2e-6


def test_window_equals_full_inside_the_window_and_differs_beyond():
    torch.manual_seed(0)
    T, NH, NKV, D, W = 12, 4, 2, 8, 5
    q, k, v = torch.randn(T, NH, D), torch.randn(T, NKV, D), torch.randn(T, NKV, D)
    full = plain.causal_gqa_attention(q, k, v, None)
    win = plain.causal_gqa_attention(q, k, v, W)
    assert torch.equal(full[:W], win[:W])
    assert not torch.allclose(full[W:], win[W:])
    # a windowed query equals full attention over just its last W keys
    i = 9
    ref = plain.causal_gqa_attention(q[i - W + 1:i + 1], k[i - W + 1:i + 1], v[i - W + 1:i + 1], None)[-1]
    assert torch.allclose(win[i], ref, atol=1e-6)


def test_rope_position_zero_is_identity_and_pairs_are_split_half():
    x = torch.arange(16, dtype=torch.float32).reshape(1, 2, 8)
    assert torch.equal(plain.rope_split_half(x, [0], 10000.0), x)
    y = plain.rope_split_half(x, [1], 10000.0)
    # pair 0 of head 0 is (x[0], x[4]) rotated by 1 radian
    c, s = np.cos(np.float32(1.0)), np.sin(np.float32(1.0))
    assert abs(float(y[0, 0, 0]) - (0 * c - 4 * s)) < 1e-6
    assert abs(float(y[0, 0, 4]) - (0 * s + 4 * c)) < 1e-6


def test_greedy_takes_first_maximum_and_flags_non_finite():
    assert plain.sample_token([0.5, 2.0, 2.0, -1.0], 0.0, 0, 1, 0) == 1
    assert plain.sample_token([0.5, 2.0, 3.0], 0.7, 1, 1, 0) == 2
    assert plain.sample_token([0.5, float("nan")], 0.0, 0, 1, 0) == -1


def test_sampling_is_seeded_and_follows_the_distribution():
    logits = [0.0, 1.0, 2.0, 0.5]
    a = [plain.sample_token(logits, 0.8, 0, 7, d) for d in range(2000)]
    b = [plain.sample_token(logits, 0.8, 0, 7, d) for d in range(2000)]
    assert a == b
    assert a != [plain.sample_token(logits, 0.8, 0, 8, d) for d in range(2000)]
    p = np.exp(np.asarray(logits) / 0.8)
    p /= p.sum()
    freq = np.bincount(a, minlength=4) / len(a)
    assert np.abs(freq - p).max() < 0.04
    # top-k keeps the k largest; ties at the edge go to the smaller index
    only = {plain.sample_token([1.0, 3.0, 3.0, 3.0, 0.0], 1.0, 2, 3, d) for d in range(200)}
    assert only == {1, 2}


def test_bf16_precision_is_close_to_fp32():
    folder = os.path.join(GOLDEN, "model_b")
    weights = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    cfg = plain.read_config(os.path.join(folder, "config.json"))
    toks = [3, 70, 11, 5, 9, 42]
    a = plain.forward_logits(weights, cfg, toks)
    b = plain.forward_logits(weights, cfg, toks, precision="bfloat16")
    assert 0 < float((a - b).abs().max()) < 0.05 * float(a.abs().max())
