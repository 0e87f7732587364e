"""The engine against the plain implementation, in fp32 and in bf16, cut in every way:
whole; most in one step and the tail token by token; portions of changing size; and mixed
batches over a pool so small that pages are used again."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import helpers
from tests.helpers import (collect, compare_with_plain, make_folder, random_tokens, steps_mixed, steps_portions,
                           steps_prefill_then_decode, steps_whole, tiny_config)

pytestmark = pytest.mark.gpu

LENGTHS = {"a": [5, 11, 17, 70, 133], "b": [1, 9, 40, 70, 150]}
PRECISION = {"float32": "float32", "bfloat16": "bfloat16"}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {key: make_folder(tmp_path_factory, key, "float32") for key in ("a", "b")}


def requests_for(key):
    vocab = tiny_config(key).vocab_size
    return {f"r{i}": random_tokens(n, vocab, 100 * i + n) for i, n in enumerate(LENGTHS[key])}


def engine_for(folder, dtype, max_tokens=1024, page_size=16, guard_pages=False):
    from microllm_rocm_b200.engine.loading import load_engine
    return load_engine(folder, dtype=dtype, page_size=page_size, max_tokens=max_tokens, max_requests=8, guard_pages=guard_pages)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["a", "b"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions"])
def test_one_request_at_a_time(folders, key, dtype, cut):
    reqs = requests_for(key)
    steps = {"whole": steps_whole, "tail": steps_prefill_then_decode, "portions": steps_portions}[cut](reqs)
    got = collect(engine_for(folders[key], dtype), steps)
    compare_with_plain(got, folders[key], reqs, PRECISION[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["a", "b"])
def test_mixed_batches_with_reused_pages(folders, key, dtype):
    vocab = tiny_config(key).vocab_size
    lengths = [60, 33, 150, 90, 47, 128, 75, 20, 101, 64]
    reqs = {f"m{i}": random_tokens(n, vocab, 7 * i + n) for i, n in enumerate(lengths)}
    steps, peak = steps_mixed(reqs, max_live=4, seed=3)
    # a page of a fixed pattern in front of and behind every pool, read back after every step: with a pool this
    # tight the first and the last page are in use all the time, and nothing may be stored beside them
    engine = engine_for(folders[key], dtype, max_tokens=peak, guard_pages=True)
    assert len(engine.cache.guarded) == tiny_config(key).num_hidden_layers
    got = collect(engine, steps)
    engine.cache.check_guards()
    compare_with_plain(got, folders[key], reqs, PRECISION[dtype])
    stats = engine.cache.stats()
    for group in engine.cache.groups:
        assert stats[group]["allocations"] > stats[group]["pages"], "the pool was not tight enough to reuse pages"
    if key == "b":
        assert stats["pages_released_by_window"] > 0


@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_prompts_of_hundreds_of_tokens_reach_the_tensor_memory_kernels(tmp_path_factory, cut):
    """Configuration c (head size 64, window 200 in the second layer): prompt portions of 48 tokens and
    more go through the tcgen05 attention kernel, portions of 256 and more through the CTA-pair product
    with the activation in its epilogue; decoded tokens beside them through the fused few-token kernels."""
    from microllm_rocm_b200.kernels import ops
    folder = make_folder(tmp_path_factory, "c", "float32")
    vocab = tiny_config("c").vocab_size
    reqs = {f"c{i}": random_tokens(n, vocab, 31 * i + n) for i, n in enumerate([300, 520, 77, 260])}
    if cut == "mixed":
        steps, peak = steps_mixed(reqs, max_live=3, seed=5, decode_tail=6)
        # larger portions than the tiny configurations use, so that some reach the 128-row tiles
        engine = engine_for(folder, "bfloat16", max_tokens=peak)
    else:
        steps = {"whole": steps_whole, "tail": steps_prefill_then_decode,
                 "portions": lambda r: steps_portions(r, sizes=(260, 7, 130, 2, 64, 300, 49))}[cut](reqs)
        engine = engine_for(folder, "bfloat16", max_tokens=2048)
    got = collect(engine, steps)
    compare_with_plain(got, folder, reqs, "bfloat16")
    loaded = {source for source, _ in ops._libs}
    assert "attention_tc.cu" in loaded
    if cut != "mixed":
        assert "gemm_tc2.cu" in loaded


@pytest.mark.parametrize("page_size", [16, 64, 128])
def test_head_size_128_with_six_heads_per_kv_head(tmp_path_factory, page_size):
    """Configuration d has the benchmark model's head geometry (head size 128, six query heads on one kv head):
    the tcgen05 attention kernel and the keys-on-M decode kernel at the sizes they are compiled for in the
    benchmark, over pages of 16, 64 and 128 tokens, against the plain implementation."""
    folder = make_folder(tmp_path_factory, "d", "float32")
    vocab = tiny_config("d").vocab_size
    reqs = {f"d{i}": random_tokens(n, vocab, 17 * i + n) for i, n in enumerate([330, 129, 64])}
    engine = engine_for(folder, "bfloat16", max_tokens=2048, page_size=page_size)
    got = collect(engine, steps_prefill_then_decode(reqs, tail=24))
    compare_with_plain(got, folder, reqs, "bfloat16")
    steps, peak = steps_mixed(reqs, max_live=3, seed=9, decode_tail=5)
    live = sum(-(-len(t) // page_size) * page_size for t in reqs.values())       # all three may be live at once
    engine = engine_for(folder, "bfloat16", max_tokens=live, page_size=page_size, guard_pages=True)
    compare_with_plain(collect(engine, steps), folder, reqs, "bfloat16")
    engine.cache.check_guards()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_issued_from_a_recording_give_the_bits_of_layers_called_one_by_one(tmp_path_factory, dtype):
    """Six layers, three with all keys and three with a window: the first layer of a step always runs call by
    call, the first layer of each structure after it is recorded, the others are issued natively from that
    recording with their own weights and pages swapped in.  Steps of every size class (a prompt portion large
    enough for the step-wide table of angles, one for the tensor-memory streaming products, single tokens), in
    one engine with the recording on and in one with it off: the logits must be the same bits."""
    from microllm_rocm_b200.config import Qwen2Config, get_architecture
    from microllm_rocm_b200.engine.loading import load_engine
    from microllm_rocm_b200.engine.step import StepEntry
    from microllm_rocm_b200.weights import write_random_model
    cfg = Qwen2Config.from_dict(dict(helpers.TINY["b"], num_hidden_layers=6, max_window_layers=3))
    folder = str(tmp_path_factory.mktemp("six_layers"))
    write_random_model(get_architecture("Qwen2ForCausalLM"), cfg, 9, folder, "float32")
    a = random_tokens(200, cfg.vocab_size, 1)
    b = random_tokens(120, cfg.vocab_size, 2)

    def run(replay):
        engine = load_engine(folder, dtype=dtype, page_size=16, max_tokens=512, max_requests=4)
        engine.model.replay_layers = replay
        engine.cache.add("a")
        engine.cache.add("b")
        outs = [engine.step([StepEntry("a", a[:100], [0, 50, 99])]),
                engine.step([StepEntry("a", a[100:130], [29]), StepEntry("b", b[:20], [19])]),      # 50 tokens
                engine.step([StepEntry("a", a[130:131], [0]), StepEntry("b", b[20:90], [0, 69])]),   # 71 tokens
                engine.step([StepEntry("a", a[131:132], [0]), StepEntry("b", b[90:91], [0])])]
        for i in range(3):
            outs.append(engine.step([StepEntry("a", a[132 + i:133 + i], [0])]))
        engine.check_device_errors()
        return torch.cat([o.float().cpu() for o in outs]), engine.model.layers_replayed

    want, none = run(False)
    got, replayed = run(True)
    assert none == 0 and replayed == 7 * 3            # per step: layers 2, 4 and 5
    assert torch.isfinite(got).all()
    assert torch.equal(got, want)


def test_benchmark_shape_bf16_tracks_the_true_fp32_path():
    """The Qwen2.5-1.5B shape with random weights (28 layers, the kernels and tile sizes the benchmark runs):
    a prompt portion of 304 tokens beside one of 100, then a decode token beside a portion, then decode
    steps.  No plain implementation at this size; the bf16 path is held against the engine's own true fp32
    path.  bf16 rounds at about six places per layer to 2^-8 relative: over 28 layers the logits' relative
    L2 distance is expected near 0.4 % * sqrt(170) = 5 %, measured 2.3-3.4 %; a wrong tile, a dropped key
    range or a misplaced head shows as tens of percent."""
    from microllm_rocm_b200.config import preset
    from microllm_rocm_b200.engine.loading import random_engine
    from microllm_rocm_b200.engine.step import StepEntry
    cfg = preset("qwen2.5-1.5b")
    gen = torch.Generator().manual_seed(1)
    a = torch.randint(0, cfg.vocab_size, (310,), generator=gen).tolist()
    b = torch.randint(0, cfg.vocab_size, (140,), generator=gen).tolist()

    def run(dtype):
        engine = random_engine(cfg, seed=0, dtype=dtype, page_size=64, max_tokens=1024, max_requests=4, draw_on_device=True)
        engine.cache.add("a")
        engine.cache.add("b")
        outs = [engine.step([StepEntry("a", a[:304], [301, 302, 303]), StepEntry("b", b[:100], [99])]),
                engine.step([StepEntry("a", a[304:305], [0]), StepEntry("b", b[100:135], [34])])]
        for i in range(5):
            outs.append(engine.step([StepEntry("a", a[305 + i:306 + i], [0]), StepEntry("b", b[135 + i:136 + i], [0])]))
        engine.check_device_errors()
        return torch.cat([o.float().cpu() for o in outs])

    want = run("float32")
    torch.cuda.empty_cache()
    got = run("bfloat16")
    assert torch.isfinite(got).all() and got.shape == want.shape == (16, cfg.vocab_size)
    distance = (got - want).norm(dim=1) / want.norm(dim=1)
    assert float(distance.max()) < 0.08, distance.tolist()


@pytest.mark.parametrize("name", ["qwen2.5-7b", "qwen2.5-14b"])
def test_wider_layer_shapes_bf16_tracks_the_true_fp32_path(name):
    """Two layers of the 7B shape (width 3,584, 28/4 heads, intermediate 18,944, untied head) and of the 14B
    shape (width 5,120, 40/8 heads, intermediate 13,824): widths and K ranges that the few-token kernels split
    differently from the benchmark's.  Prompt portions of 600, 100 and 30 tokens, a step that mixes a decode
    token with two portions, decode steps at batch 3; bf16 against the engine's fp32 path."""
    from microllm_rocm_b200.config import preset
    from microllm_rocm_b200.engine.loading import random_engine
    from microllm_rocm_b200.engine.step import StepEntry
    cfg = preset(name, num_hidden_layers=2)
    gen = torch.Generator().manual_seed(1)
    reqs = {k: torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist() for k, n in (("a", 700), ("b", 140), ("c", 40))}

    def run(dtype):
        engine = random_engine(cfg, seed=0, dtype=dtype, page_size=64, max_tokens=2048, max_requests=4, draw_on_device=True)
        for k in reqs:
            engine.cache.add(k)
        outs = [engine.step([StepEntry("a", reqs["a"][:600], [599]), StepEntry("b", reqs["b"][:100], [99])]),
                engine.step([StepEntry("a", reqs["a"][600:601], [0]), StepEntry("b", reqs["b"][100:135], [34]),
                             StepEntry("c", reqs["c"][:30], [29])])]
        for i in range(5):
            outs.append(engine.step([StepEntry("a", reqs["a"][601 + i:602 + i], [0]), StepEntry("b", reqs["b"][135 + i:136 + i], [0]),
                                     StepEntry("c", reqs["c"][30 + i:31 + i], [0])]))
        engine.check_device_errors()
        return torch.cat([o.float().cpu() for o in outs])

    want = run("float32")
    torch.cuda.empty_cache()
    got = run("bfloat16")
    torch.cuda.empty_cache()
    assert torch.isfinite(got).all() and got.shape == want.shape == (20, cfg.vocab_size)
    distance = (got - want).norm(dim=1) / want.norm(dim=1)
    assert float(distance.max()) < 0.05, distance.tolist()      # two layers: measured 1.9 % and 2.2 %


def test_prompt_steps_issued_back_to_back_leave_no_device_error():
    """Four layers of the 7B shape, three prompts of 2,048 tokens stepped one after the other WITHOUT a
    synchronisation in between, so that the host runs far ahead of the GPU and every kernel that may start
    early does.  (In this situation bounded waits inside the tensor-memory attention kernel once ran out: its
    softmax warps shared one barrier for two buffers of P.)  The device error flag must stay clear and the logits
    finite."""
    from microllm_rocm_b200.config import preset
    from microllm_rocm_b200.engine.loading import random_engine
    from microllm_rocm_b200.engine.step import StepEntry
    cfg = preset("qwen2.5-7b", num_hidden_layers=4)
    engine = random_engine(cfg, seed=0, dtype="bfloat16", page_size=64, max_tokens=8 * 2368, max_requests=8, draw_on_device=True)
    gen = torch.Generator().manual_seed(0)
    outs = []
    for _ in range(2):
        for i in range(3):
            toks = torch.randint(0, cfg.vocab_size, (2048,), generator=gen).tolist()
            engine.cache.add(f"p{i}")
            outs.append(engine.step([StepEntry(f"p{i}", toks, [2047])]))
        for i in range(3):
            engine.cache.release(f"p{i}")
    torch.cuda.synchronize()
    engine.check_device_errors()
    assert all(torch.isfinite(o).all() for o in outs)


def test_a_mixed_step_at_a_wide_shape_and_long_context_gives_the_same_bits_every_time():
    """Thirty-two layers of the 14B shape: three requests decode at 8,200 keys beside the last 22 tokens of a prompt and
    the first 2,023 of the next one.  The decoded tokens' attention (the TMA ring kernel, which starts early) and the
    prompt portions' (tensor memory) run side by side on two streams, both bound by memory; in that company a softmax
    warp of the prompt kernel once got a tile ahead of another and completed its phase of the barrier they shared.
    The step, rebuilt from scratch four times, must give the bits of the same step run with one kernel after the
    other, and no device error."""
    from microllm_rocm_b200.config import preset
    from microllm_rocm_b200.engine.loading import random_engine
    from microllm_rocm_b200.engine.step import StepEntry
    from microllm_rocm_b200.kernels import attention
    cfg = preset("qwen2.5-14b", num_hidden_layers=32)
    engine = random_engine(cfg, seed=0, dtype="bfloat16", page_size=64, max_tokens=6 * 8448, max_requests=8, draw_on_device=True)
    gen = torch.Generator().manual_seed(0)
    toks = [torch.randint(0, cfg.vocab_size, (8300,), generator=gen).tolist() for _ in range(5)]
    lens = [8206, 8201, 8197]

    def feed(rid, seq, upto):
        p = engine.cache.length(rid)
        while p < upto:
            n = min(2048, upto - p)
            engine.step([StepEntry(rid, seq[p:p + n], [])])
            p += n

    def scenario(tag):
        ids = [f"{tag}{i}" for i in range(5)]
        for i in ids:
            assert engine.cache.add(i)
        for i in range(3):
            feed(ids[i], toks[i], lens[i])
        feed(ids[3], toks[3], 8170)
        entries = [StepEntry(ids[i], [toks[i][lens[i]]], [0]) for i in range(3)]
        entries.append(StepEntry(ids[3], toks[3][8170:8192], [0, 10, 21]))
        entries.append(StepEntry(ids[4], toks[4][:2023], [0, 1000, 2022]))
        out = engine.step(entries).clone()
        torch.cuda.synchronize()
        engine.check_device_errors()
        for i in ids:
            engine.cache.release(i)
        return out

    attention.CONCURRENT_ATTENTION = False
    try:
        want = scenario("one stream ")
    finally:
        attention.CONCURRENT_ATTENTION = True
    assert torch.isfinite(want).all()
    for trial in range(4):
        got = scenario(f"trial {trial} ")
        assert torch.equal(got, want), (trial, float((got - want).abs().max()))


@pytest.mark.parametrize("key", ["a", "b"])
def test_fp32_is_bit_stable_across_cuts(folders, key):
    """In the fp32 path every summation order is fixed by the token's own position, so the
    four ways of cutting give identical bits, not merely close ones."""
    reqs = requests_for(key)
    base = collect(engine_for(folders[key], "float32"), steps_whole(reqs))
    for other in (steps_prefill_then_decode(reqs), steps_portions(reqs)):
        got = collect(engine_for(folders[key], "float32"), other)
        for k, row in base.items():
            assert torch.equal(row, got[k]), k


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decode_and_first_tokens(folders, dtype):
    """A two-token prompt, then 200 tokens one by one: the first positions of a sequence
    and a long decode across many pages and, for the windowed layers, far past the window."""
    key = "b"
    toks = random_tokens(202, tiny_config(key).vocab_size, 5)
    steps = [{"step": 0, "entries": [{"id": "d", "tokens": toks[:2], "want": [0, 1]}], "end": []}]
    for i in range(2, len(toks)):
        steps.append({"step": i - 1, "entries": [{"id": "d", "tokens": [toks[i]], "want": [0]}],
                      "end": ["d"] if i == len(toks) - 1 else []})
    got = collect(engine_for(folders[key], dtype), steps)
    compare_with_plain(got, folders[key], {"d": toks}, PRECISION[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(folders, tmp_path, dtype):
    """bin/trace_run as a user runs it: a process, JSON lines in, files and `done` lines out."""
    key = "a"
    reqs = {f"t{i}": random_tokens(n, tiny_config(key).vocab_size, n) for i, n in enumerate([70, 45, 100])}
    steps, peak = steps_mixed(reqs, max_live=3, seed=1)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    proc = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", folders[key], "--dtype", dtype,
                           "--out", str(out), "--max-tokens", str(peak)],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
    fed, got = {}, {}
    vocab = tiny_config(key).vocab_size
    for s in steps:
        keys = []
        for e in s["entries"]:
            base = fed.get(e["id"], 0)
            keys += [(e["id"], base + w) for w in e["want"]]
            fed[e["id"]] = base + len(e["tokens"])
        data = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(len(keys), vocab)
        for k, row in zip(keys, data):
            got[k] = torch.from_numpy(row.copy())
    compare_with_plain(got, folders[key], reqs, PRECISION[dtype])
