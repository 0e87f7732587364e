"""Generation through the Python entry point and the command line: greedy and seeded
temperature sampling against the plain implementation, many requests at once, and a pool so
small that requests are preempted and recomputed."""
import json
import os
import subprocess
import sys

import pytest
import torch

from tests.helpers import make_folder, plain_logits, random_tokens, tiny_config
from tests.plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {key: make_folder(tmp_path_factory, key, "float32") for key in ("a", "b")}


def plain_generate(folder, prompt, n, **kw):
    weights = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    cfg = plain.read_config(os.path.join(folder, "config.json"))
    return plain.generate(weights, cfg, prompt, n, **kw)


def llm_for(folder, dtype, **kw):
    from microllm_rocm_b200 import LLM
    return LLM(folder, dtype=dtype, page_size=16, **kw)


@pytest.mark.parametrize("key,lengths,new", [("a", [5, 11, 17], 8), ("b", [1, 9, 40, 70], 12)])
def test_greedy_generation_fp32_equals_plain(folders, key, lengths, new):
    from microllm_rocm_b200 import GenerationConfig
    vocab = tiny_config(key).vocab_size
    prompts = [random_tokens(n, vocab, n) for n in lengths]
    llm = llm_for(folders[key], "float32", max_tokens=1024)
    got = llm.generate(prompts, GenerationConfig(max_new_tokens=new, temperature=0.0))
    for p, g in zip(prompts, got):
        assert g == plain_generate(folders[key], p, new)
    # one by one gives the same tokens as all together
    llm2 = llm_for(folders[key], "float32", max_tokens=1024)
    assert [llm2.generate([p], GenerationConfig(max_new_tokens=new, temperature=0.0))[0] for p in prompts] == got


def test_seeded_temperature_sampling_fp32_equals_plain(folders):
    from microllm_rocm_b200 import GenerationConfig
    key = "b"
    prompts = [random_tokens(n, tiny_config(key).vocab_size, n) for n in [1, 9, 40, 70]]
    cfg = GenerationConfig(max_new_tokens=12, temperature=0.8, seed=7)
    got = llm_for(folders[key], "float32", max_tokens=1024).generate(prompts, cfg)
    for p, g in zip(prompts, got):
        assert g == plain_generate(folders[key], p, 12, temperature=0.8, seed=7)
    again = llm_for(folders[key], "float32", max_tokens=1024).generate(prompts, cfg)
    assert again == got
    other = llm_for(folders[key], "float32", max_tokens=1024).generate(
        prompts, GenerationConfig(max_new_tokens=12, temperature=0.8, seed=8))
    assert other != got
    topk = llm_for(folders[key], "float32", max_tokens=1024).generate(
        prompts[:2], GenerationConfig(max_new_tokens=6, temperature=1.3, top_k=4, seed=3))
    for p, g in zip(prompts, topk):
        assert g == plain_generate(folders[key], p, 6, temperature=1.3, top_k=4, seed=3)


@pytest.mark.parametrize("key", ["a", "b"])
def test_greedy_generation_bf16_follows_the_plain_logits(folders, key):
    """bf16 tokens may leave the fp32 ones at a near tie; what must hold is that every chosen
    token is (within bf16 error) a maximum of the plain bf16 logits for the same prefix."""
    from microllm_rocm_b200 import GenerationConfig
    prompts = [random_tokens(n, tiny_config(key).vocab_size, 3 * n) for n in [3, 20, 45]]
    got = llm_for(folders[key], "bfloat16", max_tokens=1024).generate(prompts, GenerationConfig(max_new_tokens=10, temperature=0.0))
    for p, g in zip(prompts, got):
        assert len(g) == 10
        ref = plain_logits(folders[key], p + g[:-1], "bfloat16")[len(p) - 1:]
        for i, t in enumerate(g):
            assert float(ref[i].max() - ref[i, t]) <= 0.03 * float(ref[i].abs().max()), (i, t)


def test_tight_pool_preempts_and_still_generates_the_same_tokens(folders):
    from microllm_rocm_b200 import GenerationConfig
    key = "b"
    prompts = [random_tokens(n, tiny_config(key).vocab_size, 11 * n) for n in [30, 28, 33, 25]]
    cfg = GenerationConfig(max_new_tokens=40, temperature=0.0)
    want = llm_for(folders[key], "float32", max_tokens=2048).generate(prompts, cfg)
    tight = llm_for(folders[key], "float32", num_pages=10, max_tokens_per_step=24)      # 160 tokens for 4 x ~70
    got = tight.generate(prompts, cfg)
    assert got == want
    m = tight.metrics()
    assert m["preemptions"] > 0 and m["cache"]["full"]["used"] == 0
    tight.engine.cache.check()


def test_stop_tokens_and_requests_over_time(folders):
    from microllm_rocm_b200 import GenerationConfig
    key = "a"
    llm = llm_for(folders[key], "float32", max_tokens=512)
    p = random_tokens(12, tiny_config(key).vocab_size, 1)
    full = plain_generate(folders[key], p, 10)
    stop = full[4]
    a = llm.submit(p, GenerationConfig(max_new_tokens=10, temperature=0.0, stop_tokens=(stop,)))
    llm.step()
    b = llm.submit(p, GenerationConfig(max_new_tokens=3, temperature=0.0))       # arrives one step later
    while llm.has_work():
        llm.step()
    assert llm.poll(a).generated == full[:full.index(stop) + 1]
    assert llm.poll(b).generated == full[:3]
    assert llm.poll(a).first_token_step == 0 and llm.poll(b).arrival_step == 1 and llm.poll(b).first_token_step == 1
    assert llm.poll(b).completion_step == 3
def test_command_line(folders, tmp_path):
    key = "a"
    prompt = random_tokens(9, tiny_config(key).vocab_size, 2)
    logits_file, cached_file = tmp_path / "l.f32", tmp_path / "c.f32"
    cmd = [sys.executable, os.path.join(ROOT, "bin", "microllm_hf_infer"), "--config", os.path.join(folders[key], "config.json"),
           "--weights", os.path.join(folders[key], "model.safetensors"), "--tokens", ",".join(map(str, prompt)),
           "--device", "cuda", "--workload", "both", "--new-tokens", "4", "--logits-output", str(logits_file),
           "--cache-logits-output", str(cached_file), "--top-k", "3"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    info = json.loads(proc.stdout.strip().splitlines()[-1])
    want = plain_generate(folders[key], prompt, 4)
    assert info["status"] == "pass" and info["generated_tokens"] == want and info["compute_dtype"] == "float32"
    import numpy as np
    last = torch.from_numpy(np.fromfile(logits_file, dtype="<f4"))
    assert torch.allclose(last, plain_logits(folders[key], prompt)[-1], atol=2e-5)
    assert [t["token"] for t in info["top_logits"]] == torch.topk(last, 3).indices.tolist()
    cached = torch.from_numpy(np.fromfile(cached_file, dtype="<f4"))
    assert torch.allclose(cached, plain_logits(folders[key], prompt + want[:-1])[-1], atol=2e-5)
    # --prefill-logits full: the head at every prompt position, whole prompt or token by token
    for mode in ("full", "token"):
        full_file = tmp_path / f"full_{mode}.f32"
        cmd = [sys.executable, os.path.join(ROOT, "bin", "microllm_hf_infer"), "--model", folders[key], "--tokens",
               ",".join(map(str, prompt)), "--workload", "prefill", "--prefill-logits", "full", "--cache-prefill-mode", mode,
               "--logits-output", str(full_file), "--top-k", "3"]
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        info = json.loads(proc.stdout.strip().splitlines()[-1])
        every = torch.from_numpy(np.fromfile(full_file, dtype="<f4")).view(len(prompt), -1)
        assert torch.allclose(every, plain_logits(folders[key], prompt), atol=2e-5)
        assert info["prefill_logits_mode"] == "full" and [t["token"] for t in info["top_logits"]] == torch.topk(every[-1], 3).indices.tolist()
    # continuous workload: delayed arrivals over two slots
    cmd = [sys.executable, os.path.join(ROOT, "bin", "microllm_hf_infer"), "--model", folders[key], "--workload", "continuous",
           "--tokens", ",".join(map(str, prompt)), "--continuous-slots", "2", "--continuous-prompt-lengths", "4,9,6",
           "--continuous-new-token-lengths", "3,2,4", "--continuous-arrival-steps", "0,1,1"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    info = json.loads(proc.stdout.strip().splitlines()[-1])
    assert info["generated_tokens"] == [plain_generate(folders[key], prompt[:n], k) for n, k in ((4, 3), (9, 2), (6, 4))]
    assert info["admissions"] == 3


def test_command_line_writes_a_tensor_trace_of_the_prompt_step(folders, tmp_path):
    """--trace-output: one record per intermediate tensor of the prompt's step, in the reference's layout; the
    residual stream after the last layer plus its pending delta, normed, is what the logits come from, so the
    records can be checked against the plain implementation's own intermediate values."""
    key = "a"
    prompt = random_tokens(9, tiny_config(key).vocab_size, 2)
    trace = tmp_path / "trace.jsonl"
    cmd = [sys.executable, os.path.join(ROOT, "bin", "microllm_hf_infer"), "--model", folders[key], "--tokens",
           ",".join(map(str, prompt)), "--workload", "prefill", "--trace-output", str(trace), "--trace-max-elements", "7"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    info = json.loads(proc.stdout.strip().splitlines()[-1])
    records = [json.loads(line) for line in open(trace)]
    layers = tiny_config(key).num_hidden_layers
    assert info["trace_record_count"] == len(records) == 1 + 2 * layers + 2
    assert [r["name"] for r in records][:2] == ["embedding", "run0.layer0.residual"] and records[-1]["name"] == "logits"
    assert all(r["schema_version"] == 1 and len(r["values"]) <= 7 and r["statistics"]["finite_count"] == r["statistics"]["numel"] for r in records)
    weights = plain.read_safetensors(os.path.join(folders[key], "model.safetensors"))
    emb = plain.embedding(weights["model.embed_tokens.weight"], prompt)
    assert records[0]["shape"] == list(emb.shape)
    assert torch.allclose(torch.tensor(records[0]["values"], dtype=torch.float64), emb.reshape(-1)[:7].double(), atol=1e-6)
    assert abs(records[0]["statistics"]["l2_norm"] - float(emb.double().norm())) < 1e-4
    logits = plain_logits(folders[key], prompt)[-1]
    assert torch.allclose(torch.tensor(records[-1]["values"], dtype=torch.float64), logits[:7].double(), atol=2e-5)


def test_command_line_stops_on_the_configuration_eos(folders, tmp_path):
    """--stop-on-eos true makes config.json's eos_token_id a stop token: the generation ends with it."""
    import shutil
    key = "a"
    prompt = random_tokens(9, tiny_config(key).vocab_size, 2)
    want = plain_generate(folders[key], prompt, 6)
    folder = tmp_path / "with_eos"
    shutil.copytree(folders[key], folder)
    raw = json.load(open(folder / "config.json"))
    raw["eos_token_id"] = want[2]                       # the third token the model will generate
    json.dump(raw, open(folder / "config.json", "w"))
    base = [sys.executable, os.path.join(ROOT, "bin", "microllm_hf_infer"), "--model", str(folder), "--tokens",
            ",".join(map(str, prompt)), "--workload", "decode", "--new-tokens", "6"]
    proc = subprocess.run(base + ["--stop-on-eos", "true"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    info = json.loads(proc.stdout.strip().splitlines()[-1])
    cut = want[:want.index(want[2]) + 1]
    assert info["generated_tokens"] == cut and info["stop_on_eos"] == [want[2]]
    proc = subprocess.run(base, capture_output=True, text=True, timeout=600)                    # without the flag eos is just a token
    assert json.loads(proc.stdout.strip().splitlines()[-1])["generated_tokens"] == want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_decode_steps_equal_launched_ones(folders, dtype):
    """Steady decoding replays a captured step whose inputs live on the device; it must select
    the tokens that kernel-by-kernel steps select, across page edges, past the window, with
    greedy and sampled requests side by side, and when requests finish at different times."""
    from microllm_rocm_b200 import GenerationConfig
    key = "b"
    prompts = [random_tokens(n, tiny_config(key).vocab_size, 5 * n) for n in [3, 30, 61]]
    cfgs = [GenerationConfig(max_new_tokens=90, temperature=0.0), GenerationConfig(max_new_tokens=40, temperature=0.9, seed=5),
            GenerationConfig(max_new_tokens=70, temperature=0.7, top_k=8, seed=9)]
    plain_path = llm_for(folders[key], dtype, max_tokens=1024, cuda_graphs=False)
    want = plain_path.generate(prompts, cfgs)
    graphed = llm_for(folders[key], dtype, max_tokens=1024)
    got = graphed.generate(prompts, cfgs)
    assert graphed.graph_steps > 50 and plain_path.graph_steps == 0
    assert graphed.prepared_steps > 40               # most steady steps found pages, tables and plan seen to beforehand
    if dtype == "float32":
        assert got == want
    else:
        # bf16 sums depend on how the keys were split over CTAs, which the captured step and the
        # launched one choose differently: near ties may fall the other way.  The greedy request
        # must still pick (near) maxima of the plain bf16 logits for its own prefix.
        assert [len(g) for g in got] == [len(w) for w in want]
        ref = plain_logits(folders[key], prompts[0] + got[0][:-1], "bfloat16")[len(prompts[0]) - 1:]
        for i, t in enumerate(got[0]):
            assert float(ref[i].max() - ref[i, t]) <= 0.03 * float(ref[i].abs().max()), (i, t)
    graphed.engine.cache.check()


def test_captured_decode_step_of_64_requests_rotates_with_the_present_positions(folders):
    """64 requests decoding in bf16: the step is large enough for the path that makes one table of the step's
    sines and cosines.  A captured step lives on from one replay to the next while the positions move on the
    device, so whatever it computes from the positions must be computed inside every replay.  Two engines are fed
    the SAME tokens, one through replays of a captured step, one through plain steps; their caches (the rotated
    keys every step stored) must agree, and so must the tokens they select."""
    from microllm_rocm_b200.engine.decode_graph import DecodeGraphPool
    from microllm_rocm_b200.engine.loading import load_engine
    from microllm_rocm_b200.engine.step import StepEntry
    from microllm_rocm_b200.kernels import ops
    from microllm_rocm_b200.kernels.build import LaunchCounter
    from microllm_rocm_b200 import GenerationConfig
    key, batch, steps = "b", 64, 7
    vocab = tiny_config(key).vocab_size
    prompts = [random_tokens(3 + (i * 7) % 40, vocab, 1000 + i) for i in range(batch)]
    forced = [[random_tokens(steps + 1, vocab, 5000 + i)[s] for i in range(batch)] for s in range(steps + 1)]
    ids = [f"q{i}" for i in range(batch)]

    def fresh():
        engine = load_engine(folders[key], dtype="bfloat16", page_size=16, max_tokens=batch * 64, max_requests=batch)
        for rid, p in zip(ids, prompts):
            assert engine.cache.add(rid)
        engine.step([StepEntry(rid, p, []) for rid, p in zip(ids, prompts)])
        return engine

    # plain steps: forced tokens in, selected tokens out
    plain_engine = fresh()
    picked = torch.empty(batch, dtype=torch.int32, device="cuda")
    want_tokens = []
    for s in range(steps):
        logits = plain_engine.step([StepEntry(rid, [forced[s][i]], [0]) for i, rid in enumerate(ids)])
        ops.argmax_rows(logits, picked)
        want_tokens.append(picked.tolist())

    # the same through a captured step
    engine = fresh()
    cache = engine.cache
    lengths = [cache.length(rid) for rid in ids]
    for rid, n in zip(ids, lengths):
        assert cache.reserve(rid, n + 1)
    pool = DecodeGraphPool(engine)
    graph = pool.get(ids, headroom_tokens=steps + 1)
    greedy = GenerationConfig(max_new_tokens=steps + 1, temperature=0.0)
    state = (forced[0], lengths, [greedy] * batch, [0] * batch)
    graph.load(ids, *state)
    before = LaunchCounter.own
    pool.ensure_captured(graph)
    graph.load(ids, *state)
    got_tokens = []
    for s in range(steps):
        for i, rid in enumerate(ids):
            assert cache.reserve(rid, lengths[i] + 1)
        graph.refresh_tables()
        if s:
            graph.upload_tokens(forced[s])
        graph.replay()
        got_tokens.append(graph.read_tokens())
        for i, rid in enumerate(ids):
            lengths[i] += 1
            cache.commit(rid, lengths[i])
    engine.check_device_errors()
    # same requests added in the same order to pools of the same size: the two caches use the same pages
    assert [cache.requests[r].tables for r in ids] == [plain_engine.cache.requests[r].tables for r in ids]
    for name, pages in cache.kv_storage.items():
        other = plain_engine.cache.kv_storage[name]
        for i, rid in enumerate(ids):
            for group, table in cache.requests[rid].tables.items():
                if cache.entry_group[name] != group:
                    continue
                for block, page in enumerate(table):
                    if page < 0:
                        continue
                    n = min(16, lengths[i] - 16 * block)
                    a, b = pages[page, :, :, :n].float(), other[page, :, :, :n].float()
                    assert torch.allclose(a, b, atol=2e-2, rtol=2e-2), (name, rid, block, float((a - b).abs().max()))
    agree = sum(g == w for gs, ws in zip(got_tokens, want_tokens) for g, w in zip(gs, ws))
    assert agree >= 0.97 * batch * steps, agree          # bf16 near-ties may fall the other way; stale angles would not leave 97 %


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_raised_device_flag_ends_the_step_with_an_error(folders, dtype):
    """Every kernel of a step reports through ONE device flag (a token without a page, a bounded wait of a
    tensor-memory kernel that ran out).  Whatever raised it, the step that reads it must fail instead of handing
    out tokens, both when it launches kernel by kernel and when it replays a captured decode step, and the flag
    must be clear again afterwards."""
    from microllm_rocm_b200 import GenerationConfig
    from microllm_rocm_b200.engine.step import StepError
    llm = llm_for(folders["a"], dtype, max_tokens=256)
    rid = llm.submit(random_tokens(9, tiny_config("a").vocab_size, 4), GenerationConfig(max_new_tokens=8, temperature=0.0))
    llm.engine.error_flag.fill_(43)                     # as a bounded wait inside a product would
    with pytest.raises(StepError, match="bounded wait"):
        llm.step()                                      # the prompt's step, launched kernel by kernel
    assert int(llm.engine.error_flag.item()) == 0
    # the failed step's request has ended and holds nothing; the engine goes on
    assert llm.poll(rid).state.name == "CANCELLED" and not llm.has_work()
    assert llm.metrics()["cache"]["live_requests"] == 0
    rid = llm.submit(random_tokens(9, tiny_config("a").vocab_size, 4), GenerationConfig(max_new_tokens=8, temperature=0.0))
    other = llm.submit(random_tokens(5, tiny_config("a").vocab_size, 5), GenerationConfig(max_new_tokens=8, temperature=0.0))
    while llm.graph_steps < 1:
        llm.step()
    llm.engine.error_flag.fill_(2)                      # as a kernel that met a token without a page would
    with pytest.raises(StepError, match="page"):
        llm.step()                                      # a replayed decode step (if it was launched early it ran before the
        llm.step()                                      # flag was raised: then the one after it reports)
    assert int(llm.engine.error_flag.item()) == 0
    assert llm.poll(rid).state.name == "CANCELLED" and llm.poll(other).state.name == "CANCELLED" and not llm.has_work()
    llm.engine.cache.check()
    # a failure while a step issued ahead is on its way: both steps' requests end, a later request is served whole
    prompts = [random_tokens(n, tiny_config("a").vocab_size, n) for n in (40, 33, 21)]
    fresh = llm_for(folders["a"], dtype, max_tokens=256)
    want = fresh.generate([prompts[2]], GenerationConfig(max_new_tokens=6, temperature=0.0))[0]
    small = llm_for(folders["a"], dtype, max_tokens=256, max_tokens_per_step=16, cuda_graphs=False)
    ids = [small.submit(p, GenerationConfig(max_new_tokens=6, temperature=0.0)) for p in prompts[:2]]
    small.step()
    assert small._inflight is not None                  # a step is on its way on top of the one just collected
    small.engine.error_flag.fill_(43)                   # (the step on its way has copied the flag already: the next one reports it)
    with pytest.raises(StepError, match="bounded wait"):
        small.step()
        small.step()
    assert small._inflight is None and not small.has_work()
    assert all(small.poll(i).state.name == "CANCELLED" for i in ids)
    small.engine.cache.check()
    assert small.metrics()["cache"]["live_requests"] == 0
    assert small.generate([prompts[2]], GenerationConfig(max_new_tokens=6, temperature=0.0))[0] == want


def test_the_driver_entry_point_generates_and_compares():
    """`__graft_entry__.smoke()` is what runs first on a fresh GPU box: it must import, generate a few tokens
    in fp32 and bf16 and agree with the plain implementation."""
    import __graft_entry__ as entry
    entry.smoke()


def test_steps_prepared_ahead_give_way_to_cancels_arrivals_and_ends(folders):
    """While a captured decode step runs, the host prepares the same requests' next step.  A cancel, a new
    request or a request that ends must make it fall back to the scheduler's decision: every surviving request
    gets exactly the tokens it gets alone, the pool ends empty."""
    from microllm_rocm_b200 import GenerationConfig
    key = "b"
    vocab = tiny_config(key).vocab_size
    prompts = [random_tokens(n, vocab, 3 * n + 1) for n in [9, 40, 22, 17]]
    cfgs = [GenerationConfig(max_new_tokens=n, temperature=0.0) for n in [60, 25, 80, 30]]
    alone = llm_for(folders[key], "float32", max_tokens=2048, cuda_graphs=False)
    want = [alone.generate([p], c)[0] for p, c in zip(prompts, cfgs)]
    llm = llm_for(folders[key], "float32", max_tokens=2048)
    ids = [llm.submit(p, c) for p, c in zip(prompts[:3], cfgs[:3])]
    for _ in range(12):
        llm.step()
    assert llm.prepared_steps >= 8 and llm.launched_early >= 8
    assert llm._launched is not None                       # the next replay is on its way already, with all three
    assert llm.cancel(ids[1])                              # one of the three leaves in the middle of steady decoding
    for _ in range(6):
        llm.step()
    ids.append(llm.submit(prompts[3], cfgs[3]))            # a new one arrives: a prompt step between captured ones
    while llm.has_work():
        llm.step()
    for i in (0, 2, 3):
        assert list(llm.poll(ids[i]).generated) == want[i], i
    got = list(llm.poll(ids[1]).generated)
    assert got == want[1][:len(got)] and len(got) < len(want[1])
    assert llm.metrics()["cache"]["live_requests"] == 0
    llm.engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_issued_ahead_of_their_predecessors_tokens_change_nothing(folders, dtype):
    """Steps that hold prompt portions are planned and issued while the step before them still runs; the tokens
    that step selects reach their places through a kernel on the device.  Greedy and sampled requests, stop tokens
    (a void row in the step issued ahead), a small token budget: with and without the look-ahead every request
    gets the same tokens, in fp32 those it gets alone."""
    import random
    from microllm_rocm_b200 import GenerationConfig
    key = "b"
    cfg = tiny_config(key)
    rng = random.Random(5)
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in [70, 3, 41, 120, 9, 64, 33, 17]]
    alone = llm_for(folders[key], dtype, max_tokens=4096, cuda_graphs=False)
    alone.lookahead = False
    probe = alone.generate([prompts[0]], GenerationConfig(max_new_tokens=12, temperature=0.0))[0]
    cfgs = [GenerationConfig(max_new_tokens=12 + 3 * i, temperature=0.0 if i % 2 == 0 else 0.8, seed=i,
                             stop_tokens=(probe[5],) if i == 0 else ()) for i in range(len(prompts))]
    results = []
    for ahead in (False, True):
        llm = llm_for(folders[key], dtype, max_tokens=4096, max_tokens_per_step=48, cuda_graphs=False)
        llm.lookahead = ahead
        results.append(llm.generate(prompts, cfgs))
        assert (llm.lookahead_steps > 10) == ahead
        assert llm.metrics()["cache"]["live_requests"] == 0
        llm.engine.cache.check()
    assert results[0] == results[1]
    assert results[1][0] == probe[:probe.index(probe[5]) + 1]      # ended on its stop token
    if dtype == "float32":
        for p, c, got in zip(prompts, cfgs, results[1]):
            assert alone.generate([p], c)[0] == got


def test_a_burst_at_a_serving_width_gives_the_same_tokens_issued_ahead_or_not():
    """The tiny configurations never reach the kernels a served model runs on (the tcgen05 products and prompt
    attention, the streaming products, the decode ring): a model of a served width (heads of 128 in groups of 5,
    an odd vocabulary, six layers, random weights drawn on the device) takes 24 requests with prompts of 100 to
    1,500 tokens in 512-token steps, so that prompt portions run beside decoded tokens and captured steps
    follow.  Steps issued ahead or not, twice: the same tokens every time, all of them valid ids."""
    import random
    from microllm_rocm_b200 import GenerationConfig
    from microllm_rocm_b200.config import Qwen2Config
    from microllm_rocm_b200.engine.llm import LLM
    from microllm_rocm_b200.engine.loading import random_engine
    cfg = Qwen2Config.from_dict({
        "architectures": ["Qwen2ForCausalLM"], "hidden_size": 2560, "num_attention_heads": 20, "num_key_value_heads": 4,
        "head_dim": 128, "intermediate_size": 6912, "num_hidden_layers": 6, "vocab_size": 50021, "rms_norm_eps": 1e-6,
        "rope_theta": 1000000.0, "max_position_embeddings": 4096, "tie_word_embeddings": False})
    rng = random.Random(3)
    lens = [rng.randint(100, 1500) for _ in range(24)]
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in lens]
    engine = random_engine(cfg, seed=1, dtype="bfloat16", page_size=64, max_tokens=sum(lens) + 24 * 192, max_requests=24,
                           draw_on_device=True)
    results = []
    for ahead in (True, False, True):
        llm = LLM(engine, max_tokens_per_step=512, max_seqs=24)
        llm.lookahead = ahead
        results.append(llm.generate(prompts, GenerationConfig(max_new_tokens=48, temperature=0.0)))
        assert (llm.lookahead_steps > 10) == ahead and llm.graph_steps > 10
        assert llm.metrics()["cache"]["live_requests"] == 0
    assert all(len(r) == 48 and all(0 <= t < cfg.vocab_size for t in r) for r in results[0])
    assert results[0] == results[1] == results[2]


@pytest.mark.parametrize("key,pool,budget,seed,preempts", [("b", 320, 2048, 0, True), ("b", 400, 64, 7, False),
                                                          ("a", 0, 37, 1, False)])
def test_many_requests_through_a_tight_pool_equal_one_by_one(folders, key, pool, budget, seed, preempts):
    """Thirty requests of assorted lengths, greedy and sampled, submitted in bursts while the engine steps,
    through a pool so small that running requests are preempted and recomputed, with prompts cut by a small
    token budget: in fp32 every request must get exactly the tokens it gets alone in a roomy pool (which the
    tests above tie to the plain implementation), and the cache must end empty and consistent."""
    import random
    from microllm_rocm_b200 import GenerationConfig
    cfg = tiny_config(key)
    rng = random.Random(seed)
    cap = cfg.max_position_embeddings
    lens = [n for n in [1, 2, 3, 7, 15, 16, 17, 31, 33, 64, 100, 150] if n + 64 <= cap]
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(rng.choice(lens))] for _ in range(30)]
    cfgs = [GenerationConfig(max_new_tokens=rng.choice([1, 2, 5, 17, 40, 64]), temperature=0.0 if i % 3 else 0.8,
                             top_k=0 if i % 2 else 5, seed=i) for i in range(30)]
    roomy = llm_for(folders[key], "float32", max_tokens=8192)
    want = [roomy.generate([p], c)[0] for p, c in zip(prompts, cfgs)]
    tight = llm_for(folders[key], "float32", max_tokens=pool or cap + 64, max_tokens_per_step=budget)
    pending, ids = list(zip(prompts, cfgs)), []
    while pending or tight.has_work():
        for _ in range(rng.randrange(0, 4)):
            if pending:
                ids.append(tight.submit(*pending.pop(0)))
        if tight.has_work():
            tight.step()
    assert [list(tight.poll(i).generated) for i in ids] == want
    if budget < 100:
        assert tight.lookahead_steps > 0                  # prompts cut small: some steps were issued before their predecessors' tokens were read
    metrics = tight.metrics()
    assert metrics["cache"]["live_requests"] == 0
    if preempts:
        assert metrics["preemptions"] > 0               # the pool really was too small for the load
    tight.engine.cache.check()


def test_a_long_generation_from_a_short_prompt_is_cut_anew_as_it_grows(folders):
    """A captured decode step freezes how many CTAs share a sequence's keys.  Captured after a 3-token prompt
    that is one; 200 tokens later the step must have been planned and captured again (several CTAs), and the
    tokens must still be those of the kernel-by-kernel path."""
    from microllm_rocm_b200 import GenerationConfig
    key = "b"
    prompt = random_tokens(3, tiny_config(key).vocab_size, 11)
    cfg = GenerationConfig(max_new_tokens=200, temperature=0.0)
    want = llm_for(folders[key], "float32", max_tokens=1024, cuda_graphs=False).generate([prompt], cfg)[0]
    graphed = llm_for(folders[key], "float32", max_tokens=1024)
    assert graphed.generate([prompt], cfg)[0] == want             # (the fp32 attention kernel has no key split to re-plan)
    bf16 = llm_for(folders[key], "bfloat16", max_tokens=1024)
    got = bf16.generate([prompt], cfg)[0]
    assert bf16.graphs.captures >= 2, bf16.graphs.captures
    ref = plain_logits(folders[key], prompt + got[:-1], "bfloat16")[len(prompt) - 1:]
    for i, t in enumerate(got):                                    # each pick is a (near) maximum of the plain bf16 logits
        assert float(ref[i].max() - ref[i, t]) <= 0.03 * float(ref[i].abs().max()), (i, t)
