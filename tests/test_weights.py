"""Weights: the safetensors container, binding by name, the one error that lists every
problem, dtype policy, random-weights mode."""
import json
import os
import struct

import pytest
import torch

from microllm_rocm_b200.config import Qwen2Config, get_architecture
from microllm_rocm_b200.parts import Runtime, build_model
from microllm_rocm_b200.weights import (SafetensorsError, SafetensorsFile, WeightLoadError, load_weights, save_file,
                                        write_random_model)
from microllm_rocm_b200.weights.safetensors import inspect_file, open_model_files
from tests.helpers import tiny_config
from tests.plain import qwen2_plain as plain

ARCH = get_architecture("Qwen2ForCausalLM")


def cpu_model(key, dtype=torch.float32):
    return build_model(ARCH.build_spec(tiny_config(key)), Runtime(torch.device("cpu"), dtype))


def rewrite(folder, edit):
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    edit(tensors)
    save_file(tensors, path)


def test_round_trip_all_float_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.randn(2, 2).to(torch.float16),
         "i": torch.arange(6, dtype=torch.int32).reshape(2, 3), "empty": torch.zeros(0, 4)}
    p = str(tmp_path / "x.safetensors")
    save_file(t, p, metadata={"k": "v"})
    f = SafetensorsFile(p)
    assert set(f.names()) == set(t)
    for n, v in t.items():
        assert f.tensor(n).dtype == v.dtype and torch.equal(f.tensor(n), v)
    # and the independent reader of the plain implementation agrees on the float tensors
    p2 = str(tmp_path / "y.safetensors")
    save_file({k: t[k] for k in "abc"}, p2)
    again = plain.read_safetensors(p2)
    for k in "abc":
        assert torch.equal(again[k], t[k].to(torch.float32))


def test_container_corruption_is_refused(tmp_path):
    p = str(tmp_path / "x.safetensors")
    save_file({"a": torch.randn(4, 4), "b": torch.randn(3)}, p)
    raw = open(p, "rb").read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])

    def write(h, payload=raw[8 + hlen:]):
        blob = json.dumps(h).encode()
        open(p, "wb").write(struct.pack("<Q", len(blob)) + blob + payload)

    open(p, "wb").write(raw[:-5])
    with pytest.raises(SafetensorsError):
        inspect_file(p)
    h = json.loads(json.dumps(header)); h["a"]["data_offsets"] = [0, 60]
    write(h)
    with pytest.raises(SafetensorsError, match="do not match shape"):
        inspect_file(p)
    h = json.loads(json.dumps(header)); h["b"]["data_offsets"] = [60, 72]; h["b"]["shape"] = [3]
    write(h)
    with pytest.raises(SafetensorsError, match="overlap|hole|cover"):
        inspect_file(p)
    h = json.loads(json.dumps(header)); h["a"]["dtype"] = "F8_E4M3"
    write(h)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        inspect_file(p)
    open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        inspect_file(p)
    blob = b'{"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}'
    open(p, "wb").write(struct.pack("<Q", len(blob)) + blob + b"\0\0\0\0")
    with pytest.raises(SafetensorsError, match="duplicate"):
        inspect_file(p)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_random_model(ARCH, tiny_config("b"), 1, str(tmp_path / "m"), "float32")

    def edit(t):
        del t["model.layers.1.self_attn.k_proj.bias"]
        del t["lm_head.weight"]
        t["model.layers.0.mlp.gate_proj.weight"] = torch.zeros(512, 100)
        t["model.layers.9.extra.weight"] = torch.zeros(2)
        t["model.norm.weight"] = torch.zeros(192, dtype=torch.int32)
    rewrite(folder, edit)
    model = cpu_model("b")
    with pytest.raises(WeightLoadError) as e:
        load_weights(model, folder)
    msg = str(e.value)
    for piece in ("model.layers.1.self_attn.k_proj.bias", "lm_head.weight", "model.layers.9.extra.weight",
                  "model.layers.0.mlp.gate_proj.weight expected [512, 192] got [512, 100]", "model.norm.weight is"):
        assert piece in msg, piece
    r = e.value.report
    assert len(r.missing) == 2 and len(r.unexpected) == 1 and len(r.wrong_shape) == 1 and len(r.wrong_dtype) == 1
    assert not model.bound, "a failed load must bind nothing"


def test_tied_head_tolerates_a_redundant_lm_head_and_non_strict_tolerates_extras(tmp_path):
    folder = write_random_model(ARCH, tiny_config("a"), 0, str(tmp_path / "m"), "float32")
    rewrite(folder, lambda t: t.update({"lm_head.weight": t["model.embed_tokens.weight"].clone()}))
    model = cpu_model("a")
    report = load_weights(model, folder)
    assert report.ignored == ["lm_head.weight"] and model.bound
    assert model.head.weight is model.embedding.table
    rewrite(folder, lambda t: t.update({"something.else": torch.zeros(1)}))
    with pytest.raises(WeightLoadError, match="something.else"):
        load_weights(cpu_model("a"), folder)
    assert "something.else" in load_weights(cpu_model("a"), folder, strict=False).ignored


@pytest.mark.parametrize("storage", ["float32", "bfloat16"])
@pytest.mark.parametrize("compute", [torch.float32, torch.bfloat16])
def test_dtype_policy(tmp_path, storage, compute):
    folder = write_random_model(ARCH, tiny_config("b"), 1, str(tmp_path / "m"), storage)
    model = cpu_model("b", compute)
    load_weights(model, folder)
    attn = model.blocks[0].mixer
    assert attn.w_qkv.dtype == compute and attn.w_o.dtype == compute and model.embedding.table.dtype == compute
    assert attn.b_qkv.dtype == torch.float32 and model.final_norm.weight.dtype == torch.float32
    assert attn.w_qkv.shape == ((6 + 2 * 2) * 32, 192) and model.blocks[0].feed_forward.w_gate_up.shape == (1024, 192)
    # values are the stored ones, rounded at most once
    stored = SafetensorsFile(os.path.join(folder, "model.safetensors")).tensor("model.layers.0.self_attn.o_proj.weight")
    assert torch.equal(attn.w_o, stored.to(compute))


def test_random_mode_is_seeded_and_has_the_stated_distributions(tmp_path):
    a = write_random_model(ARCH, tiny_config("b"), 5, str(tmp_path / "a"), "float32")
    b = write_random_model(ARCH, tiny_config("b"), 5, str(tmp_path / "b"), "float32")
    c = write_random_model(ARCH, tiny_config("b"), 6, str(tmp_path / "c"), "float32")
    fa, fb, fc = (SafetensorsFile(os.path.join(x, "model.safetensors")) for x in (a, b, c))
    assert all(torch.equal(fa.tensor(n), fb.tensor(n)) for n in fa.names())
    assert not torch.equal(fa.tensor("model.embed_tokens.weight"), fc.tensor("model.embed_tokens.weight"))
    w = fa.tensor("model.layers.0.mlp.up_proj.weight")
    assert abs(float(w.mean())) < 2e-3 and abs(float(w.std()) - 0.02) < 2e-3
    n = torch.cat([fa.tensor(k) for k in fa.names() if k.endswith("norm.weight")])
    assert abs(float(n.mean()) - 1.0) < 0.03 and abs(float(n.std()) - 0.1) < 0.03
    bias = fa.tensor("model.layers.2.self_attn.q_proj.bias")
    assert 0.01 < float(bias.std()) < 0.03
    cfg = json.load(open(os.path.join(a, "config.json")))
    assert cfg["architectures"] == ["Qwen2ForCausalLM"] and Qwen2Config.from_dict(cfg) == Qwen2Config.from_dict(
        dict(tiny_config("b").to_dict()))
    # 39 tensors: 12 per layer, embedding, final norm, head
    assert len(fa.names()) == 3 * 12 + 3


def test_random_values_are_the_documented_counter_function_of_seed_name_and_index():
    """An independent restatement with Python integers: SplitMix64's finaliser over key + GOLDEN * (3 i + j + 1),
    twelve 16-bit fields, (2 * sum - 12 * 65535) / 2^17, times the standard deviation."""
    import zlib
    from microllm_rocm_b200.parts.base import WeightSpec
    from microllm_rocm_b200.weights.random_init import draw
    M = (1 << 64) - 1

    def finalise(z):
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
        return z ^ (z >> 31)

    def value(seed, name, i):
        key = finalise((seed * 0x9E3779B97F4A7C15 + zlib.crc32(name.encode()) * 0x94D049BB133111EB + 0xBF58476D1CE4E5B9) & M)
        total = 0
        for j in range(3):
            word = finalise((key + 0x9E3779B97F4A7C15 * (3 * i + j + 1)) & M)
            total += sum((word >> (16 * f)) & 0xFFFF for f in range(4))
        return (2 * total - 12 * 65535) / 131072.0

    name = "model.layers.1.mlp.down_proj.weight"
    got = draw(WeightSpec((7, 13), "matrix", ("normal", 0.02)), 9, name, torch.device("cpu")).reshape(-1)
    want = torch.tensor([value(9, name, i) for i in range(91)], dtype=torch.float32) * 0.02
    assert torch.equal(got, want)
    ones = draw(WeightSpec((5,), "vector", ("one_plus_normal", 0.1)), 9, "model.norm.weight", torch.device("cpu"))
    assert torch.equal(ones, torch.tensor([value(9, "model.norm.weight", i) for i in range(5)], dtype=torch.float32) * 0.1 + 1.0)
    # neither the tensor's extent nor a chunk boundary changes an element's value
    longer = draw(WeightSpec((40, 13), "matrix", ("normal", 0.02)), 9, name, torch.device("cpu")).reshape(-1)
    assert torch.equal(longer[:91], got)
    big = draw(WeightSpec((1 << 16,), "matrix", ("normal", 1.0)), 1, "t", torch.device("cpu"))
    assert abs(float(big.mean())) < 0.02 and abs(float(big.std()) - 1.0) < 0.02 and float(big.abs().max()) > 3.5


@pytest.mark.gpu
def test_a_model_drawn_on_the_device_holds_the_bits_of_the_written_folder(tmp_path):
    from microllm_rocm_b200.parts.base import WeightSpec
    from microllm_rocm_b200.weights import random_init
    folder = write_random_model(ARCH, tiny_config("b"), 5, str(tmp_path / "m"), "bfloat16")
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    declared = build_model(ARCH.build_spec(tiny_config("b")), Runtime(torch.device("cpu"), torch.float32)).expected_tensors()
    on_device = random_init.random_tensors(declared, 5, torch.device("cuda"), torch.bfloat16)
    assert set(on_device) == set(f.names())
    for name in f.names():
        assert torch.equal(on_device[name].cpu(), f.tensor(name)), name
    # across a chunk boundary of the generator too
    spec = WeightSpec((random_init._CHUNK + 1000,), "matrix", ("normal", 0.02))
    a = random_init.draw(spec, 2, "x", torch.device("cuda")).cpu()
    b = random_init.draw(spec, 2, "x", torch.device("cpu"))
    assert torch.equal(a, b)


def test_sharded_folder_through_index(tmp_path):
    folder = write_random_model(ARCH, tiny_config("a"), 0, str(tmp_path / "m"), "float32")
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    names = f.names()
    half = len(names) // 2
    save_file({n: f.tensor(n).clone() for n in names[:half]}, os.path.join(folder, "s1.safetensors"))
    save_file({n: f.tensor(n).clone() for n in names[half:]}, os.path.join(folder, "s2.safetensors"))
    os.remove(os.path.join(folder, "model.safetensors"))
    index = {"weight_map": {n: ("s1.safetensors" if i < half else "s2.safetensors") for i, n in enumerate(names)}}
    json.dump(index, open(os.path.join(folder, "model.safetensors.index.json"), "w"))
    assert load_weights(cpu_model("a"), folder).ok
    index["weight_map"][names[0]] = "../s1.safetensors"
    json.dump(index, open(os.path.join(folder, "model.safetensors.index.json"), "w"))
    with pytest.raises(SafetensorsError, match="leaves the model folder"):
        open_model_files(folder)


@pytest.mark.gpu
def test_a_benchmark_size_folder_streams_onto_the_device_bit_for_bit(tmp_path):
    """The Qwen2.5-1.5B shape written as a bf16 model folder (3.1 GB) and loaded back through the streaming
    loader: pieces of the mapped file go through pinned staging buffers into the rows of the FUSED device
    tensors (q, k, v under one another; gate over up) without a second copy on the device.  Tensors are
    compared bit for bit with the file as a minimal reader sees it, and the time is printed."""
    import time
    from microllm_rocm_b200.config import find_preset
    from microllm_rocm_b200.engine.loading import load_engine
    from microllm_rocm_b200.weights import safetensors as st
    from microllm_rocm_b200.parts.base import Runtime
    from microllm_rocm_b200.parts.build import build_model
    from microllm_rocm_b200.weights.random_init import random_tensors
    arch, cfg = find_preset("qwen2.5-1.5b")
    folder = str(tmp_path / "model")
    import os
    os.makedirs(folder)
    cfg.save(folder)
    # drawn on the device (a CPU draw of 1.5 G values takes a minute), written in the checkpoint's naming
    declared = build_model(arch.build_spec(cfg), Runtime(torch.device("cpu"), torch.float32)).expected_tensors()
    t0 = time.perf_counter()
    st.save_file(random_tensors(declared, 3, torch.device("cuda"), torch.bfloat16), os.path.join(folder, "model.safetensors"))
    wrote = time.perf_counter() - t0
    torch.cuda.empty_cache()
    before = torch.cuda.memory_allocated()
    engine = load_engine(folder, dtype="bfloat16", page_size=64, max_tokens=256, max_requests=2)
    report = engine.load_report
    size = os.path.getsize(os.path.join(folder, "model.safetensors"))
    print(f"wrote {size / 1e9:.2f} GB in {wrote:.1f} s; loaded {report.bytes_read / 1e9:.2f} GB in {report.load_ms:.0f} ms "
          f"({report.bytes_read / 1e6 / report.load_ms:.2f} GB/s)")
    assert report.bytes_read == sum(t.end - t.begin for t in st.SafetensorsFile(os.path.join(folder, "model.safetensors")).infos.values())
    # device memory holds the weights once (plus the small cache of this engine and staging)
    assert torch.cuda.memory_allocated() - before < report.bytes_read * 1.05 + (256 << 20)
    f = st.SafetensorsFile(os.path.join(folder, "model.safetensors"))
    mixer, mlp = engine.model.blocks[17].mixer, engine.model.blocks[17].feed_forward
    q, kv = cfg.num_attention_heads * cfg.head_size, cfg.num_key_value_heads * cfg.head_size
    p = "model.layers.17."
    assert torch.equal(mixer.w_qkv[:q].cpu(), f.tensor(p + "self_attn.q_proj.weight"))
    assert torch.equal(mixer.w_qkv[q:q + kv].cpu(), f.tensor(p + "self_attn.k_proj.weight"))
    assert torch.equal(mixer.w_qkv[q + kv:].cpu(), f.tensor(p + "self_attn.v_proj.weight"))
    assert torch.equal(mixer.b_qkv[q:q + kv].cpu(), f.tensor(p + "self_attn.k_proj.bias").float())
    assert torch.equal(mlp.w_gate_up[cfg.intermediate_size:].cpu(), f.tensor(p + "mlp.up_proj.weight"))
    assert torch.equal(mlp.w_down.cpu(), f.tensor(p + "mlp.down_proj.weight"))
    assert torch.equal(engine.model.embedding.table[100000:100003].cpu(), f.tensor("model.embed_tokens.weight")[100000:100003])
    assert engine.model.head.weight.data_ptr() == engine.model.embedding.table.data_ptr()         # tied: one table
