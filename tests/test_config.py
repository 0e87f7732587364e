"""Configuration: keys, defaults, validation, registry, and that no size hides in code."""
import json
import os

import pytest

from microllm_rocm_b200.config import (ConfigError, Qwen2Config, architecture_of, get_architecture, load_config,
                                       preset)
from microllm_rocm_b200.config.spec import ModelSpec, RunSpec
from tests.helpers import TINY


def test_reads_every_key_of_config_json():
    cfg = Qwen2Config.from_dict(TINY["b"])
    assert (cfg.vocab_size, cfg.hidden_size, cfg.num_hidden_layers) == (384, 192, 3)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_size) == (6, 2, 32)
    assert cfg.intermediate_size == 512 and cfg.rope_theta == 1e6 and cfg.rms_norm_eps == 1e-5
    assert not cfg.tie_word_embeddings
    assert [cfg.layer_window(l) for l in range(3)] == [None, 32, 32]


def test_optional_keys_default_and_head_dim_may_be_given():
    raw = dict(vocab_size=10, hidden_size=24, num_hidden_layers=1, num_attention_heads=3, intermediate_size=8,
               max_position_embeddings=16)
    cfg = Qwen2Config.from_dict(raw)
    assert cfg.num_key_value_heads == 3 and cfg.head_size == 8 and cfg.layer_window(0) is None
    assert Qwen2Config.from_dict(dict(raw, head_dim=16)).head_size == 16


def test_reference_fixture_parameter_count():
    # the reference pins Qwen2.5-0.5B at 494,032,768 parameters (tests/model/config_test.cpp:52-111)
    cfg = Qwen2Config.from_dict(dict(vocab_size=151936, hidden_size=896, num_hidden_layers=24, num_attention_heads=14,
                                     num_key_value_heads=2, intermediate_size=4864, max_position_embeddings=32768,
                                     rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=True))
    assert cfg.parameter_count() == 494032768


@pytest.mark.parametrize("change, word", [
    (dict(hidden_act="gelu"), "hidden_act"), (dict(model_type="llama"), "model_type"),
    (dict(use_mrope=True), "mrope"), (dict(rope_scaling={"type": "yarn"}), "rope_scaling"),
    (dict(num_key_value_heads=4), "multiple"), (dict(hidden_size=190), "divide"),
    (dict(rms_norm_eps=0.0), "rms_norm_eps"), (dict(rope_theta=-1.0), "rope_theta"),
    (dict(vocab_size=0), "vocab_size"), (dict(use_sliding_window=True, sliding_window=None), "sliding_window"),
    (dict(head_dim=15), "head_dim"),
])
def test_rejections(change, word):
    with pytest.raises(ConfigError, match=word):
        Qwen2Config.from_dict(dict(TINY["b"], **change))


def test_missing_required_key_is_named():
    raw = dict(TINY["a"])
    del raw["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        Qwen2Config.from_dict(raw)


def test_registry_chooses_by_architecture_name(tmp_path):
    cfg = preset("tiny-a")
    cfg.save(str(tmp_path))
    arch, loaded = load_config(str(tmp_path))
    assert arch.name == "Qwen2ForCausalLM" and loaded == cfg
    with pytest.raises(KeyError, match="LlamaForCausalLM"):
        architecture_of({"architectures": ["LlamaForCausalLM"]})
    # files written for the reference carry only model_type
    assert architecture_of({"model_type": "qwen2"}).name == "Qwen2ForCausalLM"


def test_spec_carries_every_size_per_layer():
    arch = get_architecture("Qwen2ForCausalLM")
    spec = arch.build_spec(Qwen2Config.from_dict(TINY["b"]))
    assert len(spec.layers) == 3 and [r.layer for r in spec.order] == [0, 1, 2]
    assert [l.mixer.params["window"] for l in spec.layers] == [None, 32, 32]
    m = spec.layers[1].mixer.params
    assert (m["num_heads"], m["num_kv_heads"], m["head_dim"], m["hidden_size"]) == (6, 2, 32, 192)
    assert spec.layers[0].feed_forward.params["intermediate_size"] == 512
    assert spec.layers[2].mixer_norm.params["eps"] == 1e-5 and spec.position.params["theta"] == 1e6
    assert spec.head.params["tied_to"] is None
    assert arch.build_spec(Qwen2Config.from_dict(TINY["a"])).head.params["tied_to"] == "model.embed_tokens.weight"


def test_order_is_data_and_is_checked():
    arch = get_architecture("Qwen2ForCausalLM")
    spec = arch.build_spec(Qwen2Config.from_dict(TINY["a"]))
    import dataclasses
    twice = dataclasses.replace(spec, order=[RunSpec(0), RunSpec(1), RunSpec(0), RunSpec(1, read_cache_of=1)])
    twice.validate()
    assert [twice.cache_name(i) for i in range(4)] == ["run0", "run1", "run2", "run1"]
    with pytest.raises(ValueError, match="earlier"):
        dataclasses.replace(spec, order=[RunSpec(0, read_cache_of=1), RunSpec(1)]).validate()
    with pytest.raises(ValueError, match="does not exist"):
        dataclasses.replace(spec, order=[RunSpec(5)]).validate()


def test_no_model_size_stands_in_the_package_code():
    """Sizes of the benchmark models may appear in the presets file only."""
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "microllm_rocm_b200")
    needles = ("151936", "152064", "8960", "18944", "13824")
    for folder, _, files in os.walk(root):
        if "_build" in folder:
            continue
        for name in files:
            if not name.endswith((".py", ".cu", ".cuh")) or name == "qwen2.py" and folder.endswith("config"):
                continue
            text = open(os.path.join(folder, name), encoding="utf-8").read()
            for n in needles:
                assert n not in text, f"{n} in {os.path.join(folder, name)}"
